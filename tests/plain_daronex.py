"""A plain, slow implementation of the Daronex decoder in float64 on the CPU, one function per mechanism, written from
the design's equations and sharing no code with the engine.  A whole sequence at a time, no cache, no batching.

Notation: ``h`` is a sublayer's input ``[T, width]``; weights are stored ``[out, in]`` and applied as ``h @ W.T``;
positions count from 0.
"""
import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layers' norm: unit root mean square, then a gain stored as its distance from one."""
    return rms(x, eps) * (1.0 + w)


def rotate(x, positions, base, dims, interleaved):
    """Rotates the first ``dims`` elements of the last axis of ``x [T, ..., D]``: pair ``i`` is ``(2i, 2i + 1)`` when
    ``interleaved`` else ``(i, i + dims / 2)``, its angle ``position * base^(-2i / dims)``."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle[:, None]
    c, s = torch.cos(angle), torch.sin(angle)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def visible(T, window):
    """[query, key] -> bool: every earlier key and the query's own, or the last ``window`` of them."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) if window is None else ((i - j >= 0) & (i - j < window))


def latent_pair(h, w, p, m, eps, interleaved):
    """What a layer keeps of its tokens: the normed latent and the shared rotated key part."""
    T, r = h.shape[0], m["kv_rank"]
    both = h @ w[p + "dkv"].T
    c = rms(both[:, :r], eps) * w[p + "dkv.norm"]
    kr = both[:, r:]
    if m["rot_dim"] > 0:
        kr = rotate(kr, torch.arange(T), m["rot"]["base"], m["rot"]["dims"], interleaved)
    return c, kr


def latent_attention(h, w, p, m, eps, interleaved, window, gated, pair=None, probs=None):
    """``pair``: another layer's (latent, rotated part) to use instead of projecting this layer's own.  ``probs``: a
    list that receives the attention weights ``[heads, query, key]``."""
    T, H, d, rd, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + rd)
    qn, qr = q[..., :d], q[..., d:]
    if rd > 0:
        qr = rotate(qr, torch.arange(T), m["rot"]["base"], m["rot"]["dims"], interleaved)
    c, kr = pair if pair is not None else latent_pair(h, w, p, m, eps, interleaved)
    kn = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, vd)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    s = s.masked_fill(~visible(T, window)[None], -math.inf)
    a = torch.softmax(s, dim=-1)
    if probs is not None:
        probs.append(a)
    o = torch.einsum("hij,jhv->ihv", a, v).reshape(T, H * vd)
    if gated:
        o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, (c, kr)


def gla_recurrence(q, k, v, alpha, state=None):
    """``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head; q, k, alpha ``[T, H, dk]``, v ``[T, H, dv]``."""
    T, H, dk = q.shape
    S = torch.zeros((H, dk, v.shape[-1]), dtype=F) if state is None else state.clone()
    o = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gla(h, w, p, m, eps):
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, vd)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).reshape(T, H, d)
    o, _ = gla_recurrence(q, k, v, alpha)
    o = (rms(o, eps) * w[p + "norm"]).reshape(T, H * vd)
    g = h @ w[p + "g"].T
    return (o * (g * torch.sigmoid(g))) @ w[p + "o"].T


def feed_forward(h, w, p):
    a = torch.relu(h @ w[p + "up"].T)
    return (a * a) @ w[p + "down"].T


def forward(w, cfg, tokens, layers_out=None, probs_out=None):
    """Logits ``[T, vocab]`` of one sequence; ``w``: name -> tensor (any float type)."""
    w = {k: t.to(F) for k, t in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))]
    pairs = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        probs = [] if probs_out is not None else None
        if kind == "latent_attention":
            y, pairs[i] = latent_attention(x, w, p, m, eps, True, None, False, pair=pairs[m["kv_from"]] if m.get("kv_from") is not None else None, probs=probs)
        elif kind == "latent_attention_2":
            y, pairs[i] = latent_attention(x, w, p, m, eps, False, m["mask"]["size"], True, pair=pairs[m["kv_from"]] if m.get("kv_from") is not None else None,
                                           probs=probs)
        elif kind == "gla":
            y = gla(x, w, p, m, eps)
        else:
            raise ValueError(kind)
        if probs_out is not None:
            probs_out.append(probs[0] if probs else None)
        x = x + offset_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + offset_norm(feed_forward(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (offset_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)


def tensor_shapes(cfg):
    """name -> shape of every tensor of a model of this configuration."""
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],), "head": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        out[f"l{i}.norm1"] = (W,)
        if layer["type"] == "gla":
            H, d, vd, r = m["heads"], m["dim"], m["vdim"], m["decay_rank"]
            out.update({p + "q": (H * d, W), p + "k": (H * d, W), p + "v": (H * vd, W), p + "g": (H * vd, W), p + "o": (W, H * vd), p + "norm": (vd,),
                        p + "a1": (r, W), p + "a2": (H * d, r), p + "a2.b": (H * d,)})
        else:
            H, d, rd, vd, qr, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out.update({p + "dq": (qr, W), p + "dq.norm": (qr,), p + "uq": (H * (d + rd), qr), p + "uk": (H * d, r), p + "uv": (H * vd, r),
                        p + "o": (W, H * vd)})
            if m.get("kv_from") is None:
                out.update({p + "dkv": (r + rd, W), p + "dkv.norm": (r,)})
            if layer["type"] == "latent_attention_2":
                out[p + "g"] = (H * vd, W)
        if layer.get("mlp") is not None:
            out.update({f"l{i}.norm2": (W,), f"l{i}.mlp.up": (layer["mlp"]["ff"], W), f"l{i}.mlp.down": (W, layer["mlp"]["ff"])})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Seeded bfloat16 weights: matrices with a spread of ``gain / sqrt(inputs)`` (activations stay of order one),
    plain norm weights around one, the layers' norm weights and biases around zero."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        if name == "embed":
            x = x * 1.0
        elif name.endswith(".b"):
            x = x * 0.5 + 1.0            # the decay's bias: decays mostly near one, as a trained model's
        elif name.endswith("dq.norm") or name.endswith("dkv.norm") or name.endswith("mix.norm"):
            x = 1.0 + 0.1 * x
        elif len(shape) == 1:
            x = 0.1 * x                  # stored around zero
        else:
            x = x * (gain / math.sqrt(shape[1]))
        out[name] = x.to(torch.bfloat16)
    return out
