"""Plain, slow restatement of the Nezolorn decoder for tests: whole sequences, token by token
where the design is recurrent, no cache, no batching, one function for each mechanism.

It shares no code with the package under test.  Weights come in as a ``{tensor name:
torch.Tensor}`` dictionary with the checkpoint's names, sizes and constants as a plain ``dict``
with config.json's keys.  Arithmetic runs in ``compute`` (float64 by default: the oracle is
then tighter than either of the engine's number formats).

Notation: ``x`` the residual stream ``[T, width]``, ``h`` a mixer's or feed-forward's input,
``p`` a position (counted from 0), ``H`` heads, ``G`` key/value heads.
"""
from __future__ import annotations

import math

import torch

F = torch.nn.functional


def lin(x, w):
    """``y = x W^T`` for a weight stored ``[out, in]``."""
    return x @ w.to(x.dtype).t()


def layer_norm(x, weight, eps):
    """Mean removed, divided by ``sqrt(var + eps)`` (var = mean squared deviation), times a weight; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * weight.to(x.dtype)


def unit_rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def embed(w, cfg, tokens, compute):
    """Token row times a scale, plus a row of a hashed table of (previous token, token) pairs;
    the first token of a sequence takes the table's last row."""
    e = cfg["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(compute)[ids] * e["scale"]
    if e.get("bigram"):
        b = e["bigram"]
        rows = [b["buckets"]] + [(int(tokens[t - 1]) * b["mul_prev"] + int(tokens[t]) * b["mul_cur"]) % b["buckets"] for t in range(1, len(tokens))]
        x = x + w["bigram"].to(compute)[torch.tensor(rows, dtype=torch.long)]
    return x


def rotary_frequencies(rot, compute):
    """``f_i = base^(-2i/dims)``, then the three-band rescaling by wavelength (long waves slowed
    by ``factor``, short ones kept, a linear blend between)."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=compute)
    f = torch.tensor(float(rot["base"]), dtype=compute) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = torch.tensor(out, dtype=compute)
    return f


def rotate(x, positions, rot, compute):
    """Rotates the first ``dims`` elements of every head of ``x [T, heads, dim]``: element ``i`` pairs
    with ``i + dims/2``; the rest pass unchanged."""
    dims = rot["dims"]
    r = dims // 2
    f = rotary_frequencies(rot, compute)
    ang = torch.as_tensor(positions, dtype=compute)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :r], x[..., r:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def windowed_pooled_attention(q, k, v, window, pool, scale):
    """``q [T, H, d]``, ``k [T, G, d]`` (as the cache holds them), ``v [T, G, dv]``.  Query ``i`` sees the
    keys ``j`` with ``0 <= i - j < window`` and, for every block ``b`` of ``pool`` tokens with
    ``b pool + pool - 1 <= i - window``, the block's mean key and mean value; one softmax over both."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        nblocks = max(0, (i - window + 1) // pool) if i - window >= 0 else 0
        for h in range(H):
            g = h // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(dim=0) for b in range(nblocks)] + [k[j, g] for j in range(lo, i + 1)]
            vals = [v[b * pool:(b + 1) * pool, g].mean(dim=0) for b in range(nblocks)] + [v[j, g] for j in range(lo, i + 1)]
            K, V = torch.stack(keys), torch.stack(vals)
            p = torch.softmax((K @ q[i, h]) * scale, dim=0)
            out[i, h] = p @ V
    return out


def left_mixer(w, pre, m, h, eps, compute, store=None):
    """Grouped-query attention whose values are the keys before rotation."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = lin(h, w[pre + "q"]).view(T, H, d)
    k = lin(h, w[pre + "k"]).view(T, G, d)
    v = k
    pos = list(range(T))
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"], compute), rotate(k, pos, m["rot"], compute)
    if store is not None:                    # what a cache in a narrower format would hold
        k, v = store(k), store(v)
    o = windowed_pooled_attention(q, k, v, m["mask"]["size"], m["mask"].get("pool") or 10 ** 9, m["scale"])     # no pool: no block is ever complete
    return lin(o.reshape(T, -1), w[pre + "o"])


def matrix_memory(q, k, v, ig, fg):
    """One head of the gated matrix memory: ``q, k [T, d]``, ``v [T, dv]``, log gates ``ig, fg [T]``.
    ``m_t = max(fg + m, ig)`` from ``m_0 = 0``; ``S = exp(fg + m - m_t) S + exp(ig - m_t) k v^T``, ``n``
    likewise with ``k``; ``o = S^T q / (max(|n . q|, exp(-m_t)) + 1e-6)``."""
    T, d = k.shape
    S = torch.zeros((d, v.shape[1]), dtype=q.dtype)
    n = torch.zeros(d, dtype=q.dtype)
    m = torch.zeros((), dtype=q.dtype)
    out = []
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a, b = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        den = torch.maximum(torch.abs(n @ q[t]), torch.exp(-m)) + 1e-6
        out.append((S.t() @ q[t]) / den)
    return torch.stack(out)


def right_mixer(w, pre, m, h, eps):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (lin(h, w[pre + "q"]) * d ** -0.5).view(T, H, d)
    k = lin(h, w[pre + "k"]).view(T, H, d)
    v = lin(h, w[pre + "v"]).view(T, H, dv)
    ig = cap * torch.tanh((lin(h, w[pre + "i"]) + w[pre + "i.b"].to(h.dtype)) / cap)
    fg = F.logsigmoid(cap * torch.tanh((lin(h, w[pre + "f"]) + w[pre + "f.b"].to(h.dtype)) / cap))
    o = torch.stack([matrix_memory(q[:, j], k[:, j], v[:, j], ig[:, j], fg[:, j]) for j in range(H)], dim=1)
    o = unit_rms(o, eps).reshape(T, -1) * w[pre + "norm"].to(h.dtype) * torch.sigmoid(lin(h, w[pre + "g"]))
    return lin(o, w[pre + "o"])


def parallel_mixer(w, pre, m, h, eps, compute, store=None):
    return m["left_scale"] * left_mixer(w, pre + "left.", m["left"], h, eps, compute, store) + m["right_scale"] * right_mixer(w, pre + "right.", m["right"], h, eps)


def delta_memory(r, k, v, decay, rate):
    """One head of the generalised delta rule, all ``[T, d]``: with ``u = k / sqrt(sum k^2 + 1e-6)``,
    ``S = diag(decay) S - (rate * u) (u^T S) + k v^T`` (both terms from the old ``S``), ``o = S^T r``."""
    T, d = k.shape
    S = torch.zeros((d, d), dtype=r.dtype)
    out = []
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum() + 1e-6)
        S = decay[t][:, None] * S - torch.outer(rate[t] * u, u @ S) + torch.outer(k[t], v[t])
        out.append(S.t() @ r[t])
    return torch.stack(out)


def general_delta_mixer(w, pre, m, h, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r, k, v = (lin(h, w[pre + n]).view(T, H, d) for n in ("r", "k", "v"))
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lin(torch.tanh(lin(h, w[pre + "w1"])), w[pre + "w2"]) + w[pre + "w0"].to(h.dtype))).view(T, H, d)
    rate = torch.sigmoid(lin(h, w[pre + "a"]) + w[pre + "a.b"].to(h.dtype)).view(T, H, d)
    o = torch.stack([delta_memory(r[:, j], k[:, j], v[:, j], decay[:, j], rate[:, j]) for j in range(H)], dim=1)
    o = unit_rms(o, eps).reshape(T, -1) * w[pre + "norm"].to(h.dtype) * torch.sigmoid(lin(h, w[pre + "g"]))
    return lin(o, w[pre + "o"])


def dense_ff(w, pre, h):
    return lin(F.silu(lin(h, w[pre + "gate"])) * lin(h, w[pre + "up"]), w[pre + "down"])


def forward(w, cfg, tokens, compute=torch.float64, store=None, layers_out=None):
    """Logits ``[T, vocab]`` of one whole sequence.  ``layers_out``: a list that receives the residual
    stream after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embed(w, cfg, tokens, compute)
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "parallel":
            y = parallel_mixer(w, pre + "mix.", layer["mixer"], h, eps, compute, store)
        elif layer["type"] == "general_delta":
            y = general_delta_mixer(w, pre + "mix.", layer["mixer"], h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * y
        if layer.get("mlp"):
            x = x + mult * dense_ff(w, pre + "mlp.", layer_norm(x, w[pre + "norm2"], eps))
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(layer_norm(x, w["final.norm"], eps), w["head"])


def random_weights(cfg, seed, std=0.08, norm_std=0.1, bias_std=0.5):
    """Seeded bfloat16 tensors with the checkpoint's names for a configuration (``decay_rank`` must be in the
    configuration of a delta-rule layer)."""
    g = torch.Generator().manual_seed(seed)

    def mat(*shape, s=std):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def gain(n):
        return (1.0 + torch.randn(n, generator=g) * norm_std).to(torch.bfloat16)

    W, V = cfg["width"], cfg["vocab"]
    w = {"embed": mat(V, W, s=1.0), "head": mat(V, W), "final.norm": gain(W)}
    if cfg["embedding"].get("bigram"):
        w["bigram"] = mat(cfg["embedding"]["bigram"]["buckets"] + 1, W, s=0.5)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = gain(W)
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            w[p + "mix.left.q"], w[p + "mix.left.k"] = mat(a["heads"] * a["dim"], W, s=2 * std), mat(a["kv_heads"] * a["dim"], W, s=2 * std)
            w[p + "mix.left.o"] = mat(W, a["heads"] * a["dim"])
            H, dk, dv = b["heads"], b["dim"], b["vdim"]
            for n, rows in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H)):
                w[p + "mix.right." + n] = mat(rows, W)
            w[p + "mix.right.i.b"], w[p + "mix.right.f.b"] = mat(H, s=bias_std), (2.0 + torch.randn(H, generator=g) * bias_std).to(torch.bfloat16)
            w[p + "mix.right.norm"], w[p + "mix.right.o"] = gain(H * dv), mat(W, H * dv)
        else:
            n, R = m["heads"] * m["dim"], m["decay_rank"]
            for name in ("r", "k", "v", "g", "a"):
                w[p + "mix." + name] = mat(n, W)
            w[p + "mix.a.b"], w[p + "mix.w0"] = mat(n, s=bias_std), mat(n, s=bias_std)
            w[p + "mix.w1"], w[p + "mix.w2"] = mat(R, W), mat(n, R, s=0.5)
            w[p + "mix.norm"], w[p + "mix.o"] = gain(n), mat(W, n)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = gain(W)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
    return w
