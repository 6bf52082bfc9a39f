"""Mixers that carry a matrix state per request and head from token to token, in 32-bit.

``matrix_memory`` (the matrix memory of the xLSTM family, mLSTM): per head ``q, k [dk]``, ``v [dv]`` and two log gates
``i = cap * tanh((W_i h + b_i) / cap)``, ``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``; with the running maximum
``m' = max(f + m, i)`` (``m`` starts at 0): ``S = exp(f + m - m') S + exp(i - m') k v^T``, ``n`` likewise with ``k``,
``o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)``, ``q`` scaled by ``dk^(-1/2)``.

``delta_rule`` (the generalised delta rule): per head ``r, k, v [d]``, a decay per key channel
``w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0))`` and a removal rate ``a = sigmoid(W_a h + b_a)``; with the unit key
``u = k / sqrt(sum k^2 + 1e-6)``: ``S = diag(w) S - (a * u)(u^T S) + k v^T`` (both terms read the old ``S``), ``o = S^T r``.

``gated_linear_attention`` (gated linear attention with a decay per key channel): per head ``q, k [dk]``, ``v [dv]`` and the
decay ``a = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)``: ``S = diag(a) S + k v^T``, ``o = S^T q``, ``q`` scaled by ``dk^(-1/2)``; its
gate is ``silu(W_g h)`` and its norm weight has one head's size and is shared by the heads.

All end alike: each head's ``o`` divided by its root mean square, times a weight over all heads, times
a gate of ``W_g h`` (a sigmoid unless said otherwise), then the output projection.  All projections of the input are one fused product with a 32-bit result
(what enters the recurrence is never rounded to 16 bits); the state lives in the request's slot of the cache manager.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import StateCacheNeed
from ..weights.loader import WeightDecl
from .base import Mixer
from .linear import Linear
from .registry import register_part

_TILE = 8     # value columns of the narrowest tile of the scan kernel, each of which keeps its own n and m (csrc/recurrence.cu)


class _Recurrent(Mixer):
    graph_safe = True
    gate = "sigmoid"       # the output gate's activation

    #: (relative tensor name, rows as a function of the sizes) of the projections that are fused, in column order
    def _fused_names(self):
        raise NotImplementedError

    def _bind_common(self, tensors, fused_names, out_name):
        p = self.prefix
        ws = [tensors[p + n] for n in fused_names]
        if len({t.dtype for t in ws}) > 1:
            ws = [t.float() for t in ws]
        self.fused = Linear(torch.cat(ws, dim=0).contiguous(), self.ctx.dtype)
        self.o = Linear(tensors[p + out_name], self.ctx.dtype)
        self.norm_weight = tensors[p + "norm"].float().contiguous()

    def _finish(self, o, proj, gate_offset, heads, dv):
        y = torch.empty(o.shape, dtype=self.ctx.dtype, device=o.device)
        kernels.gated_head_norm(o, proj, gate_offset, self.norm_weight, y, heads, dv, self.eps, gate=self.gate)
        return self.o(y, defer=self.defer_output, out_dtype=self.output_dtype)


@register_part("matrix_memory")
class MatrixMemory(_Recurrent):
    """params: ``hidden_size``, ``heads``, ``dim`` (q/k size a head), ``vdim`` (value size a head), ``gate_cap``, ``eps``
    (of the per-head norm), ``prefix``.  Tensors: ``q, k [heads dim, hidden]``, ``v, g [heads vdim, hidden]``,
    ``i, f [heads, hidden]`` with biases ``i.b, f.b [heads]``, ``norm [heads vdim]``, ``o [hidden, heads vdim]``."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.heads = int(params["hidden_size"]), int(params["heads"])
        self.dk, self.dv = int(params["dim"]), int(params["vdim"])
        self.cap, self.eps = float(params["gate_cap"]), float(params["eps"])
        if not self.cap > 0.0 or min(self.hidden, self.heads, self.dk, self.dv) <= 0:
            raise ValueError("matrix_memory: sizes and the gates' cap must be positive")
        self.prefix = params.get("prefix", "")
        H, dk, dv = self.heads, self.dk, self.dv
        self.offsets = (0, H * dk, 2 * H * dk, 2 * H * dk + 2 * H * dv, 2 * H * dk + 2 * H * dv + H)      # q, k, v, i, f
        self.gate_offset = 2 * H * dk + H * dv
        self.record = (dk * dv + -(-dv // _TILE) * (dk + 1) + 3) // 4 * 4
        self.fused = self.o = self.norm_weight = self.bias_i = self.bias_f = None

    def weight_decls(self):
        p, H, dk, dv, W = self.prefix, self.heads, self.dk, self.dv, self.hidden
        return [WeightDecl(p + "q", (H * dk, W)), WeightDecl(p + "k", (H * dk, W)), WeightDecl(p + "v", (H * dv, W)), WeightDecl(p + "g", (H * dv, W)),
                WeightDecl(p + "o", (W, H * dv)), WeightDecl(p + "norm", (H * dv,), init="one_plus_normal"), WeightDecl(p + "i", (H, W)),
                WeightDecl(p + "i.b", (H,)), WeightDecl(p + "f", (H, W)), WeightDecl(p + "f.b", (H,))]

    def bind(self, tensors):
        self._bind_common(tensors, ("q", "k", "v", "g", "i", "f"), "o")
        self.bias_i = tensors[self.prefix + "i.b"].float().contiguous()
        self.bias_f = tensors[self.prefix + "f.b"].float().contiguous()

    def modules(self):
        return ["recurrence"] + self.fused.modules() + self.o.modules()

    def linears(self):
        return [self.fused, self.o]

    def cache_need(self):
        return StateCacheNeed((self.heads * self.record,), "float32")

    def forward(self, x, batch, cache):
        proj = self.fused(x, out_dtype=torch.float32)
        o = torch.empty((x.shape[0], self.heads * self.dv), dtype=torch.float32, device=x.device)
        kernels.mlstm_scan(proj, self.offsets, self.bias_i, self.bias_f, cache.state, batch.q_start, batch.state_slot, batch.num_seqs, o,
                           self.heads, self.dk, self.dv, self.dk ** -0.5, self.cap, status=batch.status,
                           longest=1 if batch.one_token_each else batch.num_tokens)
        return self._finish(o, proj, self.gate_offset, self.heads, self.dv)


@register_part("delta_rule")
class DeltaRule(_Recurrent):
    """params: ``hidden_size``, ``heads``, ``dim`` (key, value and receptance size a head), ``decay_rank`` (inner size of
    the decay's two-step projection), ``eps``, ``prefix``.  Tensors: ``r, k, v, g, a [heads dim, hidden]``, ``a.b``,
    ``w1 [rank, hidden]``, ``w2 [heads dim, rank]``, ``w0``, ``norm [heads dim]``, ``o [hidden, heads dim]``."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.heads, self.d = int(params["hidden_size"]), int(params["heads"]), int(params["dim"])
        self.rank, self.eps = int(params["decay_rank"]), float(params["eps"])
        if min(self.hidden, self.heads, self.d, self.rank) <= 0:
            raise ValueError("delta_rule: sizes must be positive")
        self.prefix = params.get("prefix", "")
        n = self.heads * self.d
        self.offsets = (0, n, 2 * n, 4 * n)       # r, k, v, a
        self.gate_offset, self.rank_offset = 3 * n, 5 * n
        self.fused = self.w2 = self.o = self.norm_weight = self.bias_a = self.decay_offset = None

    def weight_decls(self):
        p, n, W, R = self.prefix, self.heads * self.d, self.hidden, self.rank
        return ([WeightDecl(p + name, (n, W)) for name in ("k", "v", "g", "a")]
                + [WeightDecl(p + "a.b", (n,)), WeightDecl(p + "w1", (R, W)), WeightDecl(p + "w2", (n, R)), WeightDecl(p + "w0", (n,)),
                   WeightDecl(p + "norm", (n,), init="one_plus_normal"), WeightDecl(p + "o", (W, n)), WeightDecl(p + "r", (n, W))])

    def bind(self, tensors):
        self._bind_common(tensors, ("r", "k", "v", "g", "a", "w1"), "o")
        self.w2 = Linear(tensors[self.prefix + "w2"], self.ctx.dtype)
        self.bias_a = tensors[self.prefix + "a.b"].float().contiguous()
        self.decay_offset = tensors[self.prefix + "w0"].float().contiguous()

    def modules(self):
        return ["recurrence"] + self.fused.modules() + self.w2.modules() + self.o.modules()

    def linears(self):
        return [self.fused, self.w2, self.o]

    def cache_need(self):
        return StateCacheNeed((self.heads * self.d * self.d,), "float32")

    def forward(self, x, batch, cache):
        proj = self.fused(x, out_dtype=torch.float32)
        inner = torch.empty((x.shape[0], self.rank), dtype=self.ctx.dtype, device=x.device)
        kernels.tanh_cols(proj, self.rank_offset, self.rank, inner)
        decay_pre = self.w2(inner, out_dtype=torch.float32)
        o = torch.empty((x.shape[0], self.heads * self.d), dtype=torch.float32, device=x.device)
        kernels.delta_scan(proj, self.offsets, decay_pre, self.bias_a, self.decay_offset, cache.state, batch.q_start, batch.state_slot,
                           batch.num_seqs, o, self.heads, self.d, status=batch.status, longest=1 if batch.one_token_each else batch.num_tokens)
        return self._finish(o, proj, self.gate_offset, self.heads, self.d)


@register_part("gated_linear_attention")
class GatedLinearAttention(_Recurrent):
    """params: ``hidden_size``, ``heads``, ``dim`` (q/k size a head), ``vdim`` (value size a head), ``tau`` (the decay's
    temperature), ``decay_rank`` (inner size of the decay's two-step projection), ``eps`` (of the per-head norm), ``prefix``.
    Tensors: ``q, k [heads dim, hidden]``, ``v, g [heads vdim, hidden]``, ``a1 [rank, hidden]``, ``a2 [heads dim, rank]``,
    ``a2.b [heads dim]``, ``norm [vdim]`` (one head's, shared), ``o [hidden, heads vdim]``."""

    gate = "silu"

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.heads = int(params["hidden_size"]), int(params["heads"])
        self.dk, self.dv, self.rank = int(params["dim"]), int(params["vdim"]), int(params["decay_rank"])
        self.tau, self.eps = float(params["tau"]), float(params["eps"])
        if not self.tau > 0.0 or min(self.hidden, self.heads, self.dk, self.dv, self.rank) <= 0:
            raise ValueError("gated_linear_attention: sizes and tau must be positive")
        self.prefix = params.get("prefix", "")
        H, dk, dv = self.heads, self.dk, self.dv
        self.offsets = (0, H * dk, 2 * H * dk)                       # q, k, v
        self.gate_offset, self.rank_offset = 2 * H * dk + H * dv, 2 * H * dk + 2 * H * dv
        self.fused = self.a2 = self.o = self.norm_weight = self.decay_bias = None

    def weight_decls(self):
        p, H, dk, dv, W, R = self.prefix, self.heads, self.dk, self.dv, self.hidden, self.rank
        return [WeightDecl(p + "q", (H * dk, W)), WeightDecl(p + "k", (H * dk, W)), WeightDecl(p + "v", (H * dv, W)), WeightDecl(p + "g", (H * dv, W)),
                WeightDecl(p + "o", (W, H * dv)), WeightDecl(p + "norm", (dv,), init="one_plus_normal"), WeightDecl(p + "a1", (R, W)),
                WeightDecl(p + "a2", (H * dk, R)), WeightDecl(p + "a2.b", (H * dk,))]

    def bind(self, tensors):
        self._bind_common(tensors, ("q", "k", "v", "g", "a1"), "o")
        self.norm_weight = self.norm_weight.repeat(self.heads).contiguous()      # one head's weight, for every head
        self.a2 = Linear(tensors[self.prefix + "a2"], self.ctx.dtype)
        self.decay_bias = tensors[self.prefix + "a2.b"].float().contiguous()

    def modules(self):
        return ["recurrence"] + self.fused.modules() + self.a2.modules() + self.o.modules()

    def linears(self):
        return [self.fused, self.a2, self.o]

    def cache_need(self):
        return StateCacheNeed((self.heads * self.dk * self.dv,), "float32")

    def forward(self, x, batch, cache):
        proj = self.fused(x, out_dtype=torch.float32)
        inner = torch.empty((x.shape[0], self.rank), dtype=self.ctx.dtype, device=x.device)
        kernels.tanh_cols(proj, self.rank_offset, self.rank, inner, activation="none")
        decay_pre = self.a2(inner, out_dtype=torch.float32)
        o = torch.empty((x.shape[0], self.heads * self.dv), dtype=torch.float32, device=x.device)
        kernels.gla_scan(proj, self.offsets, decay_pre, self.decay_bias, self.tau, cache.state, batch.q_start, batch.state_slot, batch.num_seqs, o,
                         self.heads, self.dk, self.dv, self.dk ** -0.5, status=batch.status, longest=1 if batch.one_token_each else batch.num_tokens)
        return self._finish(o, proj, self.gate_offset, self.heads, self.dv)
