"""Two mixers side by side on the same input: ``y = left_scale * left(h) + right_scale * right(h)``.

Each side is a mixer of its own kind with its own tensors (under ``left.`` and ``right.``) and its own cache need; the
layer's cache view holds one view for each, in that order.  When the block says that the norm behind adds weighted sums
itself (``scaled_parts_ok``), the two results are handed on unsummed, each possibly still a stack of split-K partial
products; otherwise they are summed here.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import CompositeCacheNeed
from ..weights.loader import WeightDecl
from .base import Mixer, ScaledParts
from .registry import build_part, register_part


@register_part("parallel_mixers")
class ParallelMixers(Mixer):
    """params: ``left`` and ``right`` (``PartSpec`` of a mixer each), ``left_scale``, ``right_scale``, ``prefix``,
    ``left_prefix`` / ``right_prefix`` (default ``left.`` / ``right.``)."""

    scaled_parts_ok = False

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.left, self.right = build_part(params["left"], ctx), build_part(params["right"], ctx)
        self.left_scale, self.right_scale = float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0))
        prefix = params.get("prefix", "")
        self.prefixes = (prefix + params.get("left_prefix", "left."), prefix + params.get("right_prefix", "right."))

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    def _sides(self):
        return ((self.left, self.prefixes[0]), (self.right, self.prefixes[1]))

    def weight_decls(self):
        return [WeightDecl(pre + d.name, d.shape, d.init, d.integer) for part, pre in self._sides() for d in part.weight_decls()]

    def bind(self, tensors):
        for part, pre in self._sides():
            part.bind({d.name: tensors[pre + d.name] for d in part.weight_decls()})

    def modules(self):
        return ["layernorm"] + self.left.modules() + self.right.modules()

    def linears(self):
        return self.left.linears() + self.right.linears()

    def cache_need(self):
        return CompositeCacheNeed((self.left.cache_need(), self.right.cache_need()))

    def forward(self, x, batch, cache):
        # each side may leave its last product unsummed only if the sum is formed by the norm behind
        self.left.defer_output = self.right.defer_output = self.defer_output and self.scaled_parts_ok
        self.left.output_dtype = self.right.output_dtype = torch.float32 if self.scaled_parts_ok else None     # one format for the norm that adds them
        a = self.left.forward(x, batch, cache.parts[0])
        b = self.right.forward(x, batch, cache.parts[1])
        if self.scaled_parts_ok:
            return ScaledParts([(a, self.left_scale), (b, self.right_scale)])
        out = torch.empty((x.shape[0], a.shape[-1]), dtype=torch.float32, device=x.device)
        return kernels.scaled_sum(out, a, self.left_scale, b, self.right_scale)
