"""Junctions: what happens to the residual stream between two runs of the
schedule.

``reinject``: x <- W [x; x0] + s_t, with x0 the embedding's output of the
step, W of shape [hidden, 2 hidden] (the columns that meet x first) and s a
table of one row per pass through a repeated stretch of layers; run ``t`` of
the stretch enters through it with ``enter_index`` = t.  The product takes its
inputs in the compute dtype and leaves 32-bit sums; the row is added in 32
bits.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Junction, register_part
from .linear import PartialSums, linear_split
from .norm import TanhNorm


@register_part("junction", "reinject")
class Reinject(Junction):
    """Parameters: ``hidden_size``, ``passes`` (rows of the table), ``weight`` and ``step_weight`` (tensor names)."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.passes = int(self.param("passes"))
        self.names = (self.param("weight"), self.param("step_weight"))
        self.w = self.steps = None

    def weight_decls(self):
        w, s = self.names
        return [WeightDecl(w, (self.hidden, 2 * self.hidden)), WeightDecl(s, (self.passes, self.hidden), "norm")]

    def load(self, weights):
        w, s = self.names
        self.w = weights[w].to(self.ctx.compute_dtype).contiguous()
        self.steps = weights[s].to(torch.float32).contiguous()

    def decode_bytes(self, lens) -> int:
        return self.w.numel() * (4 if self.ctx.compute_dtype == torch.float32 else 2)

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * self.w.numel()

    def forward(self, x, x0, index, batch, then=None, out_dtype=None):
        both = torch.empty(x.shape[0], 2 * self.hidden, dtype=self.ctx.compute_dtype, device=x.device)
        kernels.concat_cast(both, x, x0)
        z = linear_split(both, self.w, wide=True)
        z = z.parts if isinstance(z, PartialSums) else z
        if then is None or not isinstance(then, TanhNorm):
            kernels.set_sum_row(x, z, self.steps[index])
            return then.forward(x, out_dtype) if then is not None else None
        y = torch.empty(x.shape[0], self.hidden, dtype=out_dtype, device=x.device)
        kernels.set_sum_row(x, z, self.steps[index], y=y, w=then.w, b=then.b, alpha=then.alpha)
        return y
