"""Several mixers side by side on the same input: the result is the sum of
scale_i * mixer_i(h).  Of the branches at most one may keep keys and values and
at most one a per-sequence state (a run of a layer has one of each in the
cache); each branch sees the layer's cache view and takes from it what it asked
for.  The sum is left to the block's residual sum (a
:class:`~airframe_b200.parts.linear.WeightedSum`), which takes it in 32 bits.
"""
from __future__ import annotations

from ..config.base import ConfigError, PartSpec
from .base import Mixer, build_part, register_part
from .linear import WeightedSum


@register_part("mixer", "parallel")
class ParallelMixers(Mixer):
    """Parameters: ``branches``: a list of {``mixer``: PartSpec, ``scale``: number}."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        branches = self.param("branches")
        if not isinstance(branches, (list, tuple)) or not branches:
            raise ConfigError("parallel: 'branches' must list at least one mixer")
        self.branches = []
        for b in branches:
            spec = b["mixer"]
            if not isinstance(spec, PartSpec):
                raise ConfigError("parallel: a branch's 'mixer' must be a PartSpec")
            self.branches.append((build_part("mixer", spec, ctx), float(b.get("scale", 1.0))))
        if sum(m.kv_need() is not None for m, _ in self.branches) > 1:
            raise ConfigError("parallel: at most one branch may keep keys and values")
        if sum(m.state_need() is not None for m, _ in self.branches) > 1:
            raise ConfigError("parallel: at most one branch may keep a per-sequence state")

    @property
    def graph_safe(self):
        return all(m.graph_safe for m, _ in self.branches)

    def kv_need(self):
        return next((m.kv_need() for m, _ in self.branches if m.kv_need() is not None), None)

    def state_need(self):
        return next((m.state_need() for m, _ in self.branches if m.state_need() is not None), None)

    def weight_decls(self):
        return [d for m, _ in self.branches for d in m.weight_decls()]

    def load(self, weights):
        for m, _ in self.branches:
            m.load(weights)

    def decode_bytes(self, lens) -> int:
        return sum(m.decode_bytes(lens) for m, _ in self.branches)

    def prefill_flops(self, lens) -> int:
        return sum(m.prefill_flops(lens) for m, _ in self.branches)

    def score_flops(self, lens) -> int:
        return sum(getattr(m, "score_flops", lambda _l: 0)(lens) for m, _ in self.branches)

    def forward(self, x, batch, view):
        terms = []
        for m, scale in self.branches:
            out = m.forward(x, batch, view)
            if isinstance(out, WeightedSum):
                terms.extend((t, s * scale) for t, s in out.terms)
            else:
                terms.append((out, scale))
        return WeightedSum(terms)
