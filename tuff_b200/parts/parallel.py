"""`parallel_mixers`: several mixers side by side on the same input, their outputs summed into the
residual.  Each branch is a registered mixer given as a PartSpec (or its dictionary); a branch's weight
in the sum is the branch's own `out_scale` parameter.  The branches' weights are declared under
`<branch name>.<local name>`, and their cache needs become one `CompositeNeed` in branch order (a branch
without a need gets None there)."""
from __future__ import annotations

from typing import Dict

from .base import MIXERS, CompositeNeed, Mixer, PartSpec, register_mixer


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, branches: Dict[str, PartSpec | dict]):
        if not branches:
            raise ValueError("parallel_mixers needs at least one branch")
        self.names = list(branches)
        self.branches = [MIXERS.build(PartSpec(**b) if isinstance(b, dict) else b) for b in branches.values()]
        self.replayable = all(getattr(b, "replayable", True) and
                              getattr(getattr(b, "pos", None), "replayable", True) for b in self.branches)

    def weight_decls(self):
        return {f"{n}.{local}": decl for n, b in zip(self.names, self.branches) for local, decl in b.weight_decls().items()}

    def cache_need(self):
        return CompositeNeed(tuple(b.cache_need() for b in self.branches))

    def bind(self, weights, act_dtype):
        self.act_dtype = act_dtype
        for n, b in zip(self.names, self.branches):
            b.bind({local: weights[f"{n}.{local}"] for local in b.weight_decls()}, act_dtype)
        self.w = {}

    def reserve(self, device, max_rows, max_context):
        for b in self.branches:
            b.reserve(device, max_rows, max_context)

    def forward(self, ctx, cache, h, residual, reads_only=False):
        for b, storage in zip(self.branches, cache.parts):
            b.forward(ctx, storage, h, residual, reads_only)
