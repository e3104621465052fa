"""Mixers side by side: every inner mixer reads the same input, and the result is the sum of their outputs, each
times its own constant.

    out = sum_k scale_k * mixer_k(x)

Parameters: ``mixers`` (a tuple of PartSpec, each a registered mixer with its own prefix), ``scales`` (one number
per mixer), ``positions`` (per mixer a PartSpec of a position encoding or None).  Each inner mixer keeps a cache
or state of its own: ``cache_spec()`` is the tuple of theirs, and inner mixer k works on ``sub_slot(slot, k)``.
An inner mixer must be able to add its output, times a constant, into a 32-bit buffer (``adds_into_residual`` and
``scales_residual``), so that the sum is formed in 32-bit whatever the engine's type.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import sub_slot
from ..weights.loader import WeightSpec
from .base import Part, build_part, declared, register_part


class ParallelMixers(Part):
    adds_into_residual = True        # forward(accumulate_into=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        specs = tuple(self.p("mixers"))
        self.scales = tuple(float(a) for a in self.p("scales", (1.0,) * len(specs)))
        positions = tuple(self.p("positions", (None,) * len(specs)))
        if not specs or len(self.scales) != len(specs) or len(positions) != len(specs):
            raise ValueError("parallel mixers: one scale and one position entry per mixer")
        self.positions = [build_part("position", p, rt) if p is not None else None for p in positions]
        self.mixers = [build_part("mixer", m, rt, position=p) for m, p in zip(specs, self.positions)]
        for m in self.mixers:
            if not (declared(m, "adds_into_residual") and declared(m, "scales_residual")):
                raise ValueError(f"parallel mixers: '{m.spec.kind}' cannot add its scaled output into a 32-bit sum")

    def parts(self) -> List[Part]:
        return [*self.mixers, *(p for p in self.positions if p is not None)]

    def cache_spec(self):
        return tuple(m.cache_spec() for m in self.mixers)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts() for w in p.weight_specs()]

    def fused_layout(self, dtype_of) -> list:
        return [f for p in self.parts() if hasattr(p, "fused_layout") for f in p.fused_layout(dtype_of)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None):
        total = accumulate_into
        if total is None:
            total = ctx.workspace.get("parallel.sum", (x.shape[0], x.shape[1]), torch.float32)
            total.zero_()
        for k, (m, a) in enumerate(zip(self.mixers, self.scales)):
            left = m.forward(x, ctx, sub_slot(slot, k), write_cache, accumulate_into=total, residual_scale=a)
            if left is not None:          # the mixer could not add by itself: its delta comes back unscaled
                total.add_(left.to(torch.float32), alpha=a)
        return None if accumulate_into is not None else total


register_part("mixer", "parallel", ParallelMixers)
