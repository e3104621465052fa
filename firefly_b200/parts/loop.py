"""What runs at the head of a pass over a looped range of layers.

``loop_input``: the stream x is re-made from itself and the embedding output x0, and the pass's own
offset is added:   x <- W_in [x ; x0] + step[turn]     (W_in [W, 2W], x first; step [passes, W]).
The product runs in the engine's matrix type with 32-bit accumulation and a 32-bit result, which
becomes the new residual stream; the offset is added in 32-bit.

A junction is a part of category ``junction``: ``forward(residual, pending, ctx, stream0, turn)`` ->
(residual, pending), where ``stream0`` is the embedding output of the step's tokens (kept by the model
when a junction declares ``needs_embedding_output``) and ``turn`` the number of the pass.

Parameters: hidden_size, passes.  Tensors: ``in_tensor`` [W, 2W], ``step_tensor`` [passes, W] (full names).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear


class LoopInput(Part):
    needs_embedding_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.passes = int(self.p("passes"))
        self.in_tensor = self.p("in_tensor", None) or self.name("in")
        self.step_tensor = self.p("step_tensor", None) or self.name("step")
        self.w_in = self.step = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.in_tensor, (self.hidden, 2 * self.hidden)),
                WeightSpec(self.step_tensor, (self.passes, self.hidden), init="zeros", as_float32=True)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = self._matrix(tensors[self.in_tensor])
        self.step = self._vector32(tensors[self.step_tensor])

    def forward(self, residual, pending, ctx, stream0, turn: int):
        if pending is not None:
            if not isinstance(pending, torch.Tensor):
                raise RuntimeError("loop_input: the layer in front left a folded norm; it must add its output itself")
            K.residual_add(residual, pending)
        T, W = residual.shape
        both = ctx.workspace.get("loop.both", (T, 2 * W), self.w_in.dtype)
        K.concat_cast(residual, stream0, both)
        apply_linear(both, self.w_in, residual, ctx, "loop.in")     # reads `both`, writes the stream
        K.add_row_vector(residual, self.step[turn])
        return residual, None


register_part("junction", "loop_input", LoopInput)
