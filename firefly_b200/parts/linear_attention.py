"""Linear attention with a constant decay per head (the lightning-attention form):

    q, k = silu(W_q x), silu(W_k x)   [heads, dim];   v = silu(W_v x)   [heads, vdim]
    S_t  = decay_h S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t             per head, S starts at 0
    out  = W_o (rms_norm(o over all heads together) * norm * sigmoid(W_g x))

There is no softmax, no scale and no position encoding.  The request's state slot holds S of every head in
32-bit (in the recurrence kernel's own order); a portion of a prompt continues from it, so prompts may be cut
anywhere.  The four projections are one product against the stacked matrix [q | k | v | g]; the SiLU of q, k, v
is taken in 32-bit where the recurrence reads them (``csrc/ssm.cu``).

Parameters: hidden_size, heads, dim, vdim, decay (one number per head), eps (of the output norm).
Tensors (leaves under the prefix): q, k [heads*dim, W]; v, g [heads*vdim, W]; norm [heads*vdim]; o [W, heads*vdim].
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import StateSpec
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, scaled_linear_into_residual


class LinearAttention(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.heads = int(self.p("heads"))
        self.dim = int(self.p("dim"))
        self.vdim = int(self.p("vdim", self.dim))
        self.eps = float(self.p("eps"))
        self.decay_values = tuple(float(a) for a in self.p("decay"))
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{self.prefix}: {len(self.decay_values)} decays for {self.heads} heads")
        self.state_floats = K.scan_state_floats(self.heads, self.dim, self.vdim)
        self.kq, self.kv = self.heads * self.dim, self.heads * self.vdim
        self.w_qkvg = self.w_o = self.norm = self.decay = None

    def cache_spec(self):
        return StateSpec((self.state_floats,), torch.float32)

    def _sources(self):
        return [(self.name("q"), self.kq), (self.name("k"), self.kq), (self.name("v"), self.kv), (self.name("g"), self.kv)]

    def weight_specs(self) -> List[WeightSpec]:
        out = [WeightSpec(name, (rows, self.hidden)) for name, rows in self._sources()]
        out += [WeightSpec(self.name("norm"), (self.kv,), init="norm", as_float32=True),
                WeightSpec(self.name("o"), (self.hidden, self.kv))]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        pieces, at = [], 0
        for name, rows in self._sources():
            pieces.append(Piece(name, at))
            at += rows
        return [FusedSpec(self.name("qkvg"), (at, self.hidden), tuple(pieces))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if self.name("qkvg") in tensors:
            self.w_qkvg = self._matrix(tensors[self.name("qkvg")])
        else:
            mats = [self._matrix(tensors[name]) for name, _ in self._sources()]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            self.w_qkvg = torch.cat(mats, dim=0).contiguous()
        self.w_o = self._matrix(tensors[self.name("o")])
        self.norm = self._vector32(tensors[self.name("norm")])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, residual_scale: float = 1.0):
        T, ws = x.shape[0], ctx.workspace
        dt = self.w_qkvg.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against matrices {dt}")
        proj = ws.get("lin_attn.proj", (T, 2 * self.kq + 2 * self.kv), dt)
        apply_linear(x, self.w_qkvg, proj, ctx, "lin_attn.proj")
        o = ws.get("lin_attn.o", (T, self.kv), torch.float32)
        K.scalar_decay_scan((proj, 0), (proj, self.kq), (proj, 2 * self.kq), ctx.state(slot), 0, ctx, o, self.heads,
                            self.dim, self.vdim, silu_inputs=True, decay=self.decay)
        y = ws.get("lin_attn.y", (T, self.kv), dt)
        K.gated_rms_norm(o, (proj, 2 * self.kq + self.kv), self.norm, self.eps, y, 1, gate_first=False)
        return scaled_linear_into_residual(y, self.w_o, accumulate_into, residual_scale, ctx, "lin_attn.out")


register_part("mixer", "linear_attention", LinearAttention)
