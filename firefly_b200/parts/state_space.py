"""A state-space mixer with a scalar, data-dependent decay per head (the Mamba-2 form):

    [z | x | B | C | step] = W_in h          z, x: heads*vdim; B, C: groups*state; step: heads
    x, B, C  <- silu(causal convolution per channel, `conv` taps, with bias; zeros in front of the sequence)
    step     <- softplus(step + step_bias)                               (no clamp)
    S_t      = exp(-exp(A_log_h) step) S_(t-1) + step B_t x_t^T          per head, S: [state, vdim], starts at 0;
    y_t      = S_t^T C_t + D_h x_t                                       head h reads group floor(h / (heads/groups))
    out      = W_o (rms_norm(y * silu(z), in `norm_groups` equal parts) * norm)      (the gate in front of the norm)

The request's state slot holds S of every head (32-bit, in the recurrence kernel's own order) and the
convolution's last conv-1 inputs; a portion of a prompt continues from both.  Steps, decays, S and the sums of the
recurrence, the gate and the norm are 32-bit; the projection, the convolution's output and the normed rows are in
the engine's type.  Kernels: ``csrc/ssm.cu``.

Parameters: hidden_size, heads, vdim, state, groups, conv, norm_groups, eps.
Tensors (leaves under the prefix): in [2*heads*vdim + 2*groups*state + heads, W]; conv [channels, conv] and conv.b
[channels] with channels = heads*vdim + 2*groups*state; dt_bias, A_log, D [heads]; norm [heads*vdim];
o [W, heads*vdim].
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import StateSpec
from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, scaled_linear_into_residual


class StateSpaceMixer(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.heads = int(self.p("heads"))
        self.vdim = int(self.p("vdim"))
        self.N = int(self.p("state"))
        self.groups = int(self.p("groups", 1))
        self.taps = int(self.p("conv"))
        self.norm_groups = int(self.p("norm_groups", 1))
        self.eps = float(self.p("eps"))
        self.inner = self.heads * self.vdim
        self.gn = self.groups * self.N
        self.channels = self.inner + 2 * self.gn
        self.proj_width = 2 * self.inner + 2 * self.gn + self.heads
        if self.heads % self.groups or self.inner % self.norm_groups or not (1 <= self.taps <= 16):
            raise ValueError(f"{self.prefix}: {self.heads} heads in {self.groups} groups, {self.norm_groups} norm "
                             f"parts of {self.inner}, {self.taps} taps: sizes do not fit")
        self.scan_floats = K.scan_state_floats(self.heads, self.N, self.vdim)
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm = None

    def cache_spec(self):
        return StateSpec((self.scan_floats + (self.taps - 1) * self.channels,), torch.float32)

    def weight_specs(self) -> List[WeightSpec]:
        n = self.name
        return [WeightSpec(n("in"), (self.proj_width, self.hidden)),
                WeightSpec(n("conv"), (self.channels, self.taps), as_float32=True),
                WeightSpec(n("conv.b"), (self.channels,), init="zeros", as_float32=True),
                WeightSpec(n("dt_bias"), (self.heads,), as_float32=True),
                WeightSpec(n("A_log"), (self.heads,), as_float32=True),
                WeightSpec(n("D"), (self.heads,), init="ones", as_float32=True),
                WeightSpec(n("norm"), (self.inner,), init="norm", as_float32=True),
                WeightSpec(n("o"), (self.hidden, self.inner))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.name
        self.w_in, self.w_o = self._matrix(tensors[n("in")]), self._matrix(tensors[n("o")])
        self.conv_w, self.conv_b = self._vector32(tensors[n("conv")]), self._vector32(tensors[n("conv.b")])
        self.dt_bias, self.a_log = self._vector32(tensors[n("dt_bias")]), self._vector32(tensors[n("A_log")])
        self.skip, self.norm = self._vector32(tensors[n("D")]), self._vector32(tensors[n("norm")])

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, residual_scale: float = 1.0):
        T, ws = x.shape[0], ctx.workspace
        dt = self.w_in.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against matrices {dt}")
        state = ctx.state(slot)
        proj = ws.get("ssm.proj", (T, self.proj_width), dt)
        apply_linear(x, self.w_in, proj, ctx, "ssm.proj")
        xbc = ws.get("ssm.xbc", (T, self.channels), dt)
        K.causal_conv_silu(proj, self.inner, self.channels, self.conv_w, self.conv_b, state, self.scan_floats, ctx, xbc)
        o = ws.get("ssm.o", (T, self.inner), torch.float32)
        K.scalar_decay_scan((xbc, self.inner + self.gn), (xbc, self.inner), (xbc, 0), state, 0, ctx, o, self.heads,
                            self.N, self.vdim, heads_per_group=self.heads // self.groups,
                            step=(proj, 2 * self.inner + 2 * self.gn), step_bias=self.dt_bias, a_log=self.a_log,
                            skip=self.skip)
        y = ws.get("ssm.y", (T, self.inner), dt)
        K.gated_rms_norm(o, (proj, 0), self.norm, self.eps, y, self.norm_groups, gate_first=True)
        return scaled_linear_into_residual(y, self.w_o, accumulate_into, residual_scale, ctx, "ssm.out")


register_part("mixer", "state_space", StateSpaceMixer)
