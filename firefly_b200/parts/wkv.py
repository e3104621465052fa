"""A recurrent mixer with a matrix state per head and a per-channel, data-dependent decay
(RWKV-style time mixing).  For the inputs x of a sequence, with x[-1] = 0:

    mix_s[t] = x[t] + (x[t-1] - x[t]) * mu_s                     s in {r, k, v, g, w}
    r, k, v  = W_r mix_r, W_k mix_k, W_v mix_v                   [heads, dim] each
    gate     = silu(W_g mix_g)
    w[t]     = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))             per head and key channel, in (0, 1)
    o[t]     = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T per head, S: [dim, dim], starts at 0
    out      = W_o (o / rms(o over a head) * norm * gate)

The request's state slot holds S of every head and the last x of the sequence, in 32-bit; a portion
of a prompt continues from it, so prompts may be cut anywhere.  The five projections' inputs differ,
so r, k, v, g run as one batched product over the stacked matrix [4, heads*dim, W]; the decay's two
small products follow; the recurrence is one kernel (``csrc/wkv.cu``) that walks a sequence's tokens
in order.

Parameters: hidden_size, heads, dim, decay_rank (rows of w1), eps (of the head norm).
Tensors (leaves under the prefix): mu.r mu.k mu.v mu.g mu.w [W]; r k v g [heads*dim, W];
w1 [decay_rank, W]; w2 [heads*dim, decay_rank]; w0 [heads*dim]; u [heads, dim]; norm [heads*dim];
o [W, heads*dim].
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


class WKVMixer(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.heads = int(self.p("heads"))
        self.dim = int(self.p("dim"))
        self.rank = int(self.p("decay_rank"))
        self.eps = float(self.p("eps"))
        self.hd = self.heads * self.dim
        if self.dim > K.WKV_MAX_DIM:
            raise ValueError(f"{self.prefix}: head size {self.dim} > {K.WKV_MAX_DIM} is not supported by the recurrence kernel")
        # the slot: every head's state as the recurrence kernel keeps it, then the last input row
        self.prev_off = self.heads * K.wkv_state_dim(self.dim) ** 2
        self.w_rkvg = self.w1 = self.w2 = self.w_o = self.mu = self.w0 = self.u = self.norm = None

    def cache_spec(self):
        return StateSpec((self.prev_off + self.hidden,), torch.float32)

    def weight_specs(self) -> List[WeightSpec]:
        n, W, hd = self.name, self.hidden, self.hd
        out = [WeightSpec(n(f"mu.{s}"), (W,), init="norm", as_float32=True) for s in "rkvgw"]
        out += [WeightSpec(n(s), (hd, W)) for s in "rkvg"]
        out += [WeightSpec(n("w1"), (self.rank, W)), WeightSpec(n("w2"), (hd, self.rank)),
                WeightSpec(n("w0"), (hd,), init="zeros", as_float32=True),
                WeightSpec(n("u"), (self.heads, self.dim), as_float32=True),
                WeightSpec(n("norm"), (hd,), init="norm", as_float32=True), WeightSpec(n("o"), (W, hd))]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        return [FusedSpec(self.name("rkvg"), (4 * self.hd, self.hidden),
                          tuple(Piece(self.name(s), i * self.hd) for i, s in enumerate("rkvg")))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.name
        if n("rkvg") in tensors:
            rkvg = self._matrix(tensors[n("rkvg")])
        else:
            mats = [self._matrix(tensors[n(s)]) for s in "rkvg"]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            rkvg = torch.cat(mats, dim=0).contiguous()
        self.w_rkvg = rkvg.view(4, self.hd, self.hidden)
        self.w1, self.w2, self.w_o = (self._matrix(tensors[n(s)]) for s in ("w1", "w2", "o"))
        self.mu = torch.stack([self._vector32(tensors[n(f"mu.{s}")]) for s in "rkvgw"]).contiguous()
        self.w0, self.norm = self._vector32(tensors[n("w0")]), self._vector32(tensors[n("norm")])
        self.u = self._vector32(tensors[n("u")]).reshape(-1).contiguous()

    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, residual_scale: float = 1.0):
        T, ws = x.shape[0], ctx.workspace
        state = ctx.state(slot)
        dt = self.w_rkvg.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against matrices {dt}")
        mixes = ws.get("wkv.mixes", (5, T, self.hidden), dt)
        K.wkv_shift_mix(x, self.mu, state, self.prev_off, ctx, mixes)
        rkvg = ws.get("wkv.rkvg", (4, T, self.hd), dt)
        K.batched_linear(mixes[:4], self.w_rkvg, rkvg)
        low = ws.get("wkv.low", (T, self.rank), torch.float32)
        apply_linear(mixes[4], self.w1, low, ctx, "wkv.low")
        low_t = ws.get("wkv.low_t", (T, self.rank), dt)
        K.tanh_cast(low, low_t)
        dlog = ws.get("wkv.dlog", (T, self.hd), torch.float32)
        apply_linear(low_t, self.w2, dlog, ctx, "wkv.dlog")
        o = ws.get("wkv.o", (T, self.hd), torch.float32)
        K.wkv_scan(rkvg, dlog, self.w0, self.u, state, self.prev_off, x, ctx, o, self.heads, self.dim)
        y = ws.get("wkv.y", (T, self.hd), dt)
        K.wkv_out(o, rkvg[3], self.norm, self.eps, y, self.heads, self.dim)
        return scaled_linear_into_residual(y, self.w_o, accumulate_into, residual_scale, ctx, "wkv.proj")


register_part("mixer", "wkv", WKVMixer)
