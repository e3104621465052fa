"""Routed experts with group-limited choice and a shared expert.

    z = W_router x (32-bit);  s = softmax(z) over all experts
    experts form `groups` equal groups of neighbours; a group's score is its largest s; only experts
    of the `keep` best groups may be chosen; of those, the `top` with the largest s are
    weights = chosen s / (their sum + 1e-20)
    expert(x) = W_down (g * sigmoid(1.702 g) * (u + 1)),  g = min(W_gate x, limit),  u = clamp(W_up x, -limit, limit)
    out = sum of weight * expert(x) over the chosen experts  (+ shared expert(x), with sizes and limit of its own)

All of it stays on the device (``csrc/moe.cu``): the router's choice, a plan that sorts the step's
(token, choice) pairs by expert, two grouped products over the experts' stacked matrices (the first with
the activation in its epilogue; bfloat16 on tensor cores) and one kernel that forms the weighted sum, adds the shared expert and
adds the whole, times the block's multiplier, into the 32-bit residual.  No count is read by the host,
so steps with routed experts are captured into CUDA graphs like any other.

Parameters: hidden_size, experts, top, groups, keep, ff, limit, shared_ff (0: no shared expert),
shared_limit.  Tensors: router [experts, W]; e<i>.gate, e<i>.up [ff, W]; e<i>.down [W, ff];
shared.gate, shared.up [shared_ff, W]; shared.down [W, shared_ff].

What the lines above fix can be chosen by further parameters (the defaults are the above):
    score          "softmax" | "sigmoid": s = sigmoid(z), each expert by itself
    correction     True: a tensor ``correction`` [experts] is added to s for the choice (of groups and of experts);
                   the weights stay the plain s
    group_score    "best" | "two_best": a group's score is the sum of its two largest choice scores
    renormalize    False: the weights are the chosen s as they are
    activation     "clamped_swish" | "silu": expert(x) = W_down (silu(W_gate x) * (W_up x)), no clamps, no limit
Experts outside the open groups count as minus infinity in the choice (choice scores may be negative).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear


class GroupedExperts(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    scales_residual = True           # forward(residual_scale=...)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.E = int(self.p("experts"))
        self.top = int(self.p("top"))
        self.groups = int(self.p("groups", 1))
        self.keep = int(self.p("keep", self.groups))
        self.ff = int(self.p("ff"))
        self.activation = {"clamped_swish": K.GLU_CLAMPED_SWISH, "silu": K.GLU_SILU}[str(self.p("activation", "clamped_swish"))]
        self.limit = float(self.p("limit", 0.0 if self.activation == K.GLU_SILU else ...))
        self.score = {"softmax": K.ROUTE_SOFTMAX, "sigmoid": K.ROUTE_SIGMOID}[str(self.p("score", "softmax"))]
        self.group_score = {"best": K.GROUP_BY_BEST, "two_best": K.GROUP_BY_TWO_BEST}[str(self.p("group_score", "best"))]
        self.renormalize = bool(self.p("renormalize", True))
        self.has_correction = bool(self.p("correction", False))
        self.correction = None
        self.shared_ff = int(self.p("shared_ff", 0))
        self.shared_limit = float(self.p("shared_limit", self.limit))
        if self.E % self.groups or not (0 < self.keep <= self.groups) or not (0 < self.top <= self.keep * (self.E // self.groups)):
            raise ValueError(f"{self.prefix}: {self.top} of {self.E} experts in {self.keep} of {self.groups} groups cannot be chosen")
        self.router = self.w_gate = self.w_up = self.w_down = self.w_sh_gu = self.w_sh_down = None

    def weight_specs(self) -> List[WeightSpec]:
        n, W = self.name, self.hidden
        out = [WeightSpec(n("router"), (self.E, W))]
        if self.has_correction:
            out.append(WeightSpec(n("correction"), (self.E,), init="zeros", as_float32=True))
        for e in range(self.E):
            out += [WeightSpec(n(f"e{e}.gate"), (self.ff, W)), WeightSpec(n(f"e{e}.up"), (self.ff, W)),
                    WeightSpec(n(f"e{e}.down"), (W, self.ff))]
        if self.shared_ff:
            out += [WeightSpec(n("shared.gate"), (self.shared_ff, W)), WeightSpec(n("shared.up"), (self.shared_ff, W)),
                    WeightSpec(n("shared.down"), (W, self.shared_ff))]
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        """The experts' matrices stacked, [experts * rows, columns] each kind; the shared expert's gate over up."""
        n, W = self.name, self.hidden
        out = [FusedSpec(n("experts.gate"), (self.E * self.ff, W), tuple(Piece(n(f"e{e}.gate"), e * self.ff) for e in range(self.E))),
               FusedSpec(n("experts.up"), (self.E * self.ff, W), tuple(Piece(n(f"e{e}.up"), e * self.ff) for e in range(self.E))),
               FusedSpec(n("experts.down"), (self.E * W, self.ff), tuple(Piece(n(f"e{e}.down"), e * W) for e in range(self.E)))]
        if self.shared_ff:
            out.append(FusedSpec(n("shared.gate_up"), (2 * self.shared_ff, W),
                                 (Piece(n("shared.gate"), 0), Piece(n("shared.up"), self.shared_ff))))
        return out

    def _stacked(self, tensors, fused: str, leaves: List[str]) -> torch.Tensor:
        if self.name(fused) in tensors:
            return self._matrix(tensors[self.name(fused)])
        mats = [self._matrix(tensors[self.name(leaf)]) for leaf in leaves]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.to(torch.float32) for m in mats]
        return torch.cat(mats, dim=0).contiguous()

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        E, W = self.E, self.hidden
        self.router = self._matrix(tensors[self.name("router")])
        if self.has_correction:
            self.correction = self._vector32(tensors[self.name("correction")])
        self.w_gate = self._stacked(tensors, "experts.gate", [f"e{e}.gate" for e in range(E)]).view(E, self.ff, W)
        self.w_up = self._stacked(tensors, "experts.up", [f"e{e}.up" for e in range(E)]).view(E, self.ff, W)
        self.w_down = self._stacked(tensors, "experts.down", [f"e{e}.down" for e in range(E)]).view(E, W, self.ff)
        if len({self.w_gate.dtype, self.w_up.dtype, self.w_down.dtype}) != 1:
            self.w_gate, self.w_up, self.w_down = (m.to(torch.float32) for m in (self.w_gate, self.w_up, self.w_down))
        if self.shared_ff:
            self.w_sh_gu = self._stacked(tensors, "shared.gate_up", ["shared.gate", "shared.up"])
            self.w_sh_down = self._matrix(tensors[self.name("shared.down")])

    def forward(self, x, ctx, accumulate_into=None, residual_scale: float = 1.0):
        T, ws, W, top = x.shape[0], ctx.workspace, self.hidden, self.top
        dt = self.w_gate.dtype
        if x.dtype != dt:
            raise K.KernelError(f"{self.prefix}: activations {x.dtype} against expert matrices {dt}")
        # the router: logits, scores and the choice in 32-bit
        z = ws.get("moe.z", (T, self.E), torch.float32)
        apply_linear(x, self.router, z, ctx, "moe.z")
        ids = ws.get("moe.ids", (T, top), torch.int32)
        wts = ws.get("moe.wts", (T, top), torch.float32)
        K.moe_route(z, ids, wts, self.groups, self.keep, score=self.score, correction=self.correction,
                    group_score=self.group_score, renormalize=self.renormalize)
        rows = T * top
        tc = K.moe_on_tensor_cores(dt, (W, self.ff))       # which grouped kernel runs: the plan's row tile is its
        max_tiles = K.moe_max_tiles(rows, self.E, tc)
        seg = ws.get("moe.seg", (self.E + 1,), torch.int32)
        row_of = ws.get("moe.row_of", (rows,), torch.int32)
        src_tok = ws.get("moe.src_tok", (rows,), torch.int32)
        tile_e = ws.get("moe.tile_e", (max_tiles,), torch.int32)
        tile_r = ws.get("moe.tile_r", (max_tiles,), torch.int32)
        n_tiles = ws.get("moe.n_tiles", (1,), torch.int32)
        K.moe_plan(ids, self.E, seg, row_of, src_tok, tile_e, tile_r, n_tiles, tc)
        plan = (seg, tile_e, tile_r, n_tiles, max_tiles)
        act = ws.get("moe.act", (rows, self.ff), dt)
        K.moe_grouped(x, src_tok, self.w_gate, self.w_up, plan, act, self.limit, tc, self.activation)
        outs = ws.get("moe.rows", (rows, W), torch.float32)
        K.moe_grouped(act, src_tok, self.w_down, None, plan, outs, 0.0, tc)
        shared = None
        if self.shared_ff:
            gu = ws.get("moe.sh_gu", (T, 2 * self.shared_ff), dt)
            apply_linear(x, self.w_sh_gu, gu, ctx, "moe.sh_gu")
            sact = ws.get("moe.sh_act", (T, self.shared_ff), dt)
            K.clamped_glu(gu, sact, self.shared_limit)
            shared = ws.get("moe.sh_out", (T, W), torch.float32)
            apply_linear(sact, self.w_sh_down, shared, ctx, "moe.sh_out")
        if accumulate_into is not None:
            K.moe_combine(accumulate_into, outs, row_of, wts, shared, residual_scale)
            return None
        delta = ws.get("moe.delta", (T, W), torch.float32)
        delta.zero_()
        K.moe_combine(delta, outs, row_of, wts, shared, 1.0)
        return delta


register_part("feed_forward", "grouped_experts", GroupedExperts)
