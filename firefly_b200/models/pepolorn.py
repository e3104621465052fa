"""Pepolorn as data: a ``ModelSpec`` made of registered parts.

Blocks carry their norms on the parts' outputs (``output_norm``): x += norm1(mixer(x)); x += norm2(ff(x)), the
norm an RMS norm whose weight is stored around zero (multiplier 1 + w).  A layer's mixer is a state-space mixer
(``state_space``) or two mixers side by side (``parallel``): grouped-query softmax attention inside chunks of
positions, with a partly rotated, rescaled rotary encoding and unit-normed q and k (``gqa_attention`` with its
parameters), beside linear attention with a constant decay per head (``linear_attention``).  Its feed-forward is a
gated MLP with the tanh form of GELU, routed experts (sigmoid scores, a correction for the choice only, groups
scored by their two best, weights not renormalised, SiLU experts), or nothing.  A layer may run another layer's
tensors with a cache and state of its own: the schedule then names that layer a second time.  The output is the
same kind of norm and the embedding table as the head.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.pepolorn import PepolornConfig
from .registry import register_architecture

# The design has no longest position (angles are formed from the position, the states have no length); the
# engine's block tables and its cache sizing still want a bound on a request's length.
MAX_POSITIONS = 1 << 20


def _norm(cfg: PepolornConfig, tensor: str) -> PartSpec:
    return PartSpec("rms_norm", dict(size=cfg.width, eps=cfg.norm_eps, weight_offset=1.0, tensor=tensor))


def _mixer(cfg: PepolornConfig, L, p: str) -> PartSpec:
    W, mx = cfg.width, L["mixer"]
    if L["type"] == "mamba2":
        return PartSpec("state_space", dict(
            hidden_size=W, heads=int(mx["heads"]), vdim=int(mx["vdim"]), state=int(mx["state"]),
            groups=int(mx["groups"]), conv=int(mx["conv"]), norm_groups=int(mx["norm_groups"]), eps=cfg.norm_eps),
            prefix=f"{p}.mix")
    left, right = mx["left"], mx["right"]
    rot = left["rot"]
    attention = PartSpec("gqa_attention", dict(
        hidden_size=W, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), head_dim=int(left["dim"]),
        value_dim=int(left["vdim"]), scale=float(left["scale"]), chunk=int(left["mask"]["size"]),
        unit_norm_after_rotation=True, qk_norm_eps=cfg.norm_eps, q_leaf="q", k_leaf="k", v_leaf="v", o_leaf="o"),
        prefix=f"{p}.mix.left")
    position = PartSpec("rotary", dict(head_dim=int(left["dim"]), rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                       max_positions=0, scaling=dict(rot["scaling"]) if rot.get("scaling") else None))
    linear = PartSpec("linear_attention", dict(
        hidden_size=W, heads=int(right["heads"]), dim=int(right["dim"]), vdim=int(right["vdim"]),
        decay=tuple(float(a) for a in right["decay"]), eps=cfg.norm_eps), prefix=f"{p}.mix.right")
    return PartSpec("parallel", dict(mixers=(attention, linear), positions=(position, None),
                                     scales=(float(mx["left_scale"]), float(mx["right_scale"]))), prefix=f"{p}.mix")


def _feed_forward(cfg: PepolornConfig, ml, p: str):
    if ml is None:
        return None
    if ml["kind"] == "dense":
        return PartSpec("gated_mlp", dict(hidden_size=cfg.width, intermediate_size=int(ml["ff"]), activation="gelu_tanh"),
                        prefix=f"{p}.mlp")
    r = ml["router"]
    groups = r.get("groups") or {}
    count = int(groups.get("count", 1))
    return PartSpec("grouped_experts", dict(
        hidden_size=cfg.width, experts=int(r["experts"]), top=int(r["top"]), groups=count,
        keep=int(groups.get("keep", count)), ff=int(ml["expert"]["ff"]), score="sigmoid", correction=True,
        group_score="two_best", renormalize=False, activation="silu"), prefix=f"{p}.mlp")


def pepolorn_spec(cfg: PepolornConfig) -> ModelSpec:
    layers, index_of = [], {}
    for i, L in enumerate(cfg.layers):
        if cfg.source_layer(i) != i:
            continue
        p = f"l{i}"
        ff = _feed_forward(cfg, L.get("mlp"), p)
        norms = (_norm(cfg, f"{p}.norm1"),) + ((_norm(cfg, f"{p}.norm2"),) if ff is not None else ())
        index_of[i] = len(layers)
        layers.append(LayerSpec("output_norm", _mixer(cfg, L, p), ff, norms))
    # one run per configured layer, each with a cache slot of its own; a layer that runs another's tensors is
    # that layer's block named again
    runs = tuple(ScheduleEntry(index_of[cfg.source_layer(i)]) for i in range(len(cfg.layers)))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tensor="embed")),
        layers=tuple(layers), schedule=runs, final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied_to="embed", tensor="head")),
    )


register_architecture("Pepolorn", PepolornConfig, pepolorn_spec)
