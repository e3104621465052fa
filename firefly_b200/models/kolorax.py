"""Kolorax as data: a ``ModelSpec`` made of registered parts.

Blocks are pre-norm with layer norms (weight and bias) and one multiplier on everything a part
adds to the stream: x += m * mixer(LN1(x)); x += m * experts(LN2(x)).  A layer's mixer is the
recurrent ``wkv`` mixer or ``latent_attention``; its feed-forward is a set of routed experts chosen
within the best groups, plus a shared expert, or nothing.  A range of layers may run several times
with the same weights: every pass has cache slots of its own (the schedule names a layer once per
run) and starts with the ``loop_input`` junction, which re-makes the stream from itself and the
embedding output and adds the pass's offset.  The embedding is scaled; the output is a layer norm
and the head.  Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``,
``loop.in``, ``loop.step``, ``final.norm`` (+ ``.b``), ``head``.
"""
from __future__ import annotations

from ..config.base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.kolorax import KoloraxConfig, file_hints
from .registry import register_architecture

DEFAULT_DECAY_RANK = 64      # rows of a wkv layer's first decay matrix when neither the configuration nor a file says
# The design itself has no longest position (angles are formed from the position, the state has no length); the
# engine's block tables and its cache sizing still want a bound on a request's length.
MAX_POSITIONS = 1 << 20


def _norm(cfg: KoloraxConfig, prefix: str) -> PartSpec:
    return PartSpec("layer_norm", dict(size=cfg.width, eps=cfg.norm_eps, weight_leaf="", bias_leaf=".b"), prefix=prefix)


def kolorax_spec(cfg: KoloraxConfig) -> ModelSpec:
    W = cfg.width
    layers = []
    for i, L in enumerate(cfg.layers):
        p, mx = f"l{i}", L["mixer"]
        position = None
        if L["type"] == "wkv":
            mixer = PartSpec("wkv", dict(hidden_size=W, heads=int(mx["heads"]), dim=int(mx["dim"]),
                                         decay_rank=int(mx.get("decay_rank", DEFAULT_DECAY_RANK)), eps=cfg.norm_eps),
                             prefix=f"{p}.mix")
        else:
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]),
                vdim=int(mx["vdim"]), kv_rank=int(mx["kv_rank"]), scale=float(mx["scale"]), eps=cfg.norm_eps),
                prefix=f"{p}.mix")
            position = PartSpec("rotary", dict(head_dim=int(mx["rot_dim"]),
                                               rotary_dim=int(mx["rot"].get("dims", mx["rot_dim"])),
                                               theta=float(mx["rot"]["base"]), max_positions=0))
        ml = L.get("mlp")
        ff = None
        if ml is not None:
            r, groups, shared = ml["router"], ml["router"].get("groups") or {}, ml.get("shared")
            count = int(groups.get("count", 1))
            ff = PartSpec("grouped_experts", dict(
                hidden_size=W, experts=int(r["experts"]), top=int(r["top"]), groups=count,
                keep=int(groups.get("keep", count)), ff=int(ml["expert"]["ff"]), limit=float(ml["expert"]["limit"]),
                shared_ff=int(shared["ff"]) if shared else 0,
                shared_limit=float(shared["limit"]) if shared else 0.0), prefix=f"{p}.mlp")
        norms = (_norm(cfg, f"{p}.norm1"),) + ((_norm(cfg, f"{p}.norm2"),) if ff is not None else ())
        layers.append(LayerSpec("scaled_pre_norm", mixer, ff, norms, position,
                                params=dict(residual_mult=cfg.residual_mult)))
    n = len(layers)
    junctions = ()
    if cfg.loop:
        a, b, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        junctions = (PartSpec("loop_input", dict(hidden_size=W, passes=times, in_tensor="loop.in",
                                                 step_tensor="loop.step")),)
        runs = [ScheduleEntry(i) for i in range(a)]
        for t in range(times):
            runs += [ScheduleEntry(i, junction=(0, t) if i == a else None) for i in range(a, b)]
        runs += [ScheduleEntry(i) for i in range(b, n)]
    else:
        runs = [ScheduleEntry(i) for i in range(n)]
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=W, scale=cfg.embedding_scale,
                                                   tensor="embed")),
        layers=tuple(layers), schedule=tuple(runs),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="head")),
        junctions=junctions,
    )


register_architecture("Kolorax", KoloraxConfig, kolorax_spec, file_hints=file_hints)
