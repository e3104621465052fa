"""Typed configuration of the Pepolorn design.

``config.json`` names the design under ``architecture`` and gives every size and constant:

    vocab, width, norm.eps
    layers[i]: type ("mamba2" | "parallel"), mixer {...}, mlp {...} | null, weights_of: j (optional)
        mamba2 mixer:    heads, vdim, state, groups, conv, norm_groups
        parallel mixer:  left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims, scaling {factor,
                         original, fast, slow} | null}}, right {heads, dim, vdim, decay [per head]},
                         left_scale, right_scale
        mlp kind "dense": ff
        mlp kind "moe":   router {experts, top, groups {count, keep}}, expert {ff}
    A layer with ``weights_of: j`` has no tensors of its own and runs layer j's (with a cache and state of its
    own); the rest of its entry must equal layer j's.

The nested objects are kept as they are and checked here, so that a wrong or missing key is told by name before
anything is built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Tuple

from .base import ConfigError, ModelConfig

MIXERS = ("mamba2", "parallel")


def _need(obj, key: str, typ, where: str):
    if not isinstance(obj, Mapping) or key not in obj or obj[key] is None:
        raise ConfigError(f"config.json: {where} needs '{key}'")
    v = obj[key]
    if typ is int:
        if isinstance(v, bool) or not (isinstance(v, int) or (isinstance(v, float) and v == int(v))):
            raise ConfigError(f"config.json: {where}.{key} must be an integer, got {v!r}")
        if int(v) <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be positive, got {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        return float(v)
    return v


def _check_mlp(ml, where: str) -> None:
    kind = _need(ml, "kind", str, where)
    if kind == "dense":
        _need(ml, "ff", int, where)
    elif kind == "moe":
        r = _need(ml, "router", None, where)
        E, top = _need(r, "experts", int, where + ".router"), _need(r, "top", int, where + ".router")
        g = r.get("groups") or {}
        count = _need(g, "count", int, where + ".router.groups") if g else 1
        keep = _need(g, "keep", int, where + ".router.groups") if g else 1
        if E % count or keep > count or top > keep * (E // count):
            raise ConfigError(f"config.json: {where}.router: {top} of {E} experts in {keep} of {count} groups cannot be chosen")
        _need(_need(ml, "expert", None, where), "ff", int, where + ".expert")
    else:
        raise ConfigError(f"config.json: {where}.kind '{kind}' is not one of ('dense', 'moe')")


def _check_mixer(kind: str, mx, where: str) -> None:
    if kind == "mamba2":
        for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
            _need(mx, key, int, where)
        if mx["heads"] % mx["groups"] or (mx["heads"] * mx["vdim"]) % mx["norm_groups"]:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of groups, heads * vdim of norm_groups")
        return
    left, right = _need(mx, "left", None, where), _need(mx, "right", None, where)
    _need(mx, "left_scale", float, where)
    _need(mx, "right_scale", float, where)
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _need(left, key, int, where + ".left")
    _need(left, "scale", float, where + ".left")
    _need(_need(left, "mask", None, where + ".left"), "size", int, where + ".left.mask")
    rot = _need(left, "rot", None, where + ".left")
    _need(rot, "base", float, where + ".left.rot")
    dims = _need(rot, "dims", int, where + ".left.rot")
    if dims % 2 or dims > left["dim"]:
        raise ConfigError(f"config.json: {where}.left.rot.dims must be even and at most dim")
    if rot.get("scaling"):
        for key in ("factor", "original", "fast", "slow"):
            _need(rot["scaling"], key, float, where + ".left.rot.scaling")
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"config.json: {where}.left.heads must be a multiple of kv_heads")
    for key in ("heads", "dim", "vdim"):
        _need(right, key, int, where + ".right")
    decay = _need(right, "decay", None, where + ".right")
    if not isinstance(decay, (list, tuple)) or len(decay) != right["heads"] or \
            any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
        raise ConfigError(f"config.json: {where}.right.decay must be one number per head")


@dataclass(frozen=True)
class PepolornConfig(ModelConfig):
    architecture: ClassVar[str] = "Pepolorn"

    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PepolornConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=cls._get(raw, "vocab", int), width=cls._get(raw, "width", int),
                  norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"), layers=tuple(layers))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": [dict(L) for L in self.layers]}

    def source_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", str, where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {MIXERS}")
            _check_mixer(kind, _need(L, "mixer", None, where), where + ".mixer")
            if L.get("mlp") is not None:
                _check_mlp(L["mlp"], where + ".mlp")
            j = L.get("weights_of")
            if j is not None:
                if isinstance(j, bool) or not isinstance(j, int) or not (0 <= j < len(self.layers)) or j == i \
                        or self.layers[j].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer that has tensors of its own")
                a = {k: v for k, v in L.items() if k != "weights_of"}
                if a != dict(self.layers[j]):
                    raise ConfigError(f"config.json: {where} runs layer {j}'s weights but is described differently")
