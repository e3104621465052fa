"""Typed configuration of the Kolorax design.

``config.json`` names the design under ``architecture`` and gives every size and constant:

    vocab, width, residual_mult, embedding.scale, norm.eps
    layers[i]: type ("wkv" | "latent_attention"), mixer {...}, mlp {...} | null
        wkv mixer:              heads, dim  (decay_rank: rows of the decay's first matrix; a model folder
                                need not give it, the tensor's shape does)
        latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}
        mlp (kind "moe"):       router {experts, top, groups {count, keep}}, expert {ff, limit},
                                shared {ff, limit} | null
    loop {start, stop, times} | null: layers start .. stop-1 run ``times`` times in a row

The nested objects are kept as they are (frozen by convention) and checked here, so that a wrong or
missing key is told by name before anything is built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig

MIXERS = ("wkv", "latent_attention")


def _need(obj: Mapping[str, Any], key: str, typ, where: str):
    if not isinstance(obj, Mapping) or key not in obj or obj[key] is None:
        raise ConfigError(f"config.json: {where} needs '{key}'")
    v = obj[key]
    if typ is int:
        if isinstance(v, bool) or not (isinstance(v, int) or (isinstance(v, float) and v == int(v))):
            raise ConfigError(f"config.json: {where}.{key} must be an integer, got {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        return float(v)
    return v


@dataclass(frozen=True)
class KoloraxConfig(ModelConfig):
    architecture: ClassVar[str] = "Kolorax"

    vocab: int
    width: int
    residual_mult: float
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]
    loop: Optional[Mapping[str, int]] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KoloraxConfig":
        g = cls._get
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = raw.get("loop")
        cfg = cls(
            vocab=g(raw, "vocab", int), width=g(raw, "width", int),
            residual_mult=g(raw, "residual_mult", float, 1.0),
            embedding_scale=_need(raw.get("embedding") or {"scale": 1.0}, "scale", float, "embedding"),
            norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
            layers=tuple(layers),
            loop=None if not loop else {k: _need(loop, k, int, "loop") for k in ("start", "stop", "times")},
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps}, "layers": [dict(L) for L in self.layers]}
        if self.loop:
            out["loop"] = dict(self.loop)
        return out

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
            mx = _need(L, "mixer", None, where)
            for key in ("heads", "dim"):
                if _need(mx, key, int, f"{where}.mixer") <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.{key} must be positive")
            if kind == "latent_attention":
                for key in ("rot_dim", "vdim", "kv_rank"):
                    _need(mx, key, int, f"{where}.mixer")
                _need(mx, "scale", float, f"{where}.mixer")
                rot = _need(mx, "rot", None, f"{where}.mixer")
                _need(rot, "base", float, f"{where}.mixer.rot")
                dims = int(rot.get("dims", mx["rot_dim"]))
                if dims > int(mx["rot_dim"]) or dims % 2 or dims < 0:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most rot_dim "
                                      f"(the rotated vector is the rot_dim part)")
            ml = L.get("mlp")
            if ml is not None:
                if ml.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{ml.get('kind')}' is not supported (moe only)")
                r = _need(ml, "router", None, f"{where}.mlp")
                _need(r, "experts", int, f"{where}.mlp.router")
                _need(r, "top", int, f"{where}.mlp.router")
                ex = _need(ml, "expert", None, f"{where}.mlp")
                _need(ex, "ff", int, f"{where}.mlp.expert")
                _need(ex, "limit", float, f"{where}.mlp.expert")
                if ml.get("shared") is not None:
                    _need(ml["shared"], "ff", int, f"{where}.mlp.shared")
                    _need(ml["shared"], "limit", float, f"{where}.mlp.shared")
        if self.loop:
            a, b, n = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= len(self.layers)) or n < 1:
                raise ConfigError(f"config.json: loop {dict(self.loop)} does not fit {len(self.layers)} layers")


def file_hints(raw: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Mapping[str, Any]:
    """Sizes that only the tensors' shapes give: the rank of each wkv layer's decay projection."""
    layers = raw.get("layers")
    if not isinstance(layers, list):
        return raw
    out = []
    for i, L in enumerate(layers):
        name = f"l{i}.mix.w1"
        if isinstance(L, dict) and L.get("type") == "wkv" and isinstance(L.get("mixer"), dict) \
                and "decay_rank" not in L["mixer"] and name in shapes and len(shapes[name]) == 2:
            L = dict(L, mixer=dict(L["mixer"], decay_rank=int(shapes[name][0])))
        out.append(L)
    return dict(raw, layers=out)
