"""Typed configuration of the Gopevik decoder, read from its config.json.

    {"architecture": "Gopevik", "vocab": V, "width": W, "norm": {"eps", "groups"},
     "layers": [{"type": "parallel" | "delta", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A "parallel" mixer has "left" (grouped-query attention: heads, kv_heads, dim, vdim, scale, optional
mask.size = chunk of positions, optional rot = {base, dims, optional scaling.factor}), "right"
(retention: heads, dim, vdim, decay per head, optional rot) and the two weights left_scale and
right_scale.  A "delta" mixer has heads, kv_heads (heads of q and k), dim, vdim and conv (taps).
Every size and constant comes from the file; a missing key is an error, not a default.  The design
names no largest position; `max_positions` is this engine's bound on a request's length.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError

_LIMIT = 1_000_000
MAX_POSITIONS = 1 << 17


def _get(raw: dict, key: str, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks required key {where}{key!r}")
    return raw[key]


def _integer(raw: dict, key: str, where: str) -> int:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or not 1 <= value <= _LIMIT:
        raise ConfigError(f"config.json key {where}{key!r} must be an integer in [1, {_LIMIT}], got {value!r}")
    return value


def _number(raw: dict, key: str, where: str, positive: bool = True) -> float:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
        raise ConfigError(f"config.json key {where}{key!r} must be a finite number, got {value!r}")
    if positive and float(value) <= 0:
        raise ConfigError(f"config.json key {where}{key!r} = {value} must be positive")
    return float(value)


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    factor: float

    @classmethod
    def from_dict(cls, raw: Optional[dict], where: str, head: int) -> Optional["Rotation"]:
        if raw is None:
            return None
        dims = _integer(raw, "dims", where)
        if dims % 2 or dims > head:
            raise ConfigError(f"config.json key {where}'dims' = {dims} must be even and at most the head size {head}")
        scaling = raw.get("scaling")
        factor = _number(scaling, "factor", where + "scaling.") if scaling is not None else 1.0
        return cls(_number(raw, "base", where), dims, factor)


@dataclass(frozen=True)
class AttentionSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]
    rot: Optional[Rotation]


@dataclass(frozen=True)
class RetentionSide:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[Rotation]


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: AttentionSide
    right: RetentionSide
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    qk_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: Any
    ff: Optional[int]            # None: the layer has no feed-forward


@dataclass(frozen=True)
class GopevikConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[LayerConfig, ...]
    max_position_embeddings: int = MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict) -> "GopevikConfig":
        width = _integer(raw, "width", "")
        norm = _get(raw, "norm", "")
        groups = _integer(norm, "groups", "norm.")
        if width % groups:
            raise ConfigError(f"config.json: width {width} cannot be cut into norm.groups = {groups} equal parts")
        layers = []
        listed = _get(raw, "layers", "")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        for i, layer in enumerate(listed):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where)
            m = _get(layer, "mixer", where)
            if kind == "parallel":
                mixer = cls._parallel(m, where + "mixer.")
            elif kind == "delta":
                heads, qk = _integer(m, "heads", where + "mixer."), _integer(m, "kv_heads", where + "mixer.")
                if heads % qk:
                    raise ConfigError(f"config.json {where}mixer: {heads} heads cannot share {qk} q/k heads")
                mixer = DeltaMixerConfig(heads, qk, _integer(m, "dim", where + "mixer."), _integer(m, "vdim", where + "mixer."),
                                         _integer(m, "conv", where + "mixer."))
            else:
                raise ConfigError(f"config.json key {where}'type' = {kind!r} is not one of 'parallel', 'delta'")
            mlp = layer.get("mlp")
            ff = None
            if mlp is not None:
                if _get(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"config.json key {where}mlp.'kind' = {mlp['kind']!r}; this engine has 'dense'")
                ff = _integer(mlp, "ff", where + "mlp.")
            layers.append(LayerConfig(kind, mixer, ff))
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        return cls(architecture=_get(raw, "architecture", ""), vocab_size=_integer(raw, "vocab", ""), width=width,
                   norm_eps=_number(norm, "eps", "norm."), norm_groups=groups, layers=tuple(layers),
                   max_position_embeddings=int(raw.get("max_positions", MAX_POSITIONS)), eos_token_ids=eos)

    @staticmethod
    def _parallel(m: dict, where: str) -> ParallelMixerConfig:
        l, r = _get(m, "left", where), _get(m, "right", where)
        lw, rw = where + "left.", where + "right."
        heads, kv = _integer(l, "heads", lw), _integer(l, "kv_heads", lw)
        if heads % kv:
            raise ConfigError(f"config.json {lw}: {heads} query heads cannot share {kv} kv heads")
        dim = _integer(l, "dim", lw)
        mask = l.get("mask")
        left = AttentionSide(heads, kv, dim, _integer(l, "vdim", lw), _number(l, "scale", lw),
                             _integer(mask, "size", lw + "mask.") if mask is not None else None,
                             Rotation.from_dict(l.get("rot"), lw + "rot.", dim))
        rheads, rdim = _integer(r, "heads", rw), _integer(r, "dim", rw)
        decay = _get(r, "decay", rw)
        if not isinstance(decay, list) or len(decay) != rheads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"config.json key {rw}'decay' must list one number per head ({rheads})")
        right = RetentionSide(rheads, rdim, _integer(r, "vdim", rw), tuple(float(d) for d in decay),
                              Rotation.from_dict(r.get("rot"), rw + "rot.", rdim))
        return ParallelMixerConfig(left, right, _number(m, "left_scale", where, positive=False),
                                   _number(m, "right_scale", where, positive=False))
