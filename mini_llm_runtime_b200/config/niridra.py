"""Typed configuration of the Niridra decoder, read from its config.json.

    {"architecture": "Niridra", "vocab": V, "width": W, "norm": {"eps"}, "streams": S (optional),
     "embedding": {"scale", "bigram": {"buckets", "mul_prev", "mul_cur"} (optional)},
     "layers": [{"type": "lightning" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

A "lightning" mixer has heads, dim, vdim and one decay per head.  A "latent_attention" mixer has heads,
dim, vdim, kv_rank, scale and optionally kv_from (the index of an earlier latent layer whose cached
vectors it reads instead of making its own).  An "mlp" of kind "moe" has expert.ff, router.{experts, top,
groups.{count, keep} (optional)} and optionally shared.ff.  Every size and constant comes from the file;
a missing key is an error, not a default.  The design names no largest position; `max_positions` is this
engine's bound on a request's length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

from .base import ConfigError
from .gopevik import MAX_POSITIONS, _get, _integer, _number


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    kv_from: Optional[int]


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class NiridraLayer:
    type: str
    mixer: Any
    mlp: Optional[ExpertsConfig]


@dataclass(frozen=True)
class NiridraConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    streams: Optional[int]           # None: one stream and no connection weights
    embedding_scale: float
    pairs: Optional[PairTable]
    layers: Tuple[NiridraLayer, ...]
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
    def from_dict(cls, raw: dict) -> "NiridraConfig":
        width = _integer(raw, "width", "")
        norm = _get(raw, "norm", "")
        emb = _get(raw, "embedding", "")
        pairs = None
        if emb.get("bigram") is not None:
            t = emb["bigram"]
            pairs = PairTable(_integer(t, "buckets", "embedding.bigram."), _whole(t, "mul_prev", "embedding.bigram."),
                              _whole(t, "mul_cur", "embedding.bigram."))
        streams = _integer(raw, "streams", "") if raw.get("streams") is not None else None
        listed = _get(raw, "layers", "")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(listed):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where)
            m = _get(layer, "mixer", where)
            mw = where + "mixer."
            if kind == "lightning":
                heads = _integer(m, "heads", mw)
                decay = _get(m, "decay", mw)
                if not isinstance(decay, list) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                    raise ConfigError(f"config.json key {mw}'decay' must list one number per head ({heads})")
                mixer = LightningConfig(heads, _integer(m, "dim", mw), _integer(m, "vdim", mw), tuple(float(d) for d in decay))
            elif kind == "latent_attention":
                source = m.get("kv_from")
                rank = _integer(m, "kv_rank", mw)
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                        raise ConfigError(f"config.json key {mw}'kv_from' = {source!r} must name an earlier layer")
                    other = layers[source]
                    if other.type != "latent_attention" or other.mixer.kv_from is not None or other.mixer.kv_rank != rank:
                        raise ConfigError(f"config.json key {mw}'kv_from' = {source}: that layer keeps no latent of its own of "
                                          f"kv_rank {rank}")
                mixer = LatentConfig(_integer(m, "heads", mw), _integer(m, "dim", mw), _integer(m, "vdim", mw), rank,
                                     _number(m, "scale", mw), source)
            else:
                raise ConfigError(f"config.json key {where}'type' = {kind!r} is not one of 'lightning', 'latent_attention'")
            layers.append(NiridraLayer(kind, mixer, cls._mlp(layer.get("mlp"), where + "mlp.")))
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        return cls(architecture=_get(raw, "architecture", ""), vocab_size=_integer(raw, "vocab", ""), width=width,
                   norm_eps=_number(norm, "eps", "norm."), streams=streams, embedding_scale=_number(emb, "scale", "embedding.", positive=False),
                   pairs=pairs, layers=tuple(layers), max_position_embeddings=int(raw.get("max_positions", MAX_POSITIONS)),
                   eos_token_ids=eos)

    @staticmethod
    def _mlp(mlp: Optional[dict], where: str) -> Optional[ExpertsConfig]:
        if mlp is None:
            return None
        if _get(mlp, "kind", where) != "moe":
            raise ConfigError(f"config.json key {where}'kind' = {mlp['kind']!r}; this design has 'moe'")
        router = _get(mlp, "router", where)
        experts, top = _integer(router, "experts", where + "router."), _integer(router, "top", where + "router.")
        groups = keep = 1
        if router.get("groups") is not None:
            groups = _integer(router["groups"], "count", where + "router.groups.")
            keep = _integer(router["groups"], "keep", where + "router.groups.")
        if experts % groups or keep > groups or top > keep * (experts // groups):
            raise ConfigError(f"config.json {where}router: {experts} experts in {groups} groups of which {keep} are kept cannot give {top}")
        shared = mlp.get("shared")
        return ExpertsConfig(_integer(_get(mlp, "expert", where), "ff", where + "expert."), experts, top, groups, keep,
                             _integer(shared, "ff", where + "shared.") if shared is not None else None)


def _whole(raw: dict, key: str, where: str) -> int:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or not 0 <= value < (1 << 31):
        raise ConfigError(f"config.json key {where}{key!r} must be a non-negative integer, got {value!r}")
    return value
