"""Niridra as a model plan: an embedding with a hashed table of token pairs, a residual stream kept as
several copies that every sub-layer reads and writes through small learned weights (`streams` block),
layers whose mixer is either lightning attention (a decaying matrix state per head) or latent attention
(keys and values made from one cached vector per token, which a later layer may share), each followed by
routed experts or by nothing, and an output head that is the embedding table.  This module only turns a
`NiridraConfig` into data; the parts it names live in `parts/`.  Tensor names: `embed`, `bigram`,
`l<i>.norm1|norm2|ls1|ls2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelPlan, PartSpec, Run
from ..config.niridra import LatentConfig, LightningConfig, NiridraConfig
from ..config.registry import register_architecture


def niridra_plan(cfg: NiridraConfig) -> ModelPlan:
    width, streams = cfg.width, cfg.streams or 1
    norm = lambda name: PartSpec("rmsnorm", {"width": width, "eps": cfg.norm_eps}, {"weight": name})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LightningConfig):
            mixer = PartSpec("lightning", {"hidden_size": width, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim,
                                           "decay": list(m.decay), "eps": cfg.norm_eps},
                             {role: f"{p}mix.{role}" for role in ("q", "k", "v", "g", "o", "norm")})
            schedule.append(Run(i))
        elif isinstance(m, LatentConfig):
            roles = ("q", "uk", "uv", "o") if m.kv_from is not None else ("q", "dkv", "uk", "uv", "o")
            names = {role: f"{p}mix.{role}" for role in roles}
            if m.kv_from is None:
                names["dkv_norm"] = f"{p}mix.dkv.norm"
            mixer = PartSpec("latent_attention", {"hidden_size": width, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim,
                                                  "rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps,
                                                  "own_latent": m.kv_from is None}, names)
            schedule.append(Run(i, m.kv_from))
        else:
            raise TypeError(type(m).__name__)
        ff = None
        if layer.mlp is not None:
            e = layer.mlp
            names = {"router": p + "mlp.router", "correction": p + "mlp.correction"}
            for j in range(e.experts):
                names.update({f"e{j}.{role}": f"{p}mlp.e{j}.{role}" for role in ("gate", "up", "down")})
            if e.shared_ff is not None:
                names.update({f"shared.{role}": f"{p}mlp.shared.{role}" for role in ("gate", "up", "down", "sg")})
            ff = PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": e.ff, "experts": e.experts, "top": e.top,
                                             "groups": e.groups, "keep": e.keep, "shared_intermediate_size": e.shared_ff}, names)
        subs = (1, 2) if ff is not None else (1,)
        names = {f"scale{q}": f"{p}ls{q}" for q in subs}
        if cfg.streams is not None:
            for q in subs:
                names.update({f"in{q}": f"{p}hc{q}.in", f"out{q}": f"{p}hc{q}.out", f"mix{q}": f"{p}hc{q}.mix"})
        block = PartSpec("streams", {"width": width, "streams": streams, "connected": cfg.streams is not None}, names)
        norms = {"pre_mixer": norm(p + "norm1")}
        if ff is not None:
            norms["pre_feed_forward"] = norm(p + "norm2")
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ff, norms=norms))
    pairs = cfg.pairs
    embedding = PartSpec("hashed_embedding",
                         {"vocab_size": cfg.vocab_size, "width": width, "streams": streams, "scale": cfg.embedding_scale,
                          "buckets": pairs.buckets if pairs else 0, "mul_prev": pairs.mul_prev if pairs else 0,
                          "mul_cur": pairs.mul_cur if pairs else 0},
                         {"weight": "embed", **({"pairs": "bigram"} if pairs else {})})
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=embedding, positions={}, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("streams_rmsnorm", {"width": width, "streams": streams, "eps": cfg.norm_eps}, {"weight": "final.norm"}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "width": width}, {"weight": "embed"}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture("Niridra", NiridraConfig, niridra_plan)
