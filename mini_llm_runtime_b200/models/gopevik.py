"""Gopevik as a model plan: layers of two kinds in any order, each a block with norms on both sides of
its sub-layers (`sandwich`), grouped RMS norms, and either

  * a `parallel` mixer: attention within chunks of positions, with a sink in the softmax, partly rotated
    heads (linear position scaling), separate key and value sizes and a sigmoid gate, beside a retention
    mixer with a fixed decay per head; or
  * a `delta_rule` mixer behind short convolutions;

followed by a gated feed-forward with biases, or by none.  This module only turns a `GopevikConfig`
into data; the parts it names live in `parts/`.  Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelPlan, PartSpec, Run
from ..config.gopevik import DeltaMixerConfig, GopevikConfig, ParallelMixerConfig, Rotation
from ..config.registry import register_architecture


def _rotation_name(rot: Rotation) -> str:
    return f"rot_{rot.base!r}_{rot.dims}_{rot.factor!r}"


def gopevik_plan(cfg: GopevikConfig) -> ModelPlan:
    width = cfg.width
    norm = lambda name: PartSpec("group_rmsnorm", {"width": width, "groups": cfg.norm_groups, "eps": cfg.norm_eps}, {"weight": name})
    positions = {}

    def position(rot):
        if rot is None:
            return None
        name = _rotation_name(rot)
        positions[name] = PartSpec("rotary_frequencies", {"base": rot.base, "dims": rot.dims, "factor": rot.factor})
        return name

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, ParallelMixerConfig):
            l, r = m.left, m.right
            left = {"kind": "masked_attention", "scale": m.left_scale,
                    "params": {"hidden_size": width, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                               "value_dim": l.vdim, "scale": l.scale, "window": None, "chunk": l.chunk, "sink": True,
                               "gate": "sigmoid", "position": position(l.rot)},
                    "weights": {role: f"{p}mix.left.{role}" for role in ("q", "k", "v", "g", "o")}}
            right = {"kind": "retention", "scale": m.right_scale,
                     "params": {"hidden_size": width, "num_heads": r.heads, "head_dim": r.dim, "value_dim": r.vdim,
                                "decay": list(r.decay), "eps": cfg.norm_eps, "gate": "silu", "position": position(r.rot)},
                     "weights": {role: f"{p}mix.right.{role}" for role in ("q", "k", "v", "g", "o")}}
            mixer = PartSpec("parallel", {"mixers": [left, right]})
        elif isinstance(m, DeltaMixerConfig):
            names = {role: f"{p}mix.{role}" for role in ("q", "k", "v", "g", "b", "a", "o", "A_log", "dt_bias", "norm")}
            names.update({f"{role}_conv": f"{p}mix.{role}.conv" for role in ("q", "k", "v")})
            mixer = PartSpec("delta_rule", {"hidden_size": width, "num_heads": m.heads, "num_qk_heads": m.qk_heads, "head_dim": m.dim,
                                            "value_dim": m.vdim, "conv": m.conv, "eps": cfg.norm_eps}, names)
        else:
            raise TypeError(type(m).__name__)
        norms = {"pre_mixer": norm(p + "norm1"), "post_mixer": norm(p + "norm1b")}
        ff = None
        if layer.ff is not None:
            ff = PartSpec("gated_bias", {"hidden_size": width, "intermediate_size": layer.ff, "activation": "silu"},
                          {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down", "gate_bias": p + "mlp.gate.b",
                           "up_bias": p + "mlp.up.b", "down_bias": p + "mlp.down.b"})
            norms.update({"pre_feed_forward": norm(p + "norm2"), "post_feed_forward": norm(p + "norm2b")})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=ff, norms=norms))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": width}, {"weight": "embed"}),
        positions=positions, layers=tuple(layers), schedule=tuple(Run(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "width": width}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture("Gopevik", GopevikConfig, gopevik_plan)
