"""Small Niridra configurations and random weights for the tests.  The configurations differ in every size
and option: width, vocabulary, copies of the stream (several, one with connection weights, none at all), with
and without the table of token pairs, layer order, latent layers that share an earlier layer's cache, more
than sixteen heads, a latent size that is no multiple of 16, routers with and without groups (one expert a
group, several kept groups, one chosen expert), with and without a shared expert, layers without a
feed-forward."""
from __future__ import annotations

import copy
import math
from typing import Dict

import torch


def _moe(ff, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def _latent(heads, dim, vdim, rank, scale, mlp, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


SMALL_A = {
    "architecture": "Niridra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "streams": 3,
    "embedding": {"scale": 3.5, "bigram": {"buckets": 53, "mul_prev": 11, "mul_cur": 5}},
    "layers": [
        _latent(4, 8, 12, 16, 0.4, _moe(24, 6, 2, (3, 2), 40)),
        _lightning(3, 16, 8, [0.7, 0.95, 1.0], _moe(32, 4, 1, None, None)),
        _latent(2, 24, 8, 16, 0.3, None, kv_from=0),
        _latent(5, 8, 8, 32, 0.25, _moe(16, 8, 3, (2, 1), 24)),
    ],
}

# One copy of the stream, with its connection weights; no pair table; only lightning layers (no cache at all).
SMALL_B = {
    "architecture": "Niridra", "vocab": 61, "width": 32, "norm": {"eps": 1e-6}, "streams": 1,
    "embedding": {"scale": 1.0},
    "layers": [_lightning(2, 32, 40, [0.9, 0.5], _moe(40, 3, 3, (3, 3), 16)), _lightning(1, 64, 16, [0.98], None)],
}

# No `streams` key: a plain residual sum with the scale vectors.  Sizes that miss every fast path: a width that is no
# multiple of 8, a latent that is no multiple of 16, twenty heads on one kv head, experts one a group.
SMALL_C = {
    "architecture": "Niridra", "vocab": 130, "width": 36, "norm": {"eps": 1e-5},
    "embedding": {"scale": 6.0, "bigram": {"buckets": 7, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        _latent(20, 4, 6, 12, 0.5, _moe(20, 5, 2, (5, 3), None)),
        _latent(3, 12, 20, 12, 0.2, _moe(12, 2, 1, (1, 1), 28), kv_from=0),
        _lightning(4, 10, 6, [0.6, 0.8, 0.9, 0.99], _moe(28, 16, 4, (4, 2), 12)),
    ],
}

# Many copies, a large pair table, sizes the tiled attention kernel takes (latent of 64) with prompts beyond one tile.
SMALL_D = {
    "architecture": "Niridra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "streams": 6,
    "embedding": {"scale": 8.0, "bigram": {"buckets": 1009, "mul_prev": 131, "mul_cur": 17}},
    "layers": [
        _lightning(2, 32, 32, [0.85, 0.97], _moe(48, 4, 2, (2, 2), 32)),
        _latent(2, 16, 16, 64, 0.25, _moe(32, 12, 2, (4, 1), 16)),
        _latent(16, 8, 4, 64, 0.35, None, kv_from=1),
    ],
}

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "small_c": SMALL_C, "small_d": SMALL_D}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])


def random_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by their checkpoint names; matrices scaled so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    W, S = config["width"], config.get("streams")
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).bfloat16()

    def vector(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * torch.randn(n, generator=g)).bfloat16()

    matrix("embed", config["vocab"], W, 1.0)
    pairs = config["embedding"].get("bigram")
    if pairs:
        matrix("bigram", pairs["buckets"] + 1, W, 2.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        vector(p + "norm1", W, 1.0, 0.1)
        vector(p + "ls1", W, 0.6, 0.2)
        if layer["type"] == "lightning":
            matrix(p + "mix.q", m["heads"] * m["dim"], W, 2.0)
            matrix(p + "mix.k", m["heads"] * m["dim"], W, 2.0)
            matrix(p + "mix.v", m["heads"] * m["vdim"], W, 2.0)
            matrix(p + "mix.g", m["heads"] * m["vdim"], W)
            matrix(p + "mix.o", W, m["heads"] * m["vdim"])
            vector(p + "mix.norm", m["heads"] * m["vdim"], 1.0, 0.1)
        else:
            matrix(p + "mix.q", m["heads"] * m["dim"], W, 2.0)
            if "kv_from" not in m:
                matrix(p + "mix.dkv", m["kv_rank"], W)
                vector(p + "mix.dkv.norm", m["kv_rank"], 1.0, 0.1)
            matrix(p + "mix.uk", m["heads"] * m["dim"], m["kv_rank"], 2.0)
            matrix(p + "mix.uv", m["heads"] * m["vdim"], m["kv_rank"])
            matrix(p + "mix.o", W, m["heads"] * m["vdim"])
        subs = [1]
        mlp = layer["mlp"]
        if mlp is not None:
            subs.append(2)
            vector(p + "norm2", W, 1.0, 0.1)
            vector(p + "ls2", W, 0.6, 0.2)
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                matrix(p + f"mlp.e{e}.gate", ff, W)
                matrix(p + f"mlp.e{e}.up", ff, W)
                matrix(p + f"mlp.e{e}.down", W, ff)
            matrix(p + "mlp.router", mlp["router"]["experts"], W, 2.0)
            vector(p + "mlp.correction", mlp["router"]["experts"], -0.3, 0.4)     # choices below zero too
            if mlp.get("shared") is not None:
                matrix(p + "mlp.shared.gate", mlp["shared"]["ff"], W)
                matrix(p + "mlp.shared.up", mlp["shared"]["ff"], W)
                matrix(p + "mlp.shared.down", W, mlp["shared"]["ff"])
                matrix(p + "mlp.shared.sg", 1, W, 2.0)
        if S:
            for q in subs:
                vector(p + f"hc{q}.in", S, 1.0 / S, 0.2)
                vector(p + f"hc{q}.out", S, 0.8, 0.3)
                out[p + f"hc{q}.mix"] = (torch.eye(S) + 0.15 * torch.randn(S, S, generator=g)).bfloat16()
    vector("final.norm", W, 1.0, 0.1)
    return out
