"""Small Gopevik configurations and random weights for the tests.  The configurations differ in every
size and option: width, vocabulary, norm groups (1 and more), layer order, heads equal to or a multiple
of the key/value heads, key and value sizes that differ, rotation of a part of a head or of all of it or
none, with and without position scaling, chunks that are no multiple of a cache page, convolutions of 2
to 5 taps, layers with and without a feed-forward."""
from __future__ import annotations

import copy
import math
from typing import Dict

import torch


def _parallel(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


SMALL_A = {
    "architecture": "Gopevik", "vocab": 97, "width": 48, "norm": {"eps": 1e-5, "groups": 3},
    "layers": [
        _delta(4, 4, 16, 8, 3, 40),
        _parallel({"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 16, "scale": 0.3, "mask": {"size": 24},
                   "rot": {"base": 100.0, "dims": 8}},
                  {"heads": 3, "dim": 16, "vdim": 24, "decay": [0.9, 0.97, 0.995], "rot": {"base": 1000.0, "dims": 16}},
                  1.3, 0.6, None),
        _parallel({"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 32, "scale": 0.25, "mask": {"size": 10},
                   "rot": {"base": 5000.0, "dims": 16, "scaling": {"factor": 2.5}}},
                  {"heads": 2, "dim": 40, "vdim": 8, "decay": [0.8, 0.99]},
                  0.7, 1.1, 56),
    ],
}

SMALL_B = {
    "architecture": "Gopevik", "vocab": 130, "width": 64, "norm": {"eps": 1e-6, "groups": 1},
    "layers": [
        _parallel({"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 37},
                   "rot": {"base": 10000.0, "dims": 4, "scaling": {"factor": 4.0}}},
                  {"heads": 1, "dim": 64, "vdim": 40, "decay": [0.98], "rot": {"base": 50.0, "dims": 2}},
                  1.0, 1.0, 72),
        _delta(2, 1, 32, 40, 2, None),
        _delta(6, 3, 8, 16, 5, 24),
    ],
}

# Only recurrent layers: the model keeps no keys and values at all.
SMALL_C = {
    "architecture": "Gopevik", "vocab": 61, "width": 32, "norm": {"eps": 1e-6, "groups": 4},
    "layers": [_delta(2, 2, 16, 16, 4, None), _delta(4, 2, 8, 8, 3, 48)],
}

# Sizes that miss every fast path: a width that is no multiple of 8, head sizes that are no multiple of 16 or 8,
# an odd number of rotated pairs, a chunk of one page and a bit, equal scales, one head everywhere.
SMALL_D = {
    "architecture": "Gopevik", "vocab": 77, "width": 36, "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        _parallel({"heads": 1, "kv_heads": 1, "dim": 12, "vdim": 20, "scale": 0.4, "mask": {"size": 9},
                   "rot": {"base": 30.0, "dims": 6, "scaling": {"factor": 1.5}}},
                  {"heads": 1, "dim": 10, "vdim": 6, "decay": [0.93], "rot": {"base": 400.0, "dims": 10}},
                  1.0, 1.0, 50),
        _delta(1, 1, 24, 12, 4, 22),
        _parallel({"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.2, "mask": {"size": 1000}},
                  {"heads": 2, "dim": 34, "vdim": 18, "decay": [0.5, 1.0]},
                  0.5, 2.0, None),
    ],
}

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "small_c": SMALL_C, "small_d": SMALL_D}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])


def random_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by their checkpoint names; matrices scaled so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).bfloat16()

    def vector(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * torch.randn(n, generator=g)).bfloat16()

    matrix("embed", config["vocab"], W, math.sqrt(W))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        vector(p + "norm1", W, 1.0, 0.1)
        vector(p + "norm1b", W, 1.0, 0.1)
        m = layer["mixer"]
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            matrix(p + "mix.left.q", l["heads"] * l["dim"], W, 2.0)
            matrix(p + "mix.left.k", l["kv_heads"] * l["dim"], W, 2.0)
            matrix(p + "mix.left.v", l["kv_heads"] * l["vdim"], W)
            matrix(p + "mix.left.g", l["heads"] * l["vdim"], W)
            matrix(p + "mix.left.o", W, l["heads"] * l["vdim"])
            matrix(p + "mix.right.q", r["heads"] * r["dim"], W)
            matrix(p + "mix.right.k", r["heads"] * r["dim"], W)
            matrix(p + "mix.right.v", r["heads"] * r["vdim"], W)
            matrix(p + "mix.right.g", r["heads"] * r["vdim"], W)
            matrix(p + "mix.right.o", W, r["heads"] * r["vdim"])
        else:
            qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            matrix(p + "mix.q", qk, W)
            matrix(p + "mix.k", qk, W)
            matrix(p + "mix.v", v, W)
            matrix(p + "mix.g", v, W)
            matrix(p + "mix.b", m["heads"], W)
            matrix(p + "mix.a", m["heads"], W)
            matrix(p + "mix.o", W, v)
            for role, n in (("q", qk), ("k", qk), ("v", v)):
                out[p + f"mix.{role}.conv"] = (torch.randn(n, m["conv"], generator=g) * 0.6).bfloat16()
            vector(p + "mix.A_log", m["heads"], -1.0, 1.0)
            vector(p + "mix.dt_bias", m["heads"], 0.0, 1.0)
            vector(p + "mix.norm", m["vdim"], 1.0, 0.1)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            vector(p + "norm2", W, 1.0, 0.1)
            vector(p + "norm2b", W, 1.0, 0.1)
            matrix(p + "mlp.gate", ff, W)
            matrix(p + "mlp.up", ff, W)
            matrix(p + "mlp.down", W, ff)
            vector(p + "mlp.gate.b", ff, 0.0, 0.3)
            vector(p + "mlp.up.b", ff, 0.0, 0.3)
            vector(p + "mlp.down.b", W, 0.0, 0.3)
    vector("final.norm", W, 1.0, 0.1)
    matrix("head", config["vocab"], W)
    return out
