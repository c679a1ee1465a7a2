"""A plain, slow implementation of the Gopevik decoder: one function per mechanism, whole
sequences at once, no cache, no batching, nothing shared with the package's compute path.

Everything is computed in the dtype of the tensors it is given (the tests use float64).
A model is a config dictionary (the keys of config.json) and a dictionary of tensors by
their checkpoint names.

    layer      x <- x + norm_b(mixer(norm(x)));  x <- x + norm_b(ff(norm(x)))  (the second only with a feed-forward)
    norm       the vector in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times a weight
    parallel   left_scale * chunked attention with a sink  +  right_scale * retention
    delta      gated delta rule behind short causal convolutions
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def group_rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], groups: int, eps: float) -> torch.Tensor:
    """x [..., W]: every one of `groups` consecutive parts over its own root mean square."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    out = parts.reshape(shape)
    return out if weight is None else out * weight


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float = 1.0) -> torch.Tensor:
    """x [T, heads, D]: the first `dims` values of every head turned by position * base^(-2i/dims) / factor,
    value i paired with value i + dims/2; the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims) / factor
    angle = positions.to(x.dtype)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def chunk_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, scale: float,
                         chunk: Optional[int]) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads kv head h // (H/G).  A query at position i sees
    j <= i of its own chunk (i // chunk == j // chunk); the softmax has 1 added to its denominator."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    pi, pj = positions[:, None], positions[None, :]
    seen = pj <= pi
    if chunk:
        seen = seen & (pi // chunk == pj // chunk)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)        # the sink's score is 0
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))
        out[:, h] = p @ v[:, g]
    return out


def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float], state: Optional[torch.Tensor] = None):
    """q, k [T, H, D], v [T, H, Dv]: S <- decay_h S + k v^T, o = S^T q, token by token.  Returns (o, S)."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    d = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def short_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, j] x_(t - n + 1 + j) with zeros before the start, then silu."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j]
    return y * torch.sigmoid(y)


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor):
    """q, k [T, H, D], v [T, H, Dv], g and beta [T, H].  Per head and token: S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def silu(x):
    return x * torch.sigmoid(x)


def parallel_mixer(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    L, R = m["left"], m["right"]
    H, G, D, Dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
    q = (h @ w[p + "left.q"].T).view(T, H, D)
    k = (h @ w[p + "left.k"].T).view(T, G, D)
    v = (h @ w[p + "left.v"].T).view(T, G, Dv)
    rot = L.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_half(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_half(k, positions, rot["dims"], rot["base"], factor)
    o = chunk_sink_attention(q, k, v, positions, L["scale"], (L.get("mask") or {}).get("size"))
    o = o.reshape(T, H * Dv) * torch.sigmoid(h @ w[p + "left.g"].T)
    left = o @ w[p + "left.o"].T

    H, D, Dv = R["heads"], R["dim"], R["vdim"]
    q = (h @ w[p + "right.q"].T).view(T, H, D)
    k = (h @ w[p + "right.k"].T).view(T, H, D)
    v = (h @ w[p + "right.v"].T).view(T, H, Dv)
    rot = R.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_half(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_half(k, positions, rot["dims"], rot["base"], factor)
    k = k * D ** -0.5
    o, _ = retention(q, k, v, R["decay"])
    o = group_rms_norm(o, None, 1, eps).reshape(T, H * Dv) * silu(h @ w[p + "right.g"].T)
    right = o @ w[p + "right.o"].T
    return m["left_scale"] * left + m["right_scale"] * right


def delta_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(T, H, Dv)
    q = unit(q) * D ** -0.5
    k = unit(k)
    share = H // G
    q = q.repeat_interleave(share, dim=1)
    k = k.repeat_interleave(share, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = gated_delta_rule(q, k, v, g, beta)
    o = group_rms_norm(o, None, 1, eps) * w[p + "norm"]
    o = o.reshape(T, H * Dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence from position 0; `layers_out` collects the stream after every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    groups, eps = config["norm"]["groups"], config["norm"]["eps"]
    norm = lambda x, name: group_rms_norm(x, w[name], groups, eps)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    positions = torch.arange(x.shape[0])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = norm(x, p + "norm1")
        if layer["type"] == "parallel":
            mixed = parallel_mixer(h, positions, layer["mixer"], w, p + "mix.", eps)
        elif layer["type"] == "delta":
            mixed = delta_mixer(h, layer["mixer"], w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm(mixed, p + "norm1b")
        if layer.get("mlp") is not None:
            x = x + norm(dense_feed_forward(norm(x, p + "norm2"), w, p + "mlp."), p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, "final.norm") @ w["head"].T
