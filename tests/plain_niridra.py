"""A plain, slow implementation of the Niridra decoder: one function per mechanism, whole sequences
at once, no cache, no batching, nothing shared with the package's compute path.

Everything is computed in the dtype of the tensors it is given (the tests use float64).  A model is
a config dictionary (the keys of config.json) and a dictionary of tensors by their checkpoint names.

    embedding   table[id] * scale + bigram[(prev * a + id * b) mod n]   (row n for a sequence's first token)
    streams     s copies of the vector; a sub-layer reads a weighted sum of them and its result goes
                back into every copy beside a mix of the old ones
    lightning   linear attention with a fixed decay per head, q, k, v through SiLU
    latent      attention whose keys and values are projections of one small vector per token
    experts     routed gated feed-forwards (group-limited choice) beside a gated shared one
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Which row of the bigram table each token of a sequence adds: a hash of the token before it and
    itself; the first token takes the table's extra last row."""
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embed(tokens: List[int], table: torch.Tensor, scale: float, bigram: Optional[torch.Tensor], buckets: int, mul_prev: int,
          mul_cur: int) -> torch.Tensor:
    x = table[torch.tensor(tokens)] * scale
    if bigram is not None:
        x = x + bigram[torch.tensor(bigram_rows(tokens, buckets, mul_prev, mul_cur))]
    return x


def streams_read(xs: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """xs [T, S, W]: the sub-layer's input, sum_s w_in[s] xs[:, s]."""
    return torch.einsum("tsw,s->tw", xs, w_in)


def streams_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """New copy t = sum_s mix[s, t] old copy s + w_out[t] y, all from the old copies."""
    return torch.einsum("tsw,sr->trw", xs, mix) + w_out[None, :, None] * y[:, None, :]


def lightning_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, Dv]: S <- decay_h S + k v^T; o = S^T q, token by token from S = 0."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype)
    d = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    k = silu(h @ w[p + "k"].T).reshape(T, H, D)
    v = silu(h @ w[p + "v"].T).reshape(T, H, Dv)
    o = lightning_attention(q, k, v, m["decay"]).reshape(T, H * Dv)
    o = rms_norm(o, w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The small vector per token that keys and values are made from."""
    return rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)


def latent_attention(h: torch.Tensor, c: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """h [T, W] queries' input, c [T, R] latents of the same positions.  Causal softmax attention, no positions."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, Dv)
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(H):
        s = (q[:, i] @ k[:, i].T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        out[:, i] = torch.softmax(s, dim=-1) @ v[:, i]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def gated_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int):
    """Per token: the chosen experts (by score + correction, within the `keep` best groups, a group's score
    being the sum of its two largest choice scores) and their weights (plain scores over their sum)."""
    s = torch.sigmoid(h @ w_router.T)                       # [T, E]
    choice = s + correction
    T, E = s.shape
    per = E // groups
    grouped = choice.reshape(T, groups, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(dim=-1)          # [T, groups]
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed[:, :, None].expand(T, groups, per).reshape(T, E), -math.inf)
    chosen = masked.topk(top, dim=-1).indices               # [T, top]
    weights = s.gather(1, chosen)
    weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)
    return chosen, weights


def experts_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h, w[p + "router"], w[p + "correction"], r["top"], groups["count"], groups["keep"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(chosen.shape[1]):
            e = int(chosen[t, j])
            out[t] += weights[t, j] * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    eps = config["norm"]["eps"]
    emb = config["embedding"]
    big = emb.get("bigram")
    x = embed(tokens, w["embed"], emb["scale"], w["bigram"] if big else None, big["buckets"] if big else 0,
              big["mul_prev"] if big else 0, big["mul_cur"] if big else 0)
    S = config.get("streams")
    xs = x[:, None, :].repeat(1, S or 1, 1)
    latents = {}
    one = torch.ones(1, dtype=x.dtype)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if layer.get(sub) is None:
                continue
            w_in, w_out, mix = (w[f"{p}hc{q}.in"], w[f"{p}hc{q}.out"], w[f"{p}hc{q}.mix"]) if S else (one, one, one[:, None])
            h = rms_norm(streams_read(xs, w_in), w[f"{p}norm{q}"], eps)
            if sub == "mlp":
                y = experts_feed_forward(h, w, p + "mlp.", layer["mlp"])
            elif layer["type"] == "lightning":
                y = lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)
            elif layer["type"] == "latent_attention":
                source = layer["mixer"].get("kv_from")
                if source is None:
                    latents[i] = latent_of(h, w, p + "mix.", eps)
                y = latent_attention(h, latents[i if source is None else source], w, p + "mix.", layer["mixer"])
            else:
                raise ValueError(layer["type"])
            xs = streams_write(xs, y * w[f"{p}ls{q}"], mix, w_out)
        if layers_out is not None:
            layers_out.append(xs.sum(dim=1))
    x = rms_norm(xs.sum(dim=1), w["final.norm"], eps)
    return x @ w["embed"].T
