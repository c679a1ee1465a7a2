"""Latent attention: keys and values of all heads are projections of one small vector per token, and only
that vector is cached.

    q = Wq x  [H, D];   c = rmsnorm(Wdkv x) * w  [R]  (the latent; cached);   k_h = Uk_h c,  v_h = Uv_h c
    o_h = softmax over j <= i of (q_h . k_hj) * scale, applied to v_hj;   result = o Wo^T        (no positions)

Because q_h . (Uk_h c) = (Uk_h^T q_h) . c  and  sum_j p_j Uv_h c_j = Uv_h sum_j p_j c_j,  the queries go through
Uk_h^T first (`mlr_head_project`), attention then runs on the cached latents themselves, as keys and as values
of one kv head shared by all query heads (`mlr_attention_masked` with shared_kv: a page holds one vector per
token), and its result goes through Uv_h (`mlr_head_project` again) before the output projection.  A mixer
without a latent of its own (`own_latent` False) has no Wdkv: its run reads the cache of the run the plan names
(`Run.kv_from`), with its own Uk, Uv and queries.

Parameters: hidden_size, num_heads, head_dim, value_dim, rank, scale, eps (of the latent's norm), own_latent.
Weights: "q" [H D, W], "dkv" [R, W], "dkv_norm" [R] (both only with a latent of its own), "uk" [H D, R],
"uv" [H Dv, R], "o" [W, H Dv].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import functions as F
from ..ops import native
from ..ops.specs import GATES, MaskedAttentionSpec
from ..weights.loader import WeightSpec
from .base import CacheNeed, Mixer, RunContext, columns_of, pad_rows
from .masked_attention import emit_masked_attention


class LatentAttentionMixer(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.dim, self.vdim, self.rank = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"]), int(p["rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.own_latent = bool(p.get("own_latent", True))
        if not 1 <= self.rank <= 1024:
            raise ConfigError(f"a latent of {self.rank} values is outside what the attention kernel takes as a key and value (1 to 1024)")
        self.desc: Optional[MaskedAttentionSpec] = None

    def cache_need(self) -> CacheNeed:
        # One kv head whose keys are the latents; value size 0: the values are the keys and take no room of their own.
        return CacheNeed(None, 1, self.rank, 0)

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        specs = [WeightSpec(w["q"], (self.heads * self.dim, self.width)), WeightSpec(w["uk"], (self.heads * self.dim, self.rank)),
                 WeightSpec(w["uv"], (self.heads * self.vdim, self.rank)), WeightSpec(w["o"], (self.width, self.heads * self.vdim))]
        if self.own_latent:
            specs += [WeightSpec(w["dkv"], (self.rank, self.width)),
                      WeightSpec(w["dkv_norm"], (self.rank,), "vector", ("one_plus_normal", 0.01))]
        return specs

    def kernel_modules(self, dtype) -> List[str]:
        return ["latent", "attention_masked"] + (["experts"] if dtype is torch.bfloat16 else []) + F.product_modules(dtype)

    def _per_head(self, b, x, w, w_t, y, inputs: int, outputs: int) -> None:
        """y[m, h, :] = x[m, h, :] W_h: on the tensor cores (the batched product of `experts.cu`) for bfloat16 rows on 16-byte
        borders, else on the CUDA cores."""
        if b.rt.is_bf16 and native.module("experts").mlr_experts_tensor_cores(inputs, x.ld) and x.ptr % 16 == 0:
            b.launch("experts", "mlr_batched_product_bf16", x.ptr, x.ld, w_t.data_ptr(), y.ptr, y.ld, x.rows, self.heads, outputs, inputs, b.stream)
        else:
            b.launch("latent", "mlr_head_project", x.ptr, x.ld, w.data_ptr(), y.ptr, y.ld, x.is_bf16, x.rows, self.heads, inputs, outputs, b.stream)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        stacked = [rt.matrix(tensors[w["q"]])] + ([rt.matrix(tensors[w["dkv"]])] if self.own_latent else [])
        self.w_in = pad_rows(torch.cat(stacked, dim=0), 8)
        self.w_out = rt.matrix(tensors[w["o"]])
        # [heads, D, R] as stored; [heads, R, Dv] transposed, so that both per-head products read rows of their matrix.
        self.w_uk = rt.matrix(tensors[w["uk"]]).view(self.heads, self.dim, self.rank).contiguous()
        self.w_uv = rt.matrix(tensors[w["uv"]]).view(self.heads, self.vdim, self.rank).transpose(1, 2).contiguous()
        # The same two as [heads, outputs, inputs], the operand layout of the tensor-core product (bfloat16 only).
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous() if rt.is_bf16 else None
        self.w_uv_t = self.w_uv.transpose(1, 2).contiguous() if rt.is_bf16 else None
        self.latent_weight = rt.vector(tensors[w["dkv_norm"]]).float().contiguous() if self.own_latent else None
        self.desc = MaskedAttentionSpec(freq=None, heads=self.heads, kv_heads=1, dim=self.rank, vdim=self.rank, rot_dims=0, window=0,
                                        chunk=0, sink=0, gate_kind=GATES[None], shared_kv=1, scale=self.scale, out_scale=1.0)

    def emit(self, b, x, run: RunContext):
        rt = b.rt
        if run.cache is None or run.cache.dtype is not rt.dtype:
            raise native.KernelError("latent attention: the cache must have the activations' precision")
        if run.write_cache != self.own_latent:
            raise native.KernelError("latent attention: a mixer with a latent of its own writes its cache, one without reads another's")
        proj = rt.linear(b, x, self.w_in, activation=True)
        rows = proj.rows
        if self.own_latent:
            down = columns_of(proj, self.heads * self.dim, self.rank)
            b.launch("latent", "mlr_latent_cache", down.ptr, down.ld, proj.is_bf16, self.latent_weight.data_ptr(), 1, self.eps, self.rank,
                     run.cache.data_ptr(), run.cache.shape[0], b.meta("positions"), b.meta("segment_of_row"), b.table(run.group),
                     b.table_stride(run.group), b.page_size, rows, b.status, b.stream)
        wide = self.heads * self.rank
        q = b.temp(rows, wide, rt.dtype)
        self._per_head(b, proj, self.w_uk, self.w_uk_t, q, self.dim, self.rank)
        mixed = b.temp(rows, wide, rt.dtype)
        emit_masked_attention(b, self.desc, q, None, mixed, run)
        act = b.temp(rows, self.heads * self.vdim, rt.dtype)
        self._per_head(b, mixed, self.w_uv, self.w_uv_t, act, self.rank, self.vdim)
        return rt.linear(b, act, self.w_out, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttentionMixer)
