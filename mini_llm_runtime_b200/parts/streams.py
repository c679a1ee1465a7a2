"""A residual stream kept as several copies (hyper-connections), with the embedding that starts it and
the norm that ends it.

    embedding   x = table[id] * scale + pairs[(prev * m_prev + id * m_cur) mod buckets]; every copy starts as x
                (`hashed_embedding`; the pair table is optional; a sequence's first token takes its last row;
                the token before a step's first row is kept per request)
    block       for sub-layer q (mixer, then feed-forward):  u = sum_s in_q[s] x_s;  y = sublayer(norm_q(u));
                x_t <- sum_s mix_q[s, t] x_s + out_q[t] * (scale_q .* y)      (`streams`)
                With one copy and no connection weights this is  x <- x + scale_q .* y.
    last norm   norm(sum_s x_s)                                                (`streams_rmsnorm`)

The stream is float32 [rows, copies * width].  One launch per sub-layer (`mlr_streams_step`) writes the
sub-layer's result into all copies and reads (and norms) the input of the next sub-layer, also across the
border to the next block: the block leaves that input on the builder (`prepared`), as the other blocks do.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import native
from ..weights.loader import WeightSpec
from .base import Block, Embedding, Norm, StateNeed

MAX_STREAMS = 16


class HashedEmbedding(Embedding):
    """Parameters: vocab_size, width, streams, scale, buckets (0: no pair table), mul_prev, mul_cur.
    Weights: "weight" [vocab, width], "pairs" [buckets + 1, width]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.vocab, self.width, self.streams = int(p["vocab_size"]), int(p["width"]), int(p.get("streams", 1))
        self.scale = float(p.get("scale", 1.0))
        self.buckets, self.mul_prev, self.mul_cur = int(p.get("buckets", 0)), int(p.get("mul_prev", 0)), int(p.get("mul_cur", 0))
        if not 1 <= self.streams <= MAX_STREAMS:
            raise ValueError(f"{self.streams} copies of the stream; the kernels take 1 to {MAX_STREAMS}")
        self.table = self.pairs = None
        self.state: Optional[torch.Tensor] = None       # [requests, 1] int32, given by the model when it allocates

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.spec.weights["weight"], (self.vocab, self.width))]
        if self.buckets:
            specs.append(WeightSpec(self.spec.weights["pairs"], (self.buckets + 1, self.width)))
        return specs

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((1,), torch.int32) if self.buckets else None

    def kernel_modules(self, dtype) -> List[str]:
        return ["streams"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.table = rt.shared_matrix(self.spec.weights["weight"], tensors)
        self.pairs = rt.matrix(tensors[self.spec.weights["pairs"]]) if self.buckets else None

    def emit(self, b):
        if self.buckets and self.state is None:
            raise native.KernelError("the embedding keeps the token before a step per request: allocate the model's cache first")
        h = b.temp(b.rows, self.streams * self.width, torch.float32)
        b.launch("streams", "mlr_embed_hashed", h.ptr, self.table.data_ptr(), self.pairs.data_ptr() if self.buckets else None,
                 native.is_bf16(self.table), b.meta("token_ids"), b.meta("segment_of_row"), b.meta("segment_info"),
                 self.state.data_ptr() if self.buckets else None, self.state.stride(0) if self.buckets else 0, b.rows, self.width,
                 self.vocab, self.streams, self.scale, self.buckets, self.mul_prev, self.mul_cur, b.status, b.stream)
        return h


class _FirstRead:
    """What a `streams` block tells the block before it: that block's last launch may read this block's first input."""

    def __init__(self, block):
        self.block = block

    def foldable(self):
        return ("streams", self.block)


class StreamsBlock(Block):
    """Parameters: width, streams, connected (False: one copy, no connection weights).  Weights: "scale1", "scale2" [width]
    and, when connected, "in<q>", "out<q>" [streams], "mix<q>" [streams, streams] ([from, to]); the second set only with a
    feed-forward.  Norm slots: "pre_mixer", "pre_feed_forward" (RMS norms over the width)."""

    def __init__(self, spec, mixer, feed_forward, norms):
        super().__init__(spec, mixer, feed_forward, norms)
        self.width, self.streams = int(spec.params["width"]), int(spec.params.get("streams", 1))
        self.connected = bool(spec.params.get("connected", True))
        if not 1 <= self.streams <= MAX_STREAMS or (not self.connected and self.streams != 1):
            raise ValueError(f"{self.streams} copies of the stream; the kernels take 1 to {MAX_STREAMS}, and one without connection weights")
        self.subs = (1, 2) if feed_forward is not None else (1,)
        self.w: Dict[str, torch.Tensor] = {}

    def weight_specs(self) -> List[WeightSpec]:
        w, S = self.spec.weights, self.streams
        specs = []
        for q in self.subs:
            specs.append(WeightSpec(w[f"scale{q}"], (self.width,), "vector", ("one_plus_normal", 0.01)))
            if self.connected:
                specs += [WeightSpec(w[f"in{q}"], (S,), "vector", ("normal", 0.5)), WeightSpec(w[f"out{q}"], (S,), "vector", ("normal", 0.5)),
                          WeightSpec(w[f"mix{q}"], (S, S), "vector", ("normal", 0.5))]
        return specs

    def kernel_modules(self, dtype) -> List[str]:
        return ["streams"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        names = self.spec.weights
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        for q in self.subs:
            self.w[f"scale{q}"] = f32(rt.vector(tensors[names[f"scale{q}"]]))
            self.w[f"norm{q}"] = f32(self.norms["pre_mixer" if q == 1 else "pre_feed_forward"].weight)    # bound before the block
            for role in ("in", "out", "mix"):
                if self.connected:
                    self.w[f"{role}{q}"] = f32(rt.vector(tensors[names[f"{role}{q}"]]))
                else:
                    self.w[f"{role}{q}"] = torch.ones((1, 1) if role == "mix" else (1,), dtype=torch.float32, device=rt.device)

    def first_norm(self):
        return _FirstRead(self)

    def same_shape(self, other) -> bool:
        return isinstance(other, StreamsBlock) and (other.width, other.streams) == (self.width, self.streams)

    def _step(self, b, h, y, q: Optional[int], then: Optional["StreamsBlock"], then_q: int = 1):
        """One launch: the write of sub-layer `q` with its result `y` (or none), and the read of sub-layer `then_q` of the
        block `then` (or none).  Returns the normed input that was read."""
        out = b.temp(h.rows, self.width, b.rt.dtype) if then is not None else None
        norm = then.norms["pre_mixer" if then_q == 1 else "pre_feed_forward"] if then is not None else None
        if y is not None and (y.slices or y.norm is not None or y.dtype is not torch.float32):
            raise native.KernelError("a sub-layer of a streams block hands over a plain float32 [rows, width] result")
        b.launch("streams", "mlr_streams_step", h.ptr, y.ptr if y is not None else None, y.ld if y is not None else 0,
                 self.w[f"scale{q}"].data_ptr() if y is not None else None, self.w[f"mix{q}"].data_ptr() if y is not None else None,
                 self.w[f"out{q}"].data_ptr() if y is not None else None, then.w[f"in{then_q}"].data_ptr() if then is not None else None,
                 then.w[f"norm{then_q}"].data_ptr() if then is not None else None, float(norm.eps) if norm is not None else 0.0,
                 out.ptr if out is not None else None, out.ld if out is not None else 0, int(b.rt.is_bf16), None, h.rows, self.width,
                 self.streams, b.stream)
        return out

    def forward(self, h, pending, step, run):
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step)
        self.emit(b, b.wrap(h), b.wrap(pending), run)
        return None

    def emit(self, b, h, pending, run):
        if pending is not None:
            raise native.KernelError("a streams block takes no pending contribution: the block before it must add its own")
        b.residual = None            # nothing of this block is added into the stream by a product
        b.norm_ahead = None
        prepared, b.prepared = b.prepared, None
        if isinstance(prepared, dict) and prepared.get("streams") is self and prepared.get("stream") is h:
            x = prepared["out"]      # the launch that ended the block before has read this block's first input already
        else:
            x = self._step(b, h, None, None, self)
        after = b.norm_after_block
        following = after[1] if after is not None and after[0] == "streams" and self.same_shape(after[1]) else None
        mixed = self.mixer.emit(b, x, run)
        if self.feed_forward is None:
            ahead = self._step(b, h, mixed, 1, following)
        else:
            x = self._step(b, h, mixed, 1, self, 2)
            out = self.feed_forward.emit(b, x)
            ahead = self._step(b, h, out, 2, following)
        b.prepared = {"streams": following, "stream": h, "out": ahead} if following is not None else None
        return None


class StreamsRmsNorm(Norm):
    """The RMS norm of the sum of the stream's copies (a model's last norm).  Parameters: width, streams, eps.
    Weights: "weight" [width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width, self.streams, self.eps = int(spec.params["width"]), int(spec.params.get("streams", 1)), float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", ("one_plus_normal", 0.01))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["streams"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.vector(tensors[self.spec.weights["weight"]]).to(torch.float32).contiguous()

    def emit(self, b, h, delta, wanted_only: bool = False):
        if delta is not None:
            raise native.KernelError("the norm over a stream's copies adds no pending contribution")
        b.prepared = None
        count = b.want if wanted_only else h.rows
        out = b.temp(count, self.width, b.rt.dtype)
        b.launch("streams", "mlr_streams_step", h.ptr, None, 0, None, None, None, None, self.weight.data_ptr(), self.eps, out.ptr, out.ld,
                 out.is_bf16, b.meta("want_rows") if wanted_only else None, count, self.width, self.streams, b.stream,
                 need="want" if wanted_only else None)
        return out


register_part("embedding", "hashed_embedding", HashedEmbedding)
register_part("block", "streams", StreamsBlock)
register_part("norm", "streams_rmsnorm", StreamsRmsNorm)
