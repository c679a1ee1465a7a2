"""Pre-norm residual block: `h += mixer(norm(h))`, then `h += feed_forward(norm(h))`
(src/minillm/runtime.cpp:245-337; src/minillm/cuda/layer.cpp:42-70).

Each residual add is folded into a neighbouring kernel: either the sub-layer's last
product adds its result into `h` itself (it finds `h` in `step.residual` and returns
None), or its output is handed on as `pending` and added to `h` by the next norm's
kernel.  Either way the residual stream is read and written once per sub-layer.  Norm
slots: "pre_mixer", "pre_feed_forward".
"""
from __future__ import annotations

from ..config.registry import register_part
from .base import Block


class PreNormBlock(Block):
    def forward(self, h, pending, step, run):
        step.residual = h
        x = self.norms["pre_mixer"].forward(h, pending, step)
        mixed = self.mixer.forward(x, step, run)
        x = self.norms["pre_feed_forward"].forward(h, mixed, step)
        return self.feed_forward.forward(x, step)

    def first_norm(self):
        return self.norms["pre_mixer"]

    def emit(self, b, h, pending, run):
        b.residual = h
        after = b.norm_after_block
        x = self.norms["pre_mixer"].emit(b, h, pending)
        # Whoever adds into the stream is told which norm reads it next (a few-row product can leave it half done).
        b.norm_ahead = self.norms["pre_feed_forward"].foldable()
        mixed = self.mixer.emit(b, x, run)
        x = self.norms["pre_feed_forward"].emit(b, h, mixed)
        b.norm_ahead = after
        out = self.feed_forward.emit(b, x)
        b.norm_ahead = None
        return out


register_part("block", "pre_norm", PreNormBlock)


class SandwichBlock(Block):
    """Norms on both sides of each sub-layer: `h += post(mixer(pre(h)))`, then
    `h += post(feed_forward(pre(h)))`; a layer without a feed-forward has only the first.

    The sub-layers' results are contributions that a norm stands behind, so they are not added into the
    stream by their last product; the norm behind a sub-layer adds it and applies the norm before the
    next sub-layer in the same launch.  Norm slots: "pre_mixer", "post_mixer", "pre_feed_forward",
    "post_feed_forward"; the norms must offer `emit_residual` (the grouped RMS norm does)."""

    def forward(self, h, pending, step, run):
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step)
        out = self.emit(b, b.wrap(h), b.wrap(pending), run)
        return out.tensor if out is not None else None

    def first_norm(self):
        return self.norms["pre_mixer"]

    def emit(self, b, h, pending, run):
        b.residual = None            # nothing of this block is added into the stream by a product
        b.norm_ahead = None
        x = self.norms["pre_mixer"].emit(b, h, pending)
        mixed = self.mixer.emit(b, x, run)
        # The norm behind the block's last sub-layer also applies the first norm of the block that follows (the model
        # names it in `norm_after_block`), whose `emit` then finds the result in `prepared` and launches nothing.
        after = b.norm_after_block
        following = after[1] if after is not None and after[0] == "group_rms" else None
        last = "post_mixer" if self.feed_forward is None else "post_feed_forward"
        if following is not None and not self.norms[last].same_shape(following):
            following = None
        if self.feed_forward is None:
            ahead = self.norms["post_mixer"].emit_residual(b, h, mixed, then=following)
        else:
            x = self.norms["post_mixer"].emit_residual(b, h, mixed, then=self.norms["pre_feed_forward"])
            out = self.feed_forward.emit(b, x)
            ahead = self.norms["post_feed_forward"].emit_residual(b, h, out, then=following)
        b.prepared = {"group_rms": following, "stream": h, "out": ahead} if following is not None else None
        return None


register_part("block", "sandwich", SandwichBlock)
