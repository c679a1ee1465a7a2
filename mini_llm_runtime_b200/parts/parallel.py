"""Several mixers side by side on the same input, their results added with constant weights:
`result = sum_i scale_i * mixer_i(x)`.

The mixers are `SequenceCore`s (input projections -> core -> output projection), so the sum costs two
matrix products, not two per mixer: all input projections are ONE stacked product, every core reads its
columns of it and writes its columns of one activation buffer (already times its scale), and the output
projections, laid side by side along their inner dimension, are ONE product that also does the adding.
At most one of the mixers may keep keys and values and at most one a state (a run has one of each).
Parameters: mixers = [{"kind", "params", "weights", "scale"}, ...].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.base import ConfigError, PartSpec
from ..config.registry import part_class, register_part
from .base import Mixer, RunContext, SequenceCore, columns_of, pad_rows


class ParallelMixer(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.children: List[SequenceCore] = []
        self.scales: List[float] = []
        for entry in spec.params["mixers"]:
            child = part_class("mixer", entry["kind"])(PartSpec(entry["kind"], entry["params"], entry["weights"]))
            if not isinstance(child, SequenceCore):
                raise ConfigError(f"mixer kind {entry['kind']!r} cannot stand beside another (it is no SequenceCore)")
            self.children.append(child)
            self.scales.append(float(entry.get("scale", 1.0)))
        if not self.children:
            raise ConfigError("a parallel mixer needs at least one mixer")
        self.width = self.children[0].width
        if any(c.width != self.width for c in self.children):
            raise ConfigError("mixers side by side must share the model width")
        if sum(c.cache_need() is not None for c in self.children) > 1 or sum(c.state_need() is not None for c in self.children) > 1:
            raise ConfigError("of mixers side by side, at most one may keep keys and values and at most one a state")
        self.w_in = self.w_out = None

    def attach_positions(self, positions) -> None:
        for child in self.children:
            if hasattr(child, "attach_positions"):
                child.attach_positions(positions)

    def cache_need(self):
        return next((c.cache_need() for c in self.children if c.cache_need() is not None), None)

    def state_need(self):
        return next((c.state_need() for c in self.children if c.state_need() is not None), None)

    def weight_specs(self):
        return [s for c in self.children for s in c.weight_specs()]

    def kernel_modules(self, dtype) -> List[str]:
        return [m for c in self.children for m in c.kernel_modules(dtype)]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        stacked, self.first_in, at = [], [], 0
        for child in self.children:
            w = pad_rows(child.stacked_input(tensors, rt), 8)
            self.first_in.append(at)
            at += w.shape[0]
            stacked.append(w)
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        outs = [rt.matrix(tensors[c.spec.weights["o"]]) for c in self.children]
        self.first_out = [sum(o.shape[1] for o in outs[:i]) for i in range(len(outs))]
        self.w_out = torch.cat(outs, dim=1).contiguous()
        for child, scale in zip(self.children, self.scales):
            child.bind_core(tensors, rt, scale)

    def emit(self, b, x, run: RunContext):
        rt = b.rt
        proj = rt.linear(b, x, self.w_in, activation=True)
        act = b.temp(x.rows, self.w_out.shape[1], rt.dtype)
        for child, first_in, first_out in zip(self.children, self.first_in, self.first_out):
            child.emit_core(b, columns_of(proj, first_in, child.in_columns()[""]), columns_of(act, first_out, child.core_width()), run)
        return rt.linear(b, act, self.w_out, out_dtype=torch.float32)


register_part("mixer", "parallel", ParallelMixer)
