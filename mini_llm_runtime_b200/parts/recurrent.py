"""Mixers with a matrix state per head and request (linear attention): retention with a fixed decay
per head, and the gated delta rule behind short convolutions.  Both are the kernel
`mlr_linear_recurrence` (csrc/kernels/recurrence.cu) under two descriptions.

Retention:   q, k [H, D], v [H, Dv];  q, k rotated on their first values;  k *= D^(-1/2);
             S <- decay_h S + k v^T;  o = S^T q;  o / rms(o) per head, times silu(g);  result = o Wo^T.
Delta rule:  q, k [G, D] (head h uses q/k head h // (H/G)), v [H, Dv], each through a causal convolution
             over time per channel and silu;  q, k made unit vectors, q *= D^(-1/2);
             beta = sigmoid(Wb x);  g = exp(-exp(A_log) softplus(Wa x + dt_bias));
             S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
             o / rms(o) per head times a weight [Dv], times silu(Wg x);  result = o Wo^T.

The state (float32, [H, Dv, D] per request, for the delta rule followed by the last taps-1 inputs of
the convolutions) lives in the model's state slots; a new request starts from zeros.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import functions as F
from ..ops.specs import GATES, RecurrenceSpec, address
from ..weights.loader import WeightSpec
from .base import RunContext, SequenceCore, StateNeed, columns_of


def emit_recurrence(b, mixer, proj, side, act, run: RunContext) -> None:
    """The recurrence of `mixer.desc` over the step's rows: q, k, v from `proj`, the rule's inputs and the gate
    from `side`, the result into `act`.  Few rows: one kernel.  Many: prepare, scan, read-out."""
    state, info = run.state, b.meta("segment_info")
    d = mixer.desc
    if b.le(proj.rows, b.rt.recurrence_fused_rows):
        # A read-out that norms all heads of a token together cannot happen in a block that owns one head: the kernel then
        # leaves its plain float32 outputs in a buffer and the read-out is a second launch.
        plain = b.temp(proj.rows, d.heads * d.vdim, torch.float32) if d.norm_all else None
        b.launch("recurrence", "mlr_linear_recurrence", address(d), proj.ptr, proj.ld, side.ptr, side.ld, proj.is_bf16,
                 act.ptr, act.ld, state.data_ptr(), state.stride(0), info, b.segments, proj.rows, plain.ptr if plain else None,
                 b.status, b.stream)
        return
    qf = b.temp(proj.rows, d.qk_heads * d.dim, torch.float32)
    kf = b.temp(proj.rows, d.qk_heads * d.dim, torch.float32)
    gates = b.temp(proj.rows, 2 * d.heads, torch.float32)
    obuf = b.temp(proj.rows, d.heads * d.vdim, torch.float32)
    b.launch("recurrence", "mlr_linear_recurrence_split", address(d), proj.ptr, proj.ld, side.ptr, side.ld, proj.is_bf16, act.ptr,
             act.ld, state.data_ptr(), state.stride(0), info, b.segments, b.meta("positions"), proj.rows, qf.ptr, kf.ptr, gates.ptr,
             obuf.ptr, b.stream)


def _check_state_size(dim: int, vdim: int) -> None:
    if not (1 <= dim <= 256 and 1 <= vdim <= 256) or (dim > 128 and vdim > 128):
        raise ConfigError(f"a state of {dim} x {vdim} per head is more than the recurrence kernel keeps in registers "
                          f"(256 x 128 or 128 x 256)")


class RetentionMixer(SequenceCore):
    """Parameters: hidden_size, num_heads, head_dim, value_dim, decay (one per head), eps (of the norm per
    head), position (name of a `rotary_frequencies` encoding, or None), gate (None | "silu" | "sigmoid").
    Weights: "q", "k" [H D, W], "v", "g" [H Dv, W], "o" [W, H Dv]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"])
        self.decay = [float(d) for d in p["decay"]]
        self.eps = float(p["eps"])
        self.gate = p.get("gate", "silu")
        self.position_name = p.get("position")
        self.position = None
        if len(self.decay) != self.heads:
            raise ConfigError(f"{len(self.decay)} decays for {self.heads} heads")
        _check_state_size(self.dim, self.vdim)
        self.desc: Optional[RecurrenceSpec] = None

    def attach_positions(self, positions) -> None:
        if self.position_name is not None:
            self.position = positions[self.position_name]
            if self.position.dims > self.dim:
                raise ConfigError(f"{self.position.dims} rotated values do not fit a head of {self.dim}")

    def state_need(self) -> StateNeed:
        return StateNeed((self.heads * self.vdim * self.dim,), torch.float32)

    def in_roles(self) -> List[Tuple[str, int]]:
        roles = [("q", self.heads * self.dim), ("k", self.heads * self.dim), ("v", self.heads * self.vdim)]
        return roles + ([("g", self.heads * self.vdim)] if self.gate else [])

    def core_width(self) -> int:
        return self.heads * self.vdim

    def kernel_modules(self, dtype) -> List[str]:
        return ["recurrence"] + F.product_modules(dtype)

    def bind_core(self, tensors, rt, out_scale: float) -> None:
        at = self.in_columns()
        freq = self.position.frequencies() if self.position is not None else None
        self._held = (freq, torch.tensor(self.decay, dtype=torch.float32, device=rt.device))
        rotate = freq is not None and freq.numel() > 0
        self.desc = RecurrenceSpec(
            freq=freq.data_ptr() if rotate else None, decay=self._held[1].data_ptr(), heads=self.heads, qk_heads=self.heads,
            dim=self.dim, vdim=self.vdim, prep=RecurrenceSpec.PREP["rotate" if rotate else None],
            rot_dims=self.position.dims if rotate else 0, rule=RecurrenceSpec.RULE["decay"], gate_kind=GATES[self.gate],
            col_q=at["q"], col_k=at["k"], col_v=at["v"], col_gate=at.get("g", 0), q_mult=1.0, k_mult=float(self.dim) ** -0.5,
            unit_eps=0.0, eps=self.eps, out_scale=float(out_scale))

    def emit_core(self, b, proj, act, run: RunContext) -> None:
        emit_recurrence(b, self, proj, proj, act, run)


class DeltaRuleMixer(SequenceCore):
    """Parameters: hidden_size, num_heads, num_qk_heads, head_dim, value_dim, conv (taps), eps.
    Weights: "q", "k" [G D, W], "v", "g" [H Dv, W], "b", "a" [H, W], "o" [W, H Dv], "q_conv", "k_conv" [G D, taps],
    "v_conv" [H Dv, taps], "A_log", "dt_bias" [H], "norm" [Dv]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.qk_heads = int(p["num_heads"]), int(p["num_qk_heads"])
        self.dim, self.vdim, self.taps = int(p["head_dim"]), int(p["value_dim"]), int(p["conv"])
        self.eps = float(p["eps"])
        if self.heads % self.qk_heads:
            raise ConfigError(f"{self.heads} heads cannot share {self.qk_heads} q/k heads")
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"a convolution of {self.taps} taps is outside what the kernel takes (1 to 16)")
        _check_state_size(self.dim, self.vdim)
        self.channels = 2 * self.qk_heads * self.dim + self.heads * self.vdim
        self.matrix_floats = self.heads * self.vdim * self.dim
        self.desc: Optional[RecurrenceSpec] = None

    def state_need(self) -> StateNeed:
        return StateNeed((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def in_roles(self) -> List[Tuple[str, int]]:
        return [("q", self.qk_heads * self.dim), ("k", self.qk_heads * self.dim), ("v", self.heads * self.vdim),
                ("g", self.heads * self.vdim), ("b", self.heads), ("a", self.heads)]

    def core_width(self) -> int:
        return self.heads * self.vdim

    def extra_weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["q_conv"], (self.qk_heads * self.dim, self.taps), "vector", ("normal", 0.3)),
                WeightSpec(w["k_conv"], (self.qk_heads * self.dim, self.taps), "vector", ("normal", 0.3)),
                WeightSpec(w["v_conv"], (self.heads * self.vdim, self.taps), "vector", ("normal", 0.3)),
                WeightSpec(w["A_log"], (self.heads,), "vector", ("normal", 0.5)),
                WeightSpec(w["dt_bias"], (self.heads,), "vector", ("normal", 0.5)),
                WeightSpec(w["norm"], (self.vdim,), "vector", ("one_plus_normal", 0.01))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["recurrence"] + F.product_modules(dtype)

    def bind_core(self, tensors, rt, out_scale: float) -> None:
        w = self.spec.weights
        vec = lambda role: rt.vector(tensors[w[role]]).float().contiguous()
        self.taps_weight = torch.cat([vec("q_conv"), vec("k_conv"), vec("v_conv")], dim=0).contiguous()
        self._held = (vec("A_log"), vec("dt_bias"), vec("norm"))
        at = self.in_columns()
        # q, k, v are the first columns of the projections' output and, convolved, all columns of a buffer of
        # their own; b, a and the gate are read from the projections' output.
        self.desc = RecurrenceSpec(
            a_log=self._held[0].data_ptr(), dt_bias=self._held[1].data_ptr(), out_weight=self._held[2].data_ptr(), heads=self.heads,
            qk_heads=self.qk_heads, dim=self.dim, vdim=self.vdim, prep=RecurrenceSpec.PREP["unit"], rot_dims=0,
            rule=RecurrenceSpec.RULE["delta"], gate_kind=GATES["silu"], col_q=at["q"], col_k=at["k"], col_v=at["v"],
            col_a=at["a"], col_b=at["b"], col_gate=at["g"], q_mult=float(self.dim) ** -0.5, k_mult=1.0, unit_eps=1e-6, eps=self.eps,
            out_scale=float(out_scale))

    def emit_core(self, b, proj, act, run: RunContext) -> None:
        # q, k, v pass the convolutions into a buffer of their own (a row's other tokens read the
        # projections' output meanwhile); then the convolutions' state moves on; the recurrence reads q, k, v
        # from the convolved buffer and b, a and the gate from the projections' output.
        state = run.state
        conv_state = state.data_ptr() + 4 * self.matrix_floats
        stride = state.stride(0)
        info, of_row = b.meta("segment_info"), b.meta("segment_of_row")
        conv = b.temp(proj.rows, self.channels, proj.dtype)
        b.launch("recurrence", "mlr_short_conv", proj.ptr, proj.ld, conv.ptr, conv.ld, proj.is_bf16, self.channels, self.taps,
                 self.taps_weight.data_ptr(), conv_state, stride, info, of_row, proj.rows, b.stream)
        b.launch("recurrence", "mlr_short_conv_state", proj.ptr, proj.ld, proj.is_bf16, self.channels, self.taps, conv_state, stride,
                 info, b.segments, b.stream)
        emit_recurrence(b, self, conv, proj, act, run)


register_part("mixer", "retention", RetentionMixer)
register_part("mixer", "delta_rule", DeltaRuleMixer)


class LightningMixer(SequenceCore):
    """Lightning attention: linear attention with a fixed decay per head, no positions and no scale.

        q, k = silu(Wq x), silu(Wk x) [H, D];  v = silu(Wv x) [H, Dv];  S <- decay_h S + k v^T;  o = S^T q;
        all heads of a token together over their root mean square, times a weight [H Dv], times sigmoid(Wg x);  result = o Wo^T.

    Parameters: hidden_size, num_heads, head_dim, value_dim, decay (one per head), eps.  Weights: "q", "k" [H D, W],
    "v", "g" [H Dv, W], "o" [W, H Dv], "norm" [H Dv].  The state is the retention mixer's: float32 [H, Dv, D] per request."""

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"])
        self.decay = [float(d) for d in p["decay"]]
        self.eps = float(p["eps"])
        if len(self.decay) != self.heads:
            raise ConfigError(f"{len(self.decay)} decays for {self.heads} heads")
        _check_state_size(self.dim, self.vdim)
        self.desc: Optional[RecurrenceSpec] = None

    def state_need(self) -> StateNeed:
        return StateNeed((self.heads * self.vdim * self.dim,), torch.float32)

    def in_roles(self) -> List[Tuple[str, int]]:
        return [("q", self.heads * self.dim), ("k", self.heads * self.dim), ("v", self.heads * self.vdim), ("g", self.heads * self.vdim)]

    def core_width(self) -> int:
        return self.heads * self.vdim

    def extra_weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["norm"], (self.heads * self.vdim,), "vector", ("one_plus_normal", 0.01))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["recurrence"] + F.product_modules(dtype)

    def bind_core(self, tensors, rt, out_scale: float) -> None:
        at = self.in_columns()
        self._held = (torch.tensor(self.decay, dtype=torch.float32, device=rt.device),
                      rt.vector(tensors[self.spec.weights["norm"]]).float().contiguous())
        self.desc = RecurrenceSpec(
            decay=self._held[0].data_ptr(), out_weight=self._held[1].data_ptr(), heads=self.heads, qk_heads=self.heads, dim=self.dim,
            vdim=self.vdim, prep=RecurrenceSpec.PREP[None], rot_dims=0, rule=RecurrenceSpec.RULE["decay"], gate_kind=GATES["sigmoid"],
            col_q=at["q"], col_k=at["k"], col_v=at["v"], col_gate=at["g"], in_act=RecurrenceSpec.IN_ACT["silu"], norm_all=1,
            q_mult=1.0, k_mult=1.0, unit_eps=0.0, eps=self.eps, out_scale=float(out_scale))

    def emit_core(self, b, proj, act, run: RunContext) -> None:
        emit_recurrence(b, self, proj, proj, act, run)


register_part("mixer", "lightning", LightningMixer)
