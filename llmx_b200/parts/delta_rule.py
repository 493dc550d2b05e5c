"""The gated delta rule: a matrix state per head that is decayed, corrected towards the new value, and read.

For the rows of a step, with `kv_heads` query/key heads of width D shared by `heads` value heads of width V
(value head h uses q/k head h // (heads / kv_heads)):
    q, k, v = silu(conv(h Wq^T)), silu(conv(h Wk^T)), silu(conv(h Wv^T))
              conv: a causal filter of `taps` taps per channel (last tap on the current token, zeros before the start)
    q, k    = q / sqrt(sum q^2 + 1e-6) * D^-1/2,  k / sqrt(sum k^2 + 1e-6)      per head
    beta    = sigmoid(h Wb^T);   g = exp(-exp(A_log) * softplus(h Wa^T + dt_bias))   per value head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                (32-bit; the read sees the write)
    y       = RMSNorm per head over V (one weight of V shared by the heads) * silu(h Wg^T)
    residual += y Wo^T
A request's state slot holds S for every head and the last taps-1 inputs of the filter, as 32-bit floats.  The six
input projections are one product over the stacked weight; filter, activation, unit scaling and gates are one kernel,
the recurrence another (csrc/recurrence.cu), the gated norm a third (csrc/rowwise.cu).

Options for designs that vary the rule:
    decay_rank r > 0   one decay per head and key channel, through a low-rank pair: g [heads, D] =
                       exp(-exp(A_log_h) * softplus(Wa2 (Wa1 h) + dt_bias)), dt_bias [heads * D]; S <- diag(g) S acts on
                       the rows of S that belong to key channels (tensor roles a1 [r, E], a2 [heads * D, r] instead of a)
    gate_rank r > 0    the output gate through a low-rank pair, act(Wg2 (Wg1 h)) (roles g1 [r, E], g2 [heads * V, r])
    gate               "silu" or "sigmoid"
A rank of -1 stands for "whatever the stored tensors have": the specs then leave that size open and `load` reads it.
The second product of a low-rank pair is made in 32-bit on both paths (its input is a few dozen values wide): what it
gives enters the recurrence.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops, runtime
from ..cache.manager import StateSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear, stored_product


class GatedDeltaRule(Part):
    def __init__(self, hidden: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int, norm_eps: float,
                 decay_rank: int = 0, gate_rank: int = 0, gate: str = "silu"):
        if gate not in ("silu", "sigmoid"):
            raise ValueError("gated delta rule: the output gate is silu or sigmoid")
        self.decay_rank, self.gate_rank, self.gate = int(decay_rank), int(gate_rank), gate
        if heads % kv_heads:
            raise ValueError("gated delta rule: head count must be divisible by the q/k head count")
        if taps < 1:
            raise ValueError("gated delta rule: the filter has at least one tap")
        self.hidden, self.heads, self.kv_heads = int(hidden), int(heads), int(kv_heads)
        self.key_dim, self.value_dim, self.taps, self.norm_eps = int(key_dim), int(value_dim), int(taps), float(norm_eps)
        self.qk_width, self.v_width = self.kv_heads * self.key_dim, self.heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width
        self.state_floats = self.heads * self.value_dim * self.key_dim
        self.slot_floats = self.state_floats + (self.taps - 1) * self.channels

    def stored_products(self):
        """The products whose result is stored (not added to the residual): a block may clear their outputs in passing."""
        return (self.inputs,)

    def cache_spec(self):
        return StateSpec((self.slot_floats,), "float32")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        E = self.hidden
        specs = {"q": TensorSpec((self.qk_width, E)), "q.conv": TensorSpec((self.qk_width, self.taps), std=0.3),
                 "k": TensorSpec((self.qk_width, E)), "k.conv": TensorSpec((self.qk_width, self.taps), std=0.3),
                 "v": TensorSpec((self.v_width, E)), "v.conv": TensorSpec((self.v_width, self.taps), std=0.3),
                 "b": TensorSpec((self.heads, E)), "A_log": TensorSpec((self.heads,), "vector", std=0.5),
                 "norm": TensorSpec((self.value_dim,), "vector", init="one_plus_normal", std=0.01),
                 "o": TensorSpec((E, self.v_width))}
        if self.decay_rank:
            specs.update({"a1": TensorSpec((self.decay_rank, E)), "a2": TensorSpec((self.heads * self.key_dim, self.decay_rank), std=0.1),
                          "dt_bias": TensorSpec((self.heads * self.key_dim,), "vector", std=0.5)})
        else:
            specs.update({"a": TensorSpec((self.heads, E)), "dt_bias": TensorSpec((self.heads,), "vector", std=0.5)})
        if self.gate_rank:
            specs.update({"g1": TensorSpec((self.gate_rank, E)), "g2": TensorSpec((self.v_width, self.gate_rank), std=0.1)})
        else:
            specs["g"] = TensorSpec((self.v_width, E))
        return specs

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        t = tensors
        if self.decay_rank:
            self.decay_rank = int(t["a1"].shape[0])
            if t["a2"].shape[1] != self.decay_rank:
                raise ValueError("gated delta rule: the decay's two low-rank matrices do not fit each other")
        if self.gate_rank:
            self.gate_rank = int(t["g1"].shape[0])
            if t["g2"].shape[1] != self.gate_rank:
                raise ValueError("gated delta rule: the gate's two low-rank matrices do not fit each other")
        # One product for everything that reads h: q | k | v | gate (or its low-rank input) | b | a (or its low-rank input).
        self.gate_in = self.gate_rank or self.v_width
        self.decay_in = self.decay_rank or self.heads
        self.inputs = Linear(torch.cat([t["q"], t["k"], t["v"], t["g1" if self.gate_rank else "g"], t["b"],
                                        t["a1" if self.decay_rank else "a"]], dim=0), precision)
        full = Precision("float32", torch.float32, precision.invariant)
        self.a2 = Linear(t["a2"].to(torch.float32), full) if self.decay_rank else None
        self.g2 = Linear(t["g2"].to(torch.float32), full) if self.gate_rank else None
        self.o = Linear(t["o"], precision)
        self.taps_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).to(torch.float32).contiguous()
        self.a_log = t["A_log"].to(torch.float32).contiguous()
        self.dt_bias = t["dt_bias"].to(torch.float32).contiguous()
        self.norm_weight = t["norm"].to(torch.float32).contiguous()

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("delta rule: rows of the path's type and the mixer's width, a float32 residual")
        qk, vw, H = self.qk_width, self.v_width, self.heads
        g_off = self.channels
        b_off, a_off = g_off + self.gate_in, g_off + self.gate_in + H
        proj = stored_product(self, self.inputs, h)                          # [rows, q | k | v | g (g1) | b | a (a1)]
        state = step.state(cache_entry)
        ready = torch.empty((rows, self.channels), dtype=torch.float32, device=h.device)
        o = torch.empty((rows, vw), dtype=torch.float32, device=h.device)
        if self.decay_rank:
            decay_in = self.a2(proj[:, a_off:a_off + self.decay_rank].contiguous())          # [rows, heads * D], 32-bit
            gates = torch.empty((rows, H + H * self.key_dim), dtype=torch.float32, device=h.device)
            ops.conv_prepare(proj, self.channels, qk, qk, self.taps_w, ready, self.a_log, self.dt_bias, b_off, a_off, gates, H,
                             self.key_dim, self.key_dim ** -0.5, state, self.state_floats, step, gate_kind="delta_channel",
                             decay_in=decay_in)
            ops.linear_recurrence(ready[:, :qk], ready[:, qk:2 * qk], ready[:, 2 * qk:], state, step, o, H, self.kv_heads,
                                  self.key_dim, self.value_dim, gate=gates[:, H:], beta=gates[:, :H], form="delta_channel")
        else:
            gates = torch.empty((rows, 2 * H), dtype=torch.float32, device=h.device)
            ops.conv_prepare(proj, self.channels, qk, qk, self.taps_w, ready, self.a_log, self.dt_bias, b_off, a_off, gates, H,
                             self.key_dim, self.key_dim ** -0.5, state, self.state_floats, step)
            ops.linear_recurrence(ready[:, :qk], ready[:, qk:2 * qk], ready[:, 2 * qk:], state, step, o, H, self.kv_heads,
                                  self.key_dim, self.value_dim, gate=gates[:, :H], beta=gates[:, H:])
        gate = self.g2(proj[:, g_off:g_off + self.gate_rank].contiguous()) if self.gate_rank else proj[:, g_off:g_off + vw]
        y = torch.empty((rows, vw), dtype=self.precision.act, device=h.device)
        ops.gated_rmsnorm(o, gate, self.norm_weight, self.norm_eps, self.value_dim, self.gate, y)
        self.o(y, out=residual, accumulate=True)
