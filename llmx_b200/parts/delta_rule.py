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
    def __init__(self, hidden: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int, norm_eps: float):
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
        return {"q": TensorSpec((self.qk_width, E)), "q.conv": TensorSpec((self.qk_width, self.taps), std=0.3),
                "k": TensorSpec((self.qk_width, E)), "k.conv": TensorSpec((self.qk_width, self.taps), std=0.3),
                "v": TensorSpec((self.v_width, E)), "v.conv": TensorSpec((self.v_width, self.taps), std=0.3),
                "b": TensorSpec((self.heads, E)), "a": TensorSpec((self.heads, E)),
                "A_log": TensorSpec((self.heads,), "vector", std=0.5), "dt_bias": TensorSpec((self.heads,), "vector", std=0.5),
                "norm": TensorSpec((self.value_dim,), "vector", init="one_plus_normal", std=0.01),
                "g": TensorSpec((self.v_width, E)), "o": TensorSpec((E, self.v_width))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        t = tensors
        self.inputs = Linear(torch.cat([t["q"], t["k"], t["v"], t["g"], t["b"], t["a"]], dim=0), precision)
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
        b_off, a_off = g_off + vw, g_off + vw + H
        proj = stored_product(self, self.inputs, h)                                             # [rows, q | k | v | g | b | a]
        state = step.state(cache_entry)
        ready = torch.empty((rows, self.channels), dtype=torch.float32, device=h.device)
        gates = torch.empty((rows, 2 * H), dtype=torch.float32, device=h.device)
        ops.conv_prepare(proj, self.channels, qk, qk, self.taps_w, ready, self.a_log, self.dt_bias, b_off, a_off, gates, H,
                         self.key_dim, self.key_dim ** -0.5, state, self.state_floats, step)
        o = torch.empty((rows, vw), dtype=torch.float32, device=h.device)
        ops.linear_recurrence(ready[:, :qk], ready[:, qk:2 * qk], ready[:, 2 * qk:], state, step, o, H, self.kv_heads,
                              self.key_dim, self.value_dim, gate=gates[:, :H], beta=gates[:, H:])
        y = torch.empty((rows, vw), dtype=self.precision.act, device=h.device)
        ops.gated_rmsnorm(o, proj[:, g_off:g_off + vw], self.norm_weight, self.norm_eps, self.value_dim, "silu", y)
        self.o(y, out=residual, accumulate=True)
