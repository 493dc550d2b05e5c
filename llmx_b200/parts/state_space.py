"""A selective state space (Mamba-2, state-space duality): a matrix state per head, decayed by a step size the token
chooses, written with the token's input and read with the token's read-out vector.

For the rows of a step, with H heads of V values, a state of N values per head and G groups that share B and C (head h
uses group h // (H / G)); inner = H * V:
    [z | x B C | dt] = h Win^T                          z, x: inner; B, C: G * N each; dt: H
    x B C   = silu(conv(x B C) + bias)                  a causal filter of `taps` taps per channel (last tap on the current
                                                        token, zeros before the start), over x, B and C together
    dt      = softplus(dt + dt_bias)                    no clamp
    S      <- exp(-exp(A_log_h) dt) S + dt B x^T        S [N, V] per head, 32-bit
    y       = S^T C + D_h x
    y       = RMSNorm in `norm_groups` equal parts of (y * silu(z)) * weight     the gate comes before the norm
    residual += y Wo^T
A request's state slot holds S for every head and the last taps-1 inputs of the filter, as 32-bit floats.  The input
projection is one product; filter, activation and step sizes are one kernel and the recurrence another
(csrc/recurrence.cu: the scaled form, B as keys, C as queries, dt as the input's factor, D as the skip), the gated norm
a third (csrc/rowwise.cu).  Tensor roles: in, conv, conv.b, dt_bias, A_log, D, norm, o.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops, runtime
from ..cache.manager import StateSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear, stored_product


class SelectiveStateSpace(Part):
    def __init__(self, hidden: int, heads: int, value_dim: int, state_dim: int, groups: int, taps: int, norm_groups: int,
                 norm_eps: float):
        if heads % groups:
            raise ValueError("selective state space: head count must be divisible by the group count")
        if (heads * value_dim) % norm_groups:
            raise ValueError("selective state space: the norm's parts must divide heads * value_dim")
        if taps < 1:
            raise ValueError("selective state space: the filter has at least one tap")
        self.hidden, self.heads, self.value_dim, self.state_dim = int(hidden), int(heads), int(value_dim), int(state_dim)
        self.groups, self.taps, self.norm_groups, self.norm_eps = int(groups), int(taps), int(norm_groups), float(norm_eps)
        self.inner = self.heads * self.value_dim
        self.bc_width = self.groups * self.state_dim
        self.channels = self.inner + 2 * self.bc_width
        self.in_width = 2 * self.inner + 2 * self.bc_width + self.heads
        self.state_floats = self.heads * self.value_dim * self.state_dim
        self.slot_floats = self.state_floats + (self.taps - 1) * self.channels

    def stored_products(self):
        """The products whose result is stored (not added to the residual): a block may clear their outputs in passing."""
        return (self.inputs,)

    def cache_spec(self):
        return StateSpec((self.slot_floats,), "float32")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        E = self.hidden
        return {"in": TensorSpec((self.in_width, E)), "conv": TensorSpec((self.channels, self.taps), std=0.3),
                "conv.b": TensorSpec((self.channels,), "vector", std=0.1),
                "dt_bias": TensorSpec((self.heads,), "vector", std=0.5), "A_log": TensorSpec((self.heads,), "vector", std=0.5),
                "D": TensorSpec((self.heads,), "vector", init="one_plus_normal", std=0.1),
                "norm": TensorSpec((self.inner,), "vector", init="one_plus_normal", std=0.01),
                "o": TensorSpec((E, self.inner))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        t = tensors
        self.inputs = Linear(t["in"], precision)
        self.o = Linear(t["o"], precision)
        f32 = lambda x: x.to(torch.float32).contiguous()      # noqa: E731
        self.taps_w, self.taps_b = f32(t["conv"]), f32(t["conv.b"])
        self.a_log, self.dt_bias, self.skip, self.norm_weight = f32(t["A_log"]), f32(t["dt_bias"]), f32(t["D"]), f32(t["norm"])

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("selective state space: rows of the path's type and the mixer's width, a float32 residual")
        H, inner, bc = self.heads, self.inner, self.bc_width
        proj = stored_product(self, self.inputs, h)                            # [rows, z | x B C | dt]
        state = step.state(cache_entry)
        ready = torch.empty((rows, self.channels), dtype=torch.float32, device=h.device)
        gates = torch.empty((rows, 2 * H), dtype=torch.float32, device=h.device)
        ops.conv_prepare(proj, self.channels, 0, 0, self.taps_w, ready, self.a_log, self.dt_bias, 0, inner + self.channels, gates, H,
                         self.state_dim, 1.0, state, self.state_floats, step, first=inner, bias=self.taps_b, gate_kind="step")
        y = torch.empty((rows, inner), dtype=torch.float32, device=h.device)
        ops.linear_recurrence(ready[:, inner + bc:], ready[:, inner:inner + bc], ready[:, :inner], state, step, y, H, self.groups,
                              self.state_dim, self.value_dim, gate=gates[:, :H], beta=gates[:, H:], form="scaled", skip=self.skip)
        out = torch.empty((rows, inner), dtype=self.precision.act, device=h.device)
        ops.gated_rmsnorm(y, proj[:, :inner], self.norm_weight, self.norm_eps, inner // self.norm_groups, "silu", out, gate_first=True)
        self.o(out, out=residual, accumulate=True)
