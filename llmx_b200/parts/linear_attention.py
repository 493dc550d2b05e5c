"""Decayed linear attention: a matrix state per head instead of a cache of keys.

For the rows of a step, per head h with key width D and value width V:
    q, k = silu(h Wq^T), silu(h Wk^T)      [heads, D]
    v    = silu(h Wv^T)                    [heads, V]
    S_t  = decay_h S_{t-1} + k_t v_t^T     (32-bit, one [D, V] matrix per request and head, in a state slot)
    o_t  = S_t^T q_t                       (no other scale)
    y    = RMSNorm over all heads' outputs together (weight of heads * V) * sigmoid(h Wg^T)
    residual += y Wo^T
The per-head decays are constants of the architecture's configuration.  The four input projections are one product
over the stacked weight; the activation, the recurrence (csrc/recurrence.cu) and the gated norm (csrc/rowwise.cu)
are kernels of their own; the recurrence has a form for steps of a row or a few and one for long portions.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops, runtime
from ..cache.manager import StateSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear, stored_product


class DecayedLinearAttention(Part):
    def __init__(self, hidden: int, heads: int, key_dim: int, value_dim: int, decay: Sequence[float], norm_eps: float,
                 names=("q", "k", "v", "g", "o", "norm")):
        if len(decay) != heads:
            raise ValueError("decayed linear attention: one decay per head")
        self.hidden, self.heads, self.key_dim, self.value_dim = int(hidden), int(heads), int(key_dim), int(value_dim)
        self.decay_values = [float(d) for d in decay]
        self.norm_eps, self.names = float(norm_eps), tuple(names)
        self.qk_width, self.v_width = self.heads * self.key_dim, self.heads * self.value_dim

    def stored_products(self):
        """The products whose result is stored (not added to the residual): a block may clear their outputs in passing."""
        return (self.inputs,)

    def cache_spec(self):
        return StateSpec((self.heads * self.value_dim * self.key_dim,), "float32")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, k, v, g, o, norm = self.names
        return {q: TensorSpec((self.qk_width, self.hidden)), k: TensorSpec((self.qk_width, self.hidden)),
                v: TensorSpec((self.v_width, self.hidden)), g: TensorSpec((self.v_width, self.hidden)),
                o: TensorSpec((self.hidden, self.v_width)),
                norm: TensorSpec((self.v_width,), "vector", init="one_plus_normal", std=0.01)}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        q, k, v, g, o, norm = self.names
        self.inputs = Linear(torch.cat([tensors[q], tensors[k], tensors[v], tensors[g]], dim=0), precision)
        self.o = Linear(tensors[o], precision)
        self.norm_weight = tensors[norm].to(torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.norm_weight.device)

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("linear attention: rows of the path's type and the mixer's width, a float32 residual")
        qk, vw = self.qk_width, self.v_width
        proj = stored_product(self, self.inputs, h)                                             # [rows, q | k | v | g]
        ops.silu_columns_(proj, 0, 2 * qk + vw)
        o = torch.empty((rows, vw), dtype=torch.float32, device=h.device)
        ops.linear_recurrence(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vw], step.state(cache_entry), step, o,
                              self.heads, self.heads, self.key_dim, self.value_dim, decay=self.decay)
        y = torch.empty((rows, vw), dtype=self.precision.act, device=h.device)
        ops.gated_rmsnorm(o, proj[:, 2 * qk + vw:], self.norm_weight, self.norm_eps, vw, "sigmoid", y)
        self.o(y, out=residual, accumulate=True)
