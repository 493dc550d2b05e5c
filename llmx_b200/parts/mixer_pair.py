"""Two mixers side by side: both read the same rows, each result is RMS-normed over the model's width with a plain
weight of its own, and `factor` times their sum joins the residual:
    residual += factor * (RMSNorm(left(h)) * w_left + RMSNorm(right(h)) * w_right)
The two mixers are any parts with a mixer's interface; each keeps its own cache entry, so the pair's `cache_spec()` is
the tuple of theirs and the layer order names two entries for it.  `names`: the prefixes of the two mixers' tensors;
the norm weights' roles are `<prefix>.out`.  The norms and the sum are one kernel (csrc/rowwise.cu, `llmx_pair_norm_add`).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch


class MixerPair(Part):
    def __init__(self, hidden: int, left: Part, right: Part, norm_eps: float, factor: float = 0.5, names=("left", "right")):
        self.hidden, self.left, self.right = int(hidden), left, right
        self.norm_eps, self.factor, self.names = float(norm_eps), float(factor), tuple(names)

    def children(self) -> Dict[str, Part]:
        return {self.names[0]: self.left, self.names[1]: self.right}

    def cache_spec(self):
        specs = tuple(s for s in (self.left.cache_spec(), self.right.cache_spec()) if s is not None)
        return specs or None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {f"{n}.out": TensorSpec((self.hidden,), "vector", init="one_plus_normal", std=0.01) for n in self.names}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.w_left = tensors[f"{self.names[0]}.out"].to(torch.float32).contiguous()
        self.w_right = tensors[f"{self.names[1]}.out"].to(torch.float32).contiguous()

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry, residual: torch.Tensor, write_cache: bool = True) -> None:
        entries = list(cache_entry) if isinstance(cache_entry, (tuple, list)) else [cache_entry]
        outs = []
        for side in (self.left, self.right):
            entry = entries.pop(0) if side.cache_spec() is not None else None
            out = torch.zeros_like(residual)          # a side adds its output projection into what it is handed
            side.forward(h, step, entry, out, write_cache)
            outs.append(out)
        ops.pair_norm_add_(residual, outs[0], outs[1], self.w_left, self.w_right, self.norm_eps, self.factor)
