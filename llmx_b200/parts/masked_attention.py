"""Grouped-query softmax attention whose keys and values have widths of their own, under a window, inside chunks, or
over everything.

For the rows of a step, with H query heads, G key/value heads (query head h reads key/value head h // (H / G)), key
width D and value width V:
    q, k, v = h Wq^T, h Wk^T, h Wv^T            (one product over the stacked weight; no biases)
    q, k    = RMSNorm per head over D with one weight of D values shared by the heads (optional), then
              rotated by position on the first `rot_dims` values of every head: value i pairs with value
              i + rot_dims / 2, the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a),
              a = p * base^(-2i / rot_dims) / rot_factor   (32-bit; `rot_factor`: linear scaling of the frequencies)
    [k ; v] -> the row's cache slot             (one row of D + V values per token and key/value head)
    o       = softmax(q K^T * scale) V over the keys lo..p of the request, where lo is the larger of
              p - window + 1 (under a window) and floor(p / chunk) * chunk (inside chunks, counted from the
              request's first token whatever way its prompt was cut), or 0
    residual += o Wo^T
Sizes, the scale, whether q/k are normed, the rotation's constants, window and chunk are constructor arguments, and so
are the tensors' roles.  The cache keeps what later rows can still see: pages wholly below the window or the chunk
of the next position are given back.  Kernels: csrc/attention_split.cu.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from .. import ops, runtime
from ..cache.manager import KVSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear, stored_product


class MaskedAttention(Part):
    def __init__(self, hidden: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, scale: Optional[float] = None,
                 qk_norm_eps: Optional[float] = None, rot_dims: int = 0, rot_base: float = 10000.0, rot_factor: float = 1.0,
                 window: Optional[int] = None, chunk: Optional[int] = None,
                 names=("q", "k", "v", "o", "q.norm", "k.norm")):
        if heads % kv_heads:
            raise ValueError("attention: head count must be divisible by the key/value head count")
        if rot_dims % 2 or rot_dims > key_dim or rot_dims < 0:
            raise ValueError("attention: the rotated width must be even and at most the key width")
        self.hidden, self.heads, self.kv_heads = int(hidden), int(heads), int(kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.key_dim)
        self.qk_norm_eps = qk_norm_eps
        self.rot_dims, self.rot_base, self.rot_factor = int(rot_dims), float(rot_base), float(rot_factor)
        self.window, self.chunk, self.names = window, chunk, tuple(names)
        self.q_width, self.k_width, self.v_width = self.heads * self.key_dim, self.kv_heads * self.key_dim, self.kv_heads * self.value_dim
        self.o_width = self.heads * self.value_dim

    def stored_products(self):
        return (self.qkv,)

    def cache_spec(self):
        return KVSpec(self.kv_heads, self.key_dim + self.value_dim, self.window, planes=1, chunk=self.chunk)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, k, v, o, qn, kn = self.names
        specs = {q: TensorSpec((self.q_width, self.hidden)), k: TensorSpec((self.k_width, self.hidden)),
                 v: TensorSpec((self.v_width, self.hidden)), o: TensorSpec((self.hidden, self.o_width))}
        if self.qk_norm_eps is not None:
            specs[qn] = TensorSpec((self.key_dim,), "vector", init="one_plus_normal", std=0.01)
            specs[kn] = TensorSpec((self.key_dim,), "vector", init="one_plus_normal", std=0.01)
        return specs

    def frequencies(self) -> np.ndarray:
        """base^(-2i / rot_dims) / rot_factor, i < rot_dims / 2, rounded once to 32-bit."""
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        return (np.power(self.rot_base, -2.0 * i / max(self.rot_dims, 1)) / self.rot_factor).astype(np.float32)

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        q, k, v, o, qn, kn = self.names
        self.qkv = Linear(torch.cat([tensors[q], tensors[k], tensors[v]], dim=0), precision)
        self.o = Linear(tensors[o], precision)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[qn].to(torch.float32).contiguous()
            self.k_norm = tensors[kn].to(torch.float32).contiguous()
        self.freq = torch.from_numpy(self.frequencies()).to(self.o.weight.device) if self.rot_dims else None
        self.tiled = precision.act is torch.bfloat16 and not precision.invariant and \
            ops.attention_tiled_fits(self.heads, self.kv_heads, self.key_dim, self.value_dim)

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("attention: rows of the path's type and the mixer's width, a float32 residual")
        group, cache = step.kv(cache_entry)
        proj = stored_product(self, self.qkv, h)                             # [rows, q | k | v], 32-bit
        q = torch.empty((rows, self.q_width), dtype=self.precision.act, device=h.device)
        slots = group.slots if write_cache else torch.full_like(group.slots, -1)
        ops.qk_norm_rope_write(proj, self.heads, self.kv_heads, self.key_dim, self.value_dim, self.q_norm, self.k_norm,
                               float(self.qk_norm_eps or 0.0), self.freq, step.positions, slots, q, cache)
        o = torch.empty((rows, self.o_width), dtype=self.precision.act, device=h.device)
        # Which kernel is a matter of speed only.  Steps that bring some request more than a few rows run the tiled
        # form (bfloat16, sizes it takes); others run the plain form, a row's keys cut into ranges when the rows alone
        # would not fill the device.
        if self.tiled and step.max_row_count > 4 and cache.dtype is torch.bfloat16:
            ops.attention_tiled(q, cache, o, step, group.block_tables, self.heads, self.kv_heads, self.key_dim, self.value_dim,
                                self.window, self.chunk, self.scale)
        else:
            span = min(x for x in (step.max_context, self.window, self.chunk) if x)
            blocks = rows * self.heads
            splits = 1 if self.precision.invariant else max(1, min(32, span // 128, 2368 // max(blocks, 1)))
            ops.attention_split(q, cache, o, step.row_request, step.positions, group.block_tables, self.heads, self.kv_heads,
                                self.key_dim, self.value_dim, self.window, self.chunk, self.scale, splits=splits)
        self.o(o, out=residual, accumulate=True)
