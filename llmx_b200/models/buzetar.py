"""Buzetar put together from the parts, and its registration.

A layer is a parallel block: one centred norm (weight, no bias), and a mixer and a clamped gated feed-forward (or
none) that both read the norm's output and add into the float32 residual.  The mixer is one of three, as the
configuration's layer list says, in any order: decayed linear attention, latent attention under a sliding window,
the gated delta rule.  The embedding and the logits carry factors; the final norm is the centred one again.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.<role>`, `l<i>.mlp.gate|up|down`, `final.norm`, `head`.

The design has no context limit of its own; positions are int32 and their angles 32-bit floats, exact up to 2^24.
"""
from __future__ import annotations

from ..config.buzetar import BuzetarConfig, DeltaMixer, LatentMixer, LightningMixer
from ..parts import (ClampedGLU, DecayedLinearAttention, GatedDeltaRule, LatentAttention, LayerNorm, LogitsHead,
                     ParallelBlock, TokenEmbedding)
from ..registry import register_architecture
from .model import Model

MAX_POSITIONS = 1 << 24


def _mixer(cfg: BuzetarConfig, m):
    E, eps = cfg.width, cfg.norm_eps
    if isinstance(m, LightningMixer):
        return DecayedLinearAttention(E, m.heads, m.dim, m.vdim, m.decay, eps)
    if isinstance(m, LatentMixer):
        return LatentAttention(E, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, m.rot_base, m.rot_dims,
                               eps, window=m.window)
    if isinstance(m, DeltaMixer):
        return GatedDeltaRule(E, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps)
    raise TypeError(type(m).__name__)


def build_buzetar(cfg: BuzetarConfig) -> Model:
    E = cfg.width
    blocks = []
    for layer in cfg.layers:
        ffn = None if layer.mlp is None else ClampedGLU(E, layer.mlp.ff, layer.mlp.limit)
        blocks.append(ParallelBlock(LayerNorm(E, cfg.norm_eps, role=""), _mixer(cfg, layer.mixer), ffn,
                                    names=("norm1", "mix", "mlp")))
    embedding = TokenEmbedding(cfg.vocab, E, scale=cfg.embedding_scale, role="")
    head = LogitsHead(LayerNorm(E, cfg.norm_eps, role=""), cfg.vocab, E, scale=cfg.logit_scale, role="")
    return Model(embedding=embedding, blocks=blocks, head=head, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
                 block_prefix=lambda i: f"l{i}.", embedding_prefix="embed.", head_norm_prefix="final.norm.",
                 head_prefix="head.")


register_architecture(("Buzetar", "buzetar"), BuzetarConfig, build_buzetar)
