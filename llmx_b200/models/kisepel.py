"""Kisepel put together from the parts, and its registration.

A layer is a parallel block: one RMS norm whose weight is stored around zero (y = x / rms(x) * (1 + w)), and a mixer
and a feed-forward (or none) that both read the norm's output and add into the float32 residual.  The mixer is one of
three, as the configuration's layer list says, in any order: decayed linear attention (`lightning`), a selective state
space (`mamba2`), or two mixers side by side (`parallel`: softmax attention inside chunks on the left, the gated delta
rule with a decay per key channel on the right; half the sum of their normed outputs).  The feed-forward is a mixture
of experts whose routing is a table from token id to experts, with a shared expert beside them.  A stretch of the
layers may run several times with the same weights (`loop`): every pass has cache entries of its own, and the
embedding output is added to the stream before every pass but the first.  The embedding and the logits carry factors;
the logits are made with the embedding table itself.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.<role>`, `l<i>.mlp.<role>`, `final.norm`.

The design has no context limit of its own; positions are int32 and their angles 32-bit floats, exact up to 2^24.
"""
from __future__ import annotations

from ..config.kisepel import KisepelConfig, LightningMixer, ParallelMixer, StateSpaceMixer
from ..parts import (DecayedLinearAttention, GatedDeltaRule, GatedMLP, LogitsHead, MaskedAttention, MixerPair,
                     ParallelBlock, RMSNorm, SelectiveStateSpace, TableRoutedExperts, TokenEmbedding)
from ..registry import register_architecture
from .model import LayerStep, Model, _as_tuple

MAX_POSITIONS = 1 << 24


def _mixer(cfg: KisepelConfig, m):
    E, eps = cfg.width, cfg.norm_eps
    if isinstance(m, LightningMixer):
        return DecayedLinearAttention(E, m.heads, m.dim, m.vdim, m.decay, eps)
    if isinstance(m, StateSpaceMixer):
        return SelectiveStateSpace(E, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, eps)
    if isinstance(m, ParallelMixer):
        a, d = m.left, m.right
        left = MaskedAttention(E, a.heads, a.kv_heads, a.dim, a.vdim, scale=a.scale, qk_norm_eps=eps, rot_dims=a.rot_dims,
                               rot_base=a.rot_base, rot_factor=a.rot_factor, chunk=a.chunk)
        # The ranks of the two low-rank pairs are the tensors' own (-1: whatever the files hold) unless the configuration
        # names them, as the one the random-weights mode writes does.
        right = GatedDeltaRule(E, d.heads, d.kv_heads, d.dim, d.vdim, d.conv, eps, decay_rank=d.decay_rank or -1,
                               gate_rank=d.gate_rank or -1, gate="sigmoid")
        return MixerPair(E, left, right, eps, factor=0.5)
    raise TypeError(type(m).__name__)


def build_kisepel(cfg: KisepelConfig) -> Model:
    E = cfg.width
    blocks = []
    for i, layer in enumerate(cfg.layers):
        mixer = _mixer(cfg, layer.mixer)
        ffn = None
        if layer.mlp is not None:
            m = layer.mlp
            shared = None if m.shared_ff is None else GatedMLP(E, m.shared_ff, names=("gate", "up", "down"))
            ffn = TableRoutedExperts(E, cfg.vocab, m.experts, m.top, m.ff, shared=shared)
        blocks.append(ParallelBlock(RMSNorm(E, cfg.norm_eps, role="", one_plus=True), mixer, ffn, names=("norm1", "mix", "mlp")))
    # The order: every run of a layer has cache entries of its own, numbered as the runs come.
    order, at = [], 0
    for i, add in cfg.layer_runs():
        n = len(_as_tuple(blocks[i].cache_spec()))
        entries = tuple(range(at, at + n))
        at += n
        order.append(LayerStep(i, entries[0] if n == 1 else (entries or None), True, add))
    embedding = TokenEmbedding(cfg.vocab, E, scale=cfg.embedding_scale, role="")
    head = LogitsHead(RMSNorm(E, cfg.norm_eps, role="", one_plus=True), cfg.vocab, E, tied_to=embedding, scale=cfg.logit_scale)
    return Model(embedding=embedding, blocks=blocks, head=head, order=order, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
                 block_prefix=lambda i: f"l{i}.", embedding_prefix="embed.", head_norm_prefix="final.norm.",
                 head_prefix="head.")


register_architecture(("Kisepel", "kisepel"), KisepelConfig, build_kisepel)
