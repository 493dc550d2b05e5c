"""Typed configuration of the Kisepel architecture, read from config.json.

config.json names the architecture by an `architecture` string and lists the layers one by one: each entry gives
its `type` (which mixer), the mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null for none).  A `loop`
entry runs a run of layers several times with the same weights.  Every size and every constant that can differ
between two models of the design is read from there; nothing is assumed equal between layers.  A value of the wrong
kind, a missing size and an unknown mixer or feed-forward kind are refused by name; keys this reader does not know
are kept in `ignored` and have no effect.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, _is_int

MIXER_TYPES = ("lightning", "mamba2", "parallel")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if not _is_int(v) or v < minimum:
        raise ConfigError(f"kisepel: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return int(v)


def _real(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"kisepel: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"kisepel: {where}.{key} must be an object, got {v!r}")
    return v


def _divides(what: str, a: int, name_a: str, b: int, name_b: str) -> None:
    if a % b:
        raise ConfigError(f"kisepel: {what}.{name_a} ({a}) must be a multiple of {name_b} ({b})")


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class StateSpaceMixer:
    """Mamba-2: `heads` heads of `vdim` values over a state of `state` values; B and C in `groups` groups."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class AttentionSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_factor: float = 1.0
    chunk: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims, "scaling": {"factor": self.rot_factor}}}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class DeltaSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None      # the ranks of the decay's and the gate's low-rank pairs: the tensors' shapes give
    gate_rank: Optional[int] = None       # them; named only in a configuration that weights are made from

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class ParallelMixer:
    left: AttentionSide
    right: DeltaSide

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class ExpertsMlp:
    """`experts` gated units of width `ff`, `top` of them a token, chosen by a table; a shared unit of width
    `shared_ff` beside them, or none."""
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff},
                "shared": None if self.shared_ff is None else {"ff": self.shared_ff}}


@dataclass(frozen=True)
class KisepelLayer:
    type: str
    mixer: Any
    mlp: Optional[ExpertsMlp]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class Loop:
    """Layers start .. stop-1 run `times` times in a row with the same weights."""
    start: int = 0
    stop: int = 0
    times: int = 1

    def to_dict(self) -> Dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _read_attention(m: Dict[str, Any], where: str) -> AttentionSide:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    _divides(where, heads, "heads", kv_heads, "kv_heads")
    dim = _int(m, "dim", where)
    rot = m.get("rot")
    base, dims, factor = 10000.0, 0, 1.0
    if rot is not None:
        rot = _obj(m, "rot", where)
        dims = _int(rot, "dims", where + ".rot", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"kisepel: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        base = _real(rot, "base", where + ".rot")
        if not base > 0:
            raise ConfigError(f"kisepel: {where}.rot.base must be positive, got {base!r}")
        scaling = rot.get("scaling")
        if scaling is not None:
            factor = _real(_obj(rot, "scaling", where + ".rot"), "factor", where + ".rot.scaling")
            if not factor > 0:
                raise ConfigError(f"kisepel: {where}.rot.scaling.factor must be positive, got {factor!r}")
    mask = m.get("mask")
    chunk = None
    if mask is not None:
        chunk = _int(_obj(m, "mask", where), "size", where + ".mask")
    return AttentionSide(heads, kv_heads, dim, _int(m, "vdim", where), _real(m, "scale", where), base, dims, factor, chunk)


def _read_mixer(kind: str, m: Dict[str, Any], where: str):
    if kind == "lightning":
        heads = _int(m, "heads", where)
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or any(
                isinstance(x, bool) or not isinstance(x, (int, float)) or not math.isfinite(float(x)) for x in decay):
            raise ConfigError(f"kisepel: {where}.decay must be a list of {heads} numbers (one per head), got {decay!r}")
        return LightningMixer(heads, _int(m, "dim", where), _int(m, "vdim", where), tuple(float(x) for x in decay))
    if kind == "mamba2":
        heads, groups = _int(m, "heads", where), _int(m, "groups", where)
        _divides(where, heads, "heads", groups, "groups")
        vdim, norm_groups = _int(m, "vdim", where), _int(m, "norm_groups", where)
        _divides(where, heads * vdim, "heads * vdim", norm_groups, "norm_groups")
        return StateSpaceMixer(heads, vdim, _int(m, "state", where), groups, _int(m, "conv", where), norm_groups)
    if kind == "parallel":
        r, rw = _obj(m, "right", where), where + ".right"
        heads, kv_heads = _int(r, "heads", rw), _int(r, "kv_heads", rw)
        _divides(rw, heads, "heads", kv_heads, "kv_heads")
        right = DeltaSide(heads, kv_heads, _int(r, "dim", rw), _int(r, "vdim", rw), _int(r, "conv", rw),
                          _int(r, "decay_rank", rw) if "decay_rank" in r else None,
                          _int(r, "gate_rank", rw) if "gate_rank" in r else None)
        return ParallelMixer(_read_attention(_obj(m, "left", where), where + ".left"), right)
    raise ConfigError(f"kisepel: {where}: mixer type {kind!r} is not one of {list(MIXER_TYPES)}")


def _read_mlp(raw: Any, where: str) -> Optional[ExpertsMlp]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"kisepel: {where} must be an object or null")
    if raw.get("kind") != "moe":
        raise ConfigError(f"kisepel: {where}.kind {raw.get('kind')!r} is not supported (\"moe\")")
    router = _obj(raw, "router", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"kisepel: {where}.router.top ({top}) exceeds the number of experts ({experts})")
    shared = raw.get("shared")
    shared_ff = None if shared is None else _int(_obj(raw, "shared", where), "ff", where + ".shared")
    return ExpertsMlp(experts, top, _int(_obj(raw, "expert", where), "ff", where + ".expert"), shared_ff)


@dataclass(frozen=True)
class KisepelConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[KisepelLayer, ...]
    norm_eps: float
    loop: Loop = Loop()
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    ignored: Tuple[str, ...] = field(default=(), compare=False)

    model_type = "kisepel"
    class_name = "Kisepel"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KisepelConfig":
        if raw.get("architecture") != "Kisepel":
            raise ConfigError(f"kisepel: config.json names architecture {raw.get('architecture')!r}")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("kisepel: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"kisepel: {where} must be an object")
            kind = entry.get("type")
            mixer = _read_mixer(kind, _obj(entry, "mixer", where), where + ".mixer")
            layers.append(KisepelLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + ".mlp")))
        loop = Loop()
        if raw.get("loop") is not None:
            lr = _obj(raw, "loop", "config")
            loop = Loop(_int(lr, "start", "loop", minimum=0), _int(lr, "stop", "loop", minimum=0), _int(lr, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"kisepel: loop must have 0 <= start <= stop <= {len(layers)} layers, got {lr!r}")
        norm = _obj(raw, "norm", "config")
        eps = _real(norm, "eps", "norm")
        if not eps >= 0:
            raise ConfigError("kisepel: norm.eps must not be negative")
        emb = raw.get("embedding")
        emb_scale = _real(emb, "scale", "embedding") if isinstance(emb, dict) and "scale" in emb else 1.0
        logit_scale = _real(raw, "logit_scale", "config") if "logit_scale" in raw else 1.0
        known = {"architecture", "layers", "loop", "norm", "embedding", "logit_scale", "vocab", "width", "torch_dtype"}
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), layers=tuple(layers), norm_eps=eps,
                   loop=loop, embedding_scale=emb_scale, logit_scale=logit_scale,
                   ignored=tuple(sorted(k for k in raw if k not in known)))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": "Kisepel", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "loop": self.loop.to_dict(),
                "layers": [layer.to_dict() for layer in self.layers]}

    def layer_runs(self):
        """The layers in the order they run, each with whether the embedding output is added to the stream before it:
        the looped run `times` times in a row (the embedding output joins before every pass but the first), the rest once."""
        n, lp = len(self.layers), self.loop
        runs = [(i, False) for i in range(lp.start)]
        for p in range(lp.times if lp.stop > lp.start else 0):
            runs += [(i, p > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        runs += [(i, False) for i in range(lp.stop, n)]
        return runs
