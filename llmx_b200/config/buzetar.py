"""Typed configuration of the Buzetar architecture, read from config.json.

config.json names the architecture by an `architecture` string and lists the layers one by one: each entry gives
its `type` (which mixer), the mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null for none).  Every size
and every constant that can differ between two models of the design is read from there; nothing is assumed equal
between layers.  A value of the wrong kind, a missing size and an unknown mixer or feed-forward kind are refused by
name; keys this reader does not know are kept in `ignored` and have no effect.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, _is_int

MIXER_TYPES = ("lightning", "latent_attention", "delta")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if not _is_int(v) or v < minimum:
        raise ConfigError(f"buzetar: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return int(v)


def _real(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"buzetar: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"buzetar: {where}.{key} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
             "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class BuzetarLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _read_mixer(kind: str, m: Dict[str, Any], where: str):
    if kind == "lightning":
        heads = _int(m, "heads", where)
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or any(
                isinstance(x, bool) or not isinstance(x, (int, float)) or not math.isfinite(float(x)) for x in decay):
            raise ConfigError(f"buzetar: {where}.decay must be a list of {heads} numbers (one per head), got {decay!r}")
        return LightningMixer(heads, _int(m, "dim", where), _int(m, "vdim", where), tuple(float(x) for x in decay))
    if kind == "latent_attention":
        rot = m.get("rot") if m.get("rot_dim") == 0 and not isinstance(m.get("rot"), dict) else _obj(m, "rot", where)
        if not isinstance(rot, dict):
            rot = {"base": 10000.0, "dims": 0}          # nothing is rotated: the base is never used
        mask = m.get("mask")
        window = None
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"buzetar: {where}.mask must be an object or null, got {mask!r}")
            window = _int(mask, "size", where + ".mask")
        rot_dim = _int(m, "rot_dim", where, minimum=0)
        dims = _int(rot, "dims", where + ".rot", minimum=0)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"buzetar: {where}.rot.dims must be even and at most rot_dim ({rot_dim}), got {dims}")
        base = _real(rot, "base", where + ".rot")
        if not base > 0:
            raise ConfigError(f"buzetar: {where}.rot.base must be positive, got {base!r}")
        return LatentMixer(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where),
                           _int(m, "q_rank", where), _int(m, "kv_rank", where), _real(m, "scale", where), base, dims, window)
    if kind == "delta":
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"buzetar: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        return DeltaMixer(heads, kv_heads, _int(m, "dim", where), _int(m, "vdim", where), _int(m, "conv", where))
    raise ConfigError(f"buzetar: {where}: mixer type {kind!r} is not one of {list(MIXER_TYPES)}")


@dataclass(frozen=True)
class BuzetarConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[BuzetarLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    ignored: Tuple[str, ...] = field(default=(), compare=False)

    model_type = "buzetar"
    class_name = "Buzetar"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BuzetarConfig":
        if raw.get("architecture") != "Buzetar":
            raise ConfigError(f"buzetar: config.json names architecture {raw.get('architecture')!r}")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("buzetar: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"buzetar: {where} must be an object")
            kind = entry.get("type")
            mixer = _read_mixer(kind, _obj(entry, "mixer", where), where + ".mixer")
            mlp_raw = entry.get("mlp")
            mlp = None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, dict):
                    raise ConfigError(f"buzetar: {where}.mlp must be an object or null")
                if mlp_raw.get("kind") != "dense":
                    raise ConfigError(f"buzetar: {where}.mlp.kind {mlp_raw.get('kind')!r} is not supported (\"dense\")")
                mlp = DenseMlp(_int(mlp_raw, "ff", where + ".mlp"), _real(mlp_raw, "limit", where + ".mlp"))
            layers.append(BuzetarLayer(kind, mixer, mlp))
        norm = _obj(raw, "norm", "config")
        eps = _real(norm, "eps", "norm")
        if not eps >= 0:
            raise ConfigError("buzetar: norm.eps must not be negative")
        emb = raw.get("embedding")
        emb_scale = _real(emb, "scale", "embedding") if isinstance(emb, dict) and "scale" in emb else 1.0
        logit_scale = _real(raw, "logit_scale", "config") if "logit_scale" in raw else 1.0
        known = {"architecture", "layers", "norm", "embedding", "logit_scale", "vocab", "width", "torch_dtype"}
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), layers=tuple(layers), norm_eps=eps,
                   embedding_scale=emb_scale, logit_scale=logit_scale, ignored=tuple(sorted(k for k in raw if k not in known)))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": "Buzetar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "layers": [layer.to_dict() for layer in self.layers]}
