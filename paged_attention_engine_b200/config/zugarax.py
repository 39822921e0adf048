"""Typed configuration of the Zugarax decoder, read from its own config.json keys.

    {"architecture": "Zugarax", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "logit_softcap": c, "layers": [{"type": ..., "mixer": {...}, "mlp": {"kind": "dense", "ff": F, "limit": l} | null}, ...]}

A layer's mixer is one of three kinds:

  attention         heads, kv_heads, dim (query/key head size), vdim, scale, mask {size} (absent:
                    every earlier key), rot {base, dims, scaling {factor, low, high, original}}
                    (`scaling` absent: plain frequencies; `rot` absent: no rotation).
  latent_attention  heads, dim (unrotated query/key channels per head), rot_dim (rotated ones),
                    vdim, kv_rank (the latent's size), scale, rot {base, dims, scaling {factor,
                    original, fast, slow}}, kv_from (absent: the layer projects its own latent; j:
                    it reads layer j's).
  mlstm             heads, dim, vdim, gate_cap.

Every size and constant that can differ between two models of the design is read here; nothing
has a default except where a key's absence means that the mechanism is absent.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError

LAYER_TYPES = ("attention", "latent_attention", "mlstm")


def _get(raw, key: str, kind, where: str):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: key '{where}{key}' is missing")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: key '{where}{key}' = {raw[key]!r} is not {kind.__name__}") from exc


def _positive(value, where: str):
    if not value > 0:
        raise ConfigError(f"config.json: key '{where}' must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Rotation:
    """Rotated channels of a head. `scaling` is None or the dictionary of the mixer's kind of
    frequency scaling, floats by name."""

    base: float
    dims: int
    scaling: tuple[tuple[str, float], ...] | None

    @classmethod
    def read(cls, raw, where: str, scaling_keys: tuple[str, ...]) -> "Rotation":
        if not isinstance(raw, Mapping):
            raise ConfigError(f"config.json: key '{where[:-1]}' is missing")
        dims = _positive(_get(raw, "dims", int, where), where + "dims")
        if dims % 2:
            raise ConfigError(f"config.json: {where}dims {dims} is odd")
        scaling = None
        if raw.get("scaling") is not None:
            scaling = tuple((k, _positive(_get(raw["scaling"], k, float, where + "scaling."), where + "scaling." + k))
                            for k in scaling_keys)
        return cls(_positive(_get(raw, "base", float, where), where + "base"), dims, scaling)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(self.scaling)
        return out


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int             # 0: every earlier key
    rot: Rotation | None    # None: positions are not encoded

    def to_dict(self) -> dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.window:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation
    kv_from: int | None     # the layer whose latent this one reads

    def to_dict(self) -> dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
               "scale": self.scale, "rot": self.rot.to_dict()}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class ZugaraxLayer:
    type: str
    mixer: Any
    ff: int                 # 0: the layer has no feed-forward
    limit: float

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": "dense", "ff": self.ff, "limit": self.limit} if self.ff else None}


@dataclass(frozen=True)
class ZugaraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float    # 0: the logits are not capped
    layers: tuple[ZugaraxLayer, ...]
    architecture: str = "Zugarax"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZugaraxConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' is missing or empty")
        layers: list[ZugaraxLayer] = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of {', '.join(LAYER_TYPES)}")
            mixer_raw = entry.get("mixer")
            if not isinstance(mixer_raw, Mapping):
                raise ConfigError(f"config.json: key '{where}mixer' is missing")
            m = where + "mixer."
            size = lambda key: _positive(_get(mixer_raw, key, int, m), m + key)
            if kind == "attention":
                heads, kv_heads = size("heads"), size("kv_heads")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {m}heads {heads} is not a multiple of kv_heads {kv_heads}")
                window = 0
                if mixer_raw.get("mask") is not None:
                    window = _positive(_get(mixer_raw["mask"], "size", int, m + "mask."), m + "mask.size")
                rot = None
                if mixer_raw.get("rot") is not None:
                    rot = Rotation.read(mixer_raw.get("rot"), m + "rot.", ("factor", "low", "high", "original"))
                dim = size("dim")
                if rot is not None and rot.dims > dim:
                    raise ConfigError(f"config.json: {m}rot.dims {rot.dims} exceeds dim {dim}")
                mixer: Any = WindowAttention(heads, kv_heads, dim, size("vdim"), _get(mixer_raw, "scale", float, m), window, rot)
            elif kind == "latent_attention":
                rot = Rotation.read(mixer_raw.get("rot"), m + "rot.", ("factor", "original", "fast", "slow"))
                rot_dim = size("rot_dim")
                if rot.dims != rot_dim:
                    raise ConfigError(f"config.json: {m}rot.dims {rot.dims} differs from rot_dim {rot_dim}")
                kv_from = mixer_raw.get("kv_from")
                if kv_from is not None:
                    kv_from = int(kv_from)
                    source = layers[kv_from].mixer if 0 <= kv_from < i else None
                    if not isinstance(source, LatentAttention) or source.kv_from is not None:
                        raise ConfigError(f"config.json: {m}kv_from {kv_from} does not name an earlier latent_attention layer with a latent of its own")
                mixer = LatentAttention(size("heads"), size("dim"), rot_dim, size("vdim"), size("kv_rank"),
                                        _get(mixer_raw, "scale", float, m), rot, kv_from)
                if kv_from is not None:
                    source = layers[kv_from].mixer
                    if (source.kv_rank, source.rot_dim, source.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                        raise ConfigError(f"config.json: {m}kv_rank, rot_dim and rot differ from those of layer {kv_from}, whose latent it reads")
            else:
                mixer = MatrixMemory(size("heads"), size("dim"), size("vdim"), _positive(_get(mixer_raw, "gate_cap", float, m), m + "gate_cap"))
            ff, limit = 0, 0.0
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp_kind = _get(mlp, "kind", str, where + "mlp.")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind '{mlp_kind}' is not supported (dense)")
                ff = _positive(_get(mlp, "ff", int, where + "mlp."), where + "mlp.ff")
                limit = _positive(_get(mlp, "limit", float, where + "mlp."), where + "mlp.limit")
            layers.append(ZugaraxLayer(kind, mixer, ff, limit))
        softcap = float(raw.get("logit_softcap") or 0.0)
        if softcap < 0:
            raise ConfigError(f"config.json: logit_softcap must not be negative, got {softcap}")
        return cls(
            vocab=_positive(_get(raw, "vocab", int, ""), "vocab"),
            width=_positive(_get(raw, "width", int, ""), "width"),
            embedding_scale=_get(raw.get("embedding"), "scale", float, "embedding."),
            norm_eps=_positive(_get(raw.get("norm"), "eps", float, "norm."), "norm.eps"),
            logit_softcap=softcap,
            layers=tuple(layers),
            architecture=str(raw.get("architecture", "Zugarax")),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "ZugaraxConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out
