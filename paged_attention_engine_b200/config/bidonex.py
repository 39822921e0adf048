"""Typed configuration of the Bidonex decoder, read from its own config.json keys.

    {"architecture": "Bidonex", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e},
     "layers": [{"type": "attention" | "general_delta", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A layer's mixer is one of two kinds:

  attention      heads, kv_heads, dim (query/key head size), vdim (value head size), scale,
                 softcap (absent or 0: none), conv (taps of the short convolution on q, k and
                 v; absent or 0: none), mask {size, keep_first} (absent: every earlier key).
  general_delta  heads, dim; the rank of the decay's two small matrices is a tensor's shape
                 (`rank` may name it: the random-weights mode needs it and writes it).

Every size and constant that can differ between two models of the design is read here; nothing
has a default except where the key's absence means that the mechanism is absent.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError

LAYER_TYPES = ("attention", "general_delta")


def _get(raw: Mapping[str, Any], key: str, kind, where: str):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: key '{where}{key}' is missing")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: key '{where}{key}' = {raw[key]!r} is not {kind.__name__}") from exc


def _positive(value: int, where: str) -> int:
    if value < 1:
        raise ConfigError(f"config.json: key '{where}' must be at least 1, got {value}")
    return value


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float        # 0: no cap
    conv: int             # taps; 0: no convolution
    window: int           # 0: every earlier key
    keep_first: int

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.softcap:
            out["softcap"] = self.softcap
        if self.conv:
            out["conv"] = self.conv
        if self.window:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return out


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    dim: int
    rank: int             # 0: whatever the checkpoint's tensors have

    def to_dict(self) -> dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim}
        if self.rank:
            out["rank"] = self.rank
        return out


@dataclass(frozen=True)
class BidonexLayer:
    type: str
    mixer: Any            # AttentionMixer or DeltaMixer
    ff: int               # 0: the layer has no feed-forward

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class BidonexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple[BidonexLayer, ...]
    architecture: str = "Bidonex"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BidonexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' is missing or empty")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of {', '.join(LAYER_TYPES)}")
            mixer_raw = entry.get("mixer")
            if not isinstance(mixer_raw, Mapping):
                raise ConfigError(f"config.json: key '{where}mixer' is missing")
            m = where + "mixer."
            if kind == "attention":
                heads = _positive(_get(mixer_raw, "heads", int, m), m + "heads")
                kv_heads = _positive(_get(mixer_raw, "kv_heads", int, m), m + "kv_heads")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {m}heads {heads} is not a multiple of kv_heads {kv_heads}")
                window = keep_first = 0
                mask = mixer_raw.get("mask")
                if mask is not None:
                    window = _positive(_get(mask, "size", int, m + "mask."), m + "mask.size")
                    keep_first = int(mask.get("keep_first") or 0)
                    if keep_first < 0:
                        raise ConfigError(f"config.json: {m}mask.keep_first must not be negative, got {keep_first}")
                softcap = float(mixer_raw.get("softcap") or 0.0)
                conv = int(mixer_raw.get("conv") or 0)
                if softcap < 0 or conv < 0:
                    raise ConfigError(f"config.json: {m}softcap and {m}conv must not be negative")
                mixer: Any = AttentionMixer(
                    heads, kv_heads, _positive(_get(mixer_raw, "dim", int, m), m + "dim"),
                    _positive(_get(mixer_raw, "vdim", int, m), m + "vdim"), _get(mixer_raw, "scale", float, m),
                    softcap, conv, window, keep_first)
            else:
                mixer = DeltaMixer(_positive(_get(mixer_raw, "heads", int, m), m + "heads"),
                                   _positive(_get(mixer_raw, "dim", int, m), m + "dim"), int(mixer_raw.get("rank") or 0))
            ff = 0
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp_kind = _get(mlp, "kind", str, where + "mlp.")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind '{mlp_kind}' is not supported (dense)")
                ff = _positive(_get(mlp, "ff", int, where + "mlp."), where + "mlp.ff")
            layers.append(BidonexLayer(kind, mixer, ff))
        eps = _get(raw.get("norm"), "eps", float, "norm.")
        if not eps > 0.0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        return cls(
            vocab=_positive(_get(raw, "vocab", int, ""), "vocab"),
            width=_positive(_get(raw, "width", int, ""), "width"),
            max_positions=_positive(_get(raw, "max_positions", int, ""), "max_positions"),
            norm_eps=eps,
            layers=tuple(layers),
            architecture=str(raw.get("architecture", "Bidonex")),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "BidonexConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "layers": [layer.to_dict() for layer in self.layers]}
