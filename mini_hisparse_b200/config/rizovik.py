"""Typed Rizovik configuration, read from the design's own config.json.

Keys: ``architecture`` ("Rizovik"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` and ``layers``, a list whose
entries give ``type`` ("attention", "attention_2" or "delta"), the mixer's sizes ``mixer``, the feed-forward ``mlp``
(null for none; else ``kind`` "moe" with ``expert.ff`` and ``router.experts`` / ``router.top``) and optionally
``weights_of``: the index of the layer whose tensors this one runs, over a cache or state of its own.

    attention     heads, kv_heads, dim, vdim, scale, mask.size, mask.pool, rot.dims, rot.base
    attention_2   heads, kv_heads, dim, vdim, scale, mask.size, mask.keep_first, rot.dims, rot.base, rot.scaling.factor
    delta         heads, kv_heads, dim, vdim, conv

No size has a default (``rot`` may be left out for a mixer that does not rotate, ``rot.scaling`` for unscaled
frequencies, ``mask.keep_first`` for none); a key this reader does not know is refused, so that a variant it cannot
compute never runs as something else.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .koronex import _need, _only
from .qwen2 import ConfigError


@dataclass(frozen=True)
class WindowMixer:
    """"attention" (pool set) and "attention_2" (keep_first set)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_dims: int
    rot_base: float
    rot_factor: float = 1.0
    pool: int | None = None
    keep_first: int | None = None


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    expert_ff: int


@dataclass(frozen=True)
class RizovikLayer:
    type: str
    mixer: WindowMixer | DeltaMixer
    mlp: RoutedFF | None
    weights_of: int | None = None


def _mlp(raw, where: str):
    if raw is None:
        return None
    kind = _need(raw, "kind", where)
    if kind != "moe":
        raise ConfigError(f"{where}kind {kind!r} is not a feed-forward of this design")
    _only(raw, ("kind", "expert", "router"), where[:-1])
    expert, router = _need(raw, "expert", where), _need(raw, "router", where)
    _only(expert, ("ff",), where + "expert")
    _only(router, ("experts", "top"), where + "router")
    out = RoutedFF(int(_need(router, "experts", where + "router.")), int(_need(router, "top", where + "router.")),
                   int(_need(expert, "ff", where + "expert.")))
    if out.experts < 1 or out.expert_ff < 1 or not 1 <= out.top <= out.experts:
        raise ConfigError(f"{where}: {out.top} of {out.experts} experts, each {out.expert_ff} wide, make no sense")
    return out


def _window_mixer(kind: str, m, where: str) -> WindowMixer:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where + "mixer")
    mask = _need(m, "mask", where + "mixer.")
    rot = m.get("rot")
    dims, base, factor = 0, 1.0, 1.0
    if rot is not None:
        _only(rot, ("dims", "base", "scaling"), where + "mixer.rot")
        dims = int(_need(rot, "dims", where + "mixer.rot."))
        if dims:
            base = float(_need(rot, "base", where + "mixer.rot."))
        scaling = rot.get("scaling")
        if scaling is not None:
            _only(scaling, ("factor",), where + "mixer.rot.scaling")
            factor = float(_need(scaling, "factor", where + "mixer.rot.scaling."))
    pool = keep = None
    if kind == "attention":
        _only(mask, ("size", "pool"), where + "mixer.mask")
        pool = int(_need(mask, "pool", where + "mixer.mask."))
        if pool < 1:
            raise ConfigError(f"{where}mixer.mask.pool must be positive")
        if factor != 1.0:
            raise ConfigError(f"{where}mixer.rot.scaling is not a part of this mixer")
    else:
        _only(mask, ("size", "keep_first"), where + "mixer.mask")
        keep = int(mask.get("keep_first") or 0)
        if keep < 0:
            raise ConfigError(f"{where}mixer.mask.keep_first cannot be negative")
    out = WindowMixer(int(_need(m, "heads", where)), int(_need(m, "kv_heads", where)), int(_need(m, "dim", where)),
                      int(_need(m, "vdim", where)), float(_need(m, "scale", where)),
                      int(_need(mask, "size", where + "mixer.mask.")), dims, base, factor, pool, keep)
    if min(out.heads, out.kv_heads, out.dim, out.vdim, out.window) < 1 or out.heads % out.kv_heads:
        raise ConfigError(f"{where}mixer: heads, kv_heads (a divisor of heads), dim, vdim and mask.size must be positive")
    if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.dim or not out.rot_factor > 0 or not out.rot_base > 0:
        raise ConfigError(f"{where}mixer.rot: dims must be even and at most dim, base and scaling.factor positive")
    return out


@dataclass(frozen=True)
class RizovikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: tuple[RizovikLayer, ...]
    architecture: str = "Rizovik"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RizovikConfig":
        _only(d, ("architecture", "architectures", "vocab", "width", "norm", "residual_mult", "layers"), "the top level")
        norm = _need(d, "norm", "")
        _only(norm, ("eps",), "norm")
        layers = []
        for i, raw in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            _only(raw, ("type", "mixer", "mlp", "weights_of"), where[:-1])
            kind = _need(raw, "type", where)
            m = _need(raw, "mixer", where)
            if kind in ("attention", "attention_2"):
                mixer = _window_mixer(kind, m, where)
            elif kind == "delta":
                _only(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where + "mixer")
                mixer = DeltaMixer(int(_need(m, "heads", where)), int(_need(m, "kv_heads", where)),
                                   int(_need(m, "dim", where)), int(_need(m, "vdim", where)), int(_need(m, "conv", where)))
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim, mixer.conv) < 1 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}mixer: heads, kv_heads (a divisor of heads), dim, vdim and conv must be positive")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design")
            j = raw.get("weights_of")
            layers.append(RizovikLayer(kind, mixer, _mlp(raw.get("mlp"), where + "mlp."), None if j is None else int(j)))
        if not layers:
            raise ConfigError("config.json: no layers")
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if not 0 <= j < len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(f"layers[{i}].weights_of {j} must name another layer that has tensors of its own")
            if (layers[j].type, layers[j].mixer, layers[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"layers[{i}] runs the tensors of layer {j}, but their entries differ")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(norm, "eps", "norm.")), residual_mult=float(_need(d, "residual_mult", "")),
                  layers=tuple(layers))
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.eps > 0:
            raise ConfigError("vocab and width must be positive and norm.eps above zero")
        return cfg

    @classmethod
    def from_json(cls, path) -> "RizovikConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))
