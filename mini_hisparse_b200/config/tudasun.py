"""Typed Tudasun configuration, read from the design's own config.json.

Keys: ``architecture`` ("Tudasun"), ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (absent or null: none),
``token_side.dim`` (absent or null: no per-layer token input) and ``layers``, a list whose entries give ``type``
("gla", "hgrn2" or "latent_attention"), the mixer's sizes ``mixer`` and the feed-forward ``mlp``: null for none;
``kind`` "dense" with ``ff``; or ``kind`` "moe" with ``expert.ff``, ``router`` (``experts``, ``identity``, ``top``,
``groups.count`` and ``groups.keep``) and ``shared.ff`` (absent or null: no shared expert).  No size has a default; a
key this reader does not know is refused, so that a variant it cannot compute never runs as something else.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .koronex import _need, _only
from .qwen2 import ConfigError


@dataclass(frozen=True)
class DecayMixer:
    """"gla" and "hgrn2": heads of ``dim`` key channels over values ``vdim`` wide; tau and decay_rank for "gla" only
    (decay_rank None: whatever the checkpoint's matrices have)."""

    heads: int
    dim: int
    vdim: int
    tau: float | None = None
    decay_rank: int | None = None


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    kv_from: int | None


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    identity: int
    top: int
    group_count: int
    group_keep: int
    expert_ff: int
    shared_ff: int | None


@dataclass(frozen=True)
class TudasunLayer:
    type: str
    mixer: DecayMixer | LatentMixer
    mlp: DenseFF | RoutedFF | None


def _mlp(raw, where: str):
    if raw is None:
        return None
    kind = _need(raw, "kind", where)
    if kind == "dense":
        _only(raw, ("kind", "ff"), where[:-1])
        ff = int(_need(raw, "ff", where))
        if ff < 1:
            raise ConfigError(f"{where}ff must be positive")
        return DenseFF(ff)
    if kind != "moe":
        raise ConfigError(f"{where}kind {kind!r} is not a feed-forward of this design")
    _only(raw, ("kind", "expert", "router", "shared"), where[:-1])
    expert, router = _need(raw, "expert", where), _need(raw, "router", where)
    _only(expert, ("ff",), where + "expert")
    _only(router, ("experts", "identity", "top", "groups"), where + "router")
    groups = router.get("groups")
    count = keep = 1
    if groups is not None:
        _only(groups, ("count", "keep"), where + "router.groups")
        count, keep = int(_need(groups, "count", where + "router.groups.")), int(_need(groups, "keep", where + "router.groups."))
    shared = raw.get("shared")
    if shared is not None:
        _only(shared, ("ff",), where + "shared")
    out = RoutedFF(int(_need(router, "experts", where + "router.")), int(router.get("identity") or 0),
                   int(_need(router, "top", where + "router.")), count, keep, int(_need(expert, "ff", where + "expert.")),
                   None if shared is None else int(_need(shared, "ff", where + "shared.")))
    n = out.experts + out.identity
    if out.experts < 0 or out.identity < 0 or n < 1 or out.expert_ff < 1:
        raise ConfigError(f"{where}router: experts, identity and expert.ff must make sense")
    if count < 1 or n % count or not 1 <= keep <= count:
        raise ConfigError(f"{where}router.groups: {n} outputs do not form {count} equal groups of which {keep} are kept")
    if not 1 <= out.top <= n // count * keep:
        raise ConfigError(f"{where}router.top {out.top} is more than the kept groups hold")
    return out


@dataclass(frozen=True)
class TudasunConfig:
    vocab: int
    width: int
    eps: float
    softcap: float | None
    side_dim: int | None
    layers: tuple[TudasunLayer, ...]
    architecture: str = "Tudasun"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TudasunConfig":
        _only(d, ("architecture", "architectures", "vocab", "width", "norm", "logit_softcap", "token_side", "layers"),
              "the top level")
        norm = _need(d, "norm", "")
        _only(norm, ("eps",), "norm")
        side = d.get("token_side")
        if side is not None:
            _only(side, ("dim",), "token_side")
        layers = []
        for i, raw in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            _only(raw, ("type", "mixer", "mlp"), where[:-1])
            kind = _need(raw, "type", where)
            m = _need(raw, "mixer", where)
            if kind == "gla":
                _only(m, ("heads", "dim", "vdim", "tau", "decay_rank"), where + "mixer")
                rank = m.get("decay_rank")
                mixer = DecayMixer(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "vdim", where)),
                                   float(_need(m, "tau", where)), None if rank is None else int(rank))
                if not mixer.tau > 0:
                    raise ConfigError(f"{where}mixer.tau must be positive")
            elif kind == "hgrn2":
                _only(m, ("heads", "dim", "vdim"), where + "mixer")
                mixer = DecayMixer(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "vdim", where)))
            elif kind == "latent_attention":
                _only(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot", "kv_from"), where + "mixer")
                rot = _need(m, "rot", where)
                _only(rot, ("dims", "base"), where + "mixer.rot")
                mixer = LatentMixer(int(_need(m, "heads", where)), int(_need(m, "dim", where)),
                                    int(_need(m, "rot_dim", where)), int(_need(m, "vdim", where)),
                                    int(_need(m, "kv_rank", where)), float(_need(m, "scale", where)),
                                    float(_need(rot, "base", where)), None if m.get("kv_from") is None else int(m["kv_from"]))
                if int(_need(rot, "dims", where)) != mixer.rot_dim:
                    raise ConfigError(f"{where}mixer.rot.dims must equal rot_dim: the whole rotated part turns")
                if mixer.rot_dim % 2 or mixer.rot_dim < 0 or mixer.kv_rank < 1:
                    raise ConfigError(f"{where}mixer: rot_dim must be even and kv_rank positive")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design")
            if min(mixer.heads, mixer.dim, mixer.vdim) < 1:
                raise ConfigError(f"{where}mixer: heads, dim and vdim must be positive")
            layers.append(TudasunLayer(kind, mixer, _mlp(raw.get("mlp"), where + "mlp.")))
        if not layers:
            raise ConfigError("config.json: no layers")
        for i, layer in enumerate(layers):
            j = getattr(layer.mixer, "kv_from", None)
            if j is None:
                continue
            if not 0 <= j < i or layers[j].type != "latent_attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from {j} must name an earlier latent layer with a latent of its own")
            a, b = layer.mixer, layers[j].mixer
            if (a.kv_rank, a.rot_dim, a.rot_base) != (b.kv_rank, b.rot_dim, b.rot_base):
                raise ConfigError(f"layers[{i}] reads the latent of layer {j}, whose kv_rank, rot_dim or rotation differ")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(norm, "eps", "norm.")), softcap=None if cap is None else float(cap),
                  side_dim=None if side is None else int(_need(side, "dim", "token_side.")), layers=tuple(layers))
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.eps > 0:
            raise ConfigError("vocab and width must be positive and norm.eps above zero")
        if cfg.softcap is not None and not cfg.softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        return cfg

    @classmethod
    def from_json(cls, path) -> "TudasunConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))
