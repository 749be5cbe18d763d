"""Typed configuration of the Bibalix decoder, read from its own config.json keys.

config.json gives ``vocab``, ``width``, ``norm.eps`` and a list ``layers``.  A layer names its mixer ``type``
("attention": differential attention; "latent_attention"), the mixer's sizes and constants under ``mixer`` (``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff``, ``mask.size`` / ``mask.keep_first``, ``rot.base`` / ``rot.dims`` /
``rot.scaling``: ``factor``, ``original``, ``fast``, ``slow``; for latent attention also ``rot_dim`` and ``kv_rank``), and
its feed-forward under ``mlp`` (null: none; ``kind`` "dense" with ``ff``; ``kind`` "moe" with ``expert.ff`` /
``expert.limit``, ``router.experts`` / ``router.top`` / ``router.scale`` and optionally ``shared.ff`` / ``shared.limit``).
Every size and constant of a model comes from this object.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from tokasaurus_b200.config.daborax_config import _number, _pos_int
from tokasaurus_b200.config.model_config import ConfigError


@dataclass(frozen=True)
class RotationScaling:
    """Blend of scaled and unscaled frequencies by how many turns a pair makes in ``original`` positions."""

    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: RotationScaling | None

    @staticmethod
    def from_dict(d: dict | None, most: int, where: str) -> "Rotation | None":
        if d is None:
            return None
        dims = d.get("dims", most)
        if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims > most or dims % 2:
            raise ConfigError(f"{where}.dims must be an even number from 0 to {most}, got {dims!r}")
        base = _number(d, "base", where, 10000.0)
        if base <= 1:
            raise ConfigError(f"{where}.base must be above 1, got {base!r}")
        scaling = None
        sc = d.get("scaling")
        if sc is not None:
            w = where + ".scaling"
            scaling = RotationScaling(_number(sc, "factor", w), _pos_int(sc, "original", w), _number(sc, "fast", w, 32.0),
                                      _number(sc, "slow", w, 1.0))
            if scaling.factor <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                raise ConfigError(f"{w}: factor, fast and slow must be positive")
        return Rotation(dims, base, scaling) if dims else None


def _mask(d: dict | None, where: str, keep_allowed: bool) -> tuple[int | None, int]:
    """(window or None, positions kept in sight before it)."""
    if not d:
        return None, 0
    size = _pos_int(d, "size", where) if d.get("size") is not None else None
    keep = d.get("keep_first", 0)
    if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
        raise ConfigError(f"{where}.keep_first must be a count, got {keep!r}")
    if keep and not keep_allowed:
        raise ConfigError(f"{where}.keep_first: this mixer's window keeps no first positions")
    return size, (keep if size is not None else 0)


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int | None
    keep_first: int
    rot: Rotation | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "DifferentialAttentionConfig":
        heads, dim = _pos_int(d, "heads", where), _pos_int(d, "dim", where)
        kv_heads = _pos_int(d, "kv_heads", where) if "kv_heads" in d else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        window, keep = _mask(d.get("mask"), where + ".mask", True)
        rot = Rotation.from_dict(d.get("rot"), dim, where + ".rot")
        if rot is not None and rot.scaling is not None:
            raise ConfigError(f"{where}.rot.scaling: this mixer's rotation is not scaled")
        return DifferentialAttentionConfig(heads, kv_heads, dim, _pos_int(d, "vdim", where) if "vdim" in d else dim,
                                           _number(d, "scale", where, 1.0 / math.sqrt(dim)), _number(d, "diff", where),
                                           window, keep, rot)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int | None
    rot: Rotation | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "LatentAttentionConfig":
        dim, rot_dim = _pos_int(d, "dim", where), _pos_int(d, "rot_dim", where)
        window, _ = _mask(d.get("mask"), where + ".mask", False)
        return LatentAttentionConfig(_pos_int(d, "heads", where), dim, rot_dim,
                                     _pos_int(d, "vdim", where) if "vdim" in d else dim, _pos_int(d, "kv_rank", where),
                                     _number(d, "scale", where, 1.0 / math.sqrt(dim + rot_dim)), window,
                                     Rotation.from_dict(d.get("rot"), rot_dim, where + ".rot"))


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int
    limit: float | None = None  # moe: the experts' clamp
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    shared_ff: int | None = None
    shared_limit: float | None = None

    @staticmethod
    def from_dict(d: dict | None, where: str) -> "FeedForwardConfig | None":
        if d is None:
            return None
        kind = d.get("kind")
        if kind == "dense":
            return FeedForwardConfig("dense", _pos_int(d, "ff", where))
        if kind != "moe":
            raise ConfigError(f"{where}.kind={kind!r} is not known ('dense', 'moe')")
        ex, r, sh = d.get("expert") or {}, d.get("router") or {}, d.get("shared")
        experts, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"{where}.router: top={top} of {experts} experts")
        limit = _number(ex, "limit", where + ".expert")
        shared_limit = _number(sh, "limit", where + ".shared") if sh else None
        if limit <= 0 or (shared_limit is not None and shared_limit <= 0):
            raise ConfigError(f"{where}: an expert's limit must be positive")
        return FeedForwardConfig("moe", _pos_int(ex, "ff", where + ".expert"), limit, experts, top,
                                 _number(r, "scale", where + ".router", 1.0),
                                 _pos_int(sh, "ff", where + ".shared") if sh else None, shared_limit)


_MIXERS = {"attention": DifferentialAttentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class BibalixLayerConfig:
    type: str
    mixer: DifferentialAttentionConfig | LatentAttentionConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class BibalixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[BibalixLayerConfig, ...]
    eos_token_id: tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "BibalixConfig":
        for key in ("vocab", "width", "layers"):
            if key not in d:
                raise ConfigError(f"config.json lacks the key {key!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, ld in enumerate(d["layers"]):
            where = f"layers[{i}]"
            kind = ld.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type={kind!r} is not known ({', '.join(repr(k) for k in _MIXERS)})")
            layers.append(BibalixLayerConfig(kind, _MIXERS[kind].from_dict(ld.get("mixer") or {}, where + ".mixer"),
                                             FeedForwardConfig.from_dict(ld.get("mlp"), where + ".mlp")))
        eps = float((d.get("norm") or {}).get("eps", 1e-6))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive and finite, got {eps!r}")
        eos = d.get("eos_token_id")
        eos_t = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return BibalixConfig(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"), norm_eps=eps,
                             layers=tuple(layers), eos_token_id=eos_t)
