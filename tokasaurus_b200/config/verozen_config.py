"""Typed configuration of the Verozen decoder, read from its own config.json keys.

config.json gives ``vocab``, ``width``, ``norm.eps``, ``norm.groups``, ``postln_alpha``, ``token_side.dim`` (absent or
null: no per-token side input) and a list ``layers``.  A layer names its mixer ``type`` ("gla", "retention" or
"attention"), the mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null: none; ``kind``
"moe" with ``expert.ff`` and ``router``: ``experts``, ``top``, ``scale``, ``groups.count``, ``groups.keep``).  Every
size and constant of a model comes from this object, except the rank of the decays' low-rank product in a "gla" layer,
which is the row count of its first factor in the weight file unless ``mixer.rank`` gives it.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from tokasaurus_b200.config.daborax_config import _number, _pos_int
from tokasaurus_b200.config.model_config import ConfigError


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float

    @staticmethod
    def from_dict(d: dict | None, dim: int, where: str) -> "RotationConfig | None":
        if d is None:
            return None
        dims = d.get("dims", dim)
        if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims > dim or dims % 2:
            raise ConfigError(f"{where}.dims must be an even number from 0 to the head size {dim}, got {dims!r}")
        base = _number(d, "base", where, 10000.0)
        if base <= 0:
            raise ConfigError(f"{where}.base must be positive, got {base!r}")
        return RotationConfig(dims, base) if dims else None


@dataclass(frozen=True)
class GatedLinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "GatedLinearAttentionConfig":
        tau = _number(d, "tau", where, 1.0)
        if tau <= 0:
            raise ConfigError(f"{where}.tau must be positive, got {tau!r}")
        dim = _pos_int(d, "dim", where)
        return GatedLinearAttentionConfig(_pos_int(d, "heads", where), dim, _pos_int(d, "vdim", where) if "vdim" in d else dim,
                                          tau, _pos_int(d, "rank", where) if d.get("rank") is not None else None)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: RotationConfig | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "RetentionConfig":
        heads, dim = _pos_int(d, "heads", where), _pos_int(d, "dim", where)
        decay = d.get("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * heads
        if not isinstance(decay, list) or len(decay) != heads or not all(
                isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(x) for x in decay):
            raise ConfigError(f"{where}.decay must list one number a head ({heads}), got {decay!r}")
        return RetentionConfig(heads, dim, _pos_int(d, "vdim", where) if "vdim" in d else dim,
                               tuple(float(x) for x in decay), RotationConfig.from_dict(d.get("rot"), dim, where + ".rot"))


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "SigmoidAttentionConfig":
        heads, dim = _pos_int(d, "heads", where), _pos_int(d, "dim", where)
        kv_heads = _pos_int(d, "kv_heads", where) if "kv_heads" in d else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        vdim = _pos_int(d, "vdim", where) if "vdim" in d else dim
        if vdim != dim:
            raise ConfigError(f"{where}: the values are the keys, so vdim must equal dim ({dim}), got {vdim}")
        return SigmoidAttentionConfig(heads, kv_heads, dim, vdim, _number(d, "scale", where, 1.0 / math.sqrt(dim)),
                                      RotationConfig.from_dict(d.get("rot"), dim, where + ".rot"))


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    scale: float

    @staticmethod
    def from_dict(d: dict | None, where: str) -> "ExpertsConfig | None":
        if d is None:
            return None
        if d.get("kind") != "moe":
            raise ConfigError(f"{where}.kind={d.get('kind')!r} is not known ('moe')")
        r = d.get("router") or {}
        g = r.get("groups") or {}
        experts, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
        groups = _pos_int(g, "count", where + ".router.groups") if "count" in g else 1
        keep = _pos_int(g, "keep", where + ".router.groups") if "keep" in g else groups
        if experts % groups or keep > groups or top > keep * (experts // groups):
            raise ConfigError(f"{where}.router: experts={experts} in groups.count={groups} of which groups.keep={keep} "
                              f"are kept cannot give top={top}")
        return ExpertsConfig(_pos_int(d.get("expert") or {}, "ff", where + ".expert"), experts, top, groups, keep,
                             _number(r, "scale", where + ".router", 1.0))


_MIXERS = {"gla": GatedLinearAttentionConfig, "retention": RetentionConfig, "attention": SigmoidAttentionConfig}


@dataclass(frozen=True)
class VerozenLayerConfig:
    type: str
    mixer: GatedLinearAttentionConfig | RetentionConfig | SigmoidAttentionConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class VerozenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    alpha: float
    side_dim: int | None
    layers: tuple[VerozenLayerConfig, ...]
    eos_token_id: tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "VerozenConfig":
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
            layers.append(VerozenLayerConfig(kind, _MIXERS[kind].from_dict(ld.get("mixer") or {}, where + ".mixer"),
                                             ExpertsConfig.from_dict(ld.get("mlp"), where + ".mlp")))
        norm = d.get("norm") or {}
        eps = float(norm.get("eps", 1e-6))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive and finite, got {eps!r}")
        width = _pos_int(d, "width", "config")
        groups = _pos_int(norm, "groups", "norm") if "groups" in norm else 1
        if width % groups:
            raise ConfigError(f"norm.groups={groups} does not divide the width {width}")
        side = d.get("token_side")
        eos = d.get("eos_token_id")
        eos_t = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return VerozenConfig(vocab=_pos_int(d, "vocab", "config"), width=width, norm_eps=eps, norm_groups=groups,
                             alpha=_number(d, "postln_alpha", "config", 1.0),
                             side_dim=_pos_int(side, "dim", "token_side") if side else None, layers=tuple(layers),
                             eos_token_id=eos_t)
