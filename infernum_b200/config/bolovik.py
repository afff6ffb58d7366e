"""Typed configuration of the Bolovik decoder (``"architecture": "Bolovik"``).

config.json of this design is nested:

    architecture, vocab, width, norm.eps, norm.groups
    layers[i].type                      "delta" or "attention"
    layers[i].mixer                     delta:     {heads, kv_heads, dim, vdim, conv}
                                        attention: {heads, kv_heads, dim, vdim, scale,
                                                    mask: {size, keep_first},
                                                    rot: {dims, base, scaling: {factor, low, high, original}}}
    layers[i].mlp                       null, {kind: "dense", ff} or
                                        {kind: "moe", expert: {ff}, router: {experts, top, groups: {count, keep}}}

Every size and constant is read here and nowhere else.  Keys that a model
leaves out mean what their absence says: no ``mask`` - every earlier token is
visible; no ``keep_first`` - the window keeps nothing; no ``rot`` - no rotation;
no ``scaling`` - plain frequencies; no ``groups`` - every expert can be chosen;
``kv_heads`` and ``vdim`` default to ``heads`` and ``dim``; ``scale`` to
``dim ** -0.5``; ``norm.groups`` to 1.  One key is not the design's and
optional: ``max_position`` bounds the scheduler's default sequence length.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .base import take_float, take_int


def _section(d: Mapping[str, Any], key: str, where: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int  # taps of the short convolution; 0: none

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "DeltaConfig":
        heads = take_int(d, "heads")
        dim = take_int(d, "dim")
        cfg = cls(heads=heads, kv_heads=take_int(d, "kv_heads", default=heads), dim=dim,
                  vdim=take_int(d, "vdim", default=dim), conv=take_int(d, "conv", default=0))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}{cfg.heads} heads are not a multiple of {cfg.kv_heads} kv_heads")
        if cfg.conv > 16:
            raise ConfigError(f"config.json: {where}a convolution of {cfg.conv} taps is beyond 16")
        return cfg


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    # (factor, low, high, original) or None
    scaling: Optional[Tuple[float, float, float, float]]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str, dim: int) -> "RotationConfig":
        dims = take_int(d, "dims", default=dim)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}dims {dims} must be even and at most the head's {dim}")
        sc = _section(d, "scaling", where, optional=True)
        scaling = None
        if sc is not None:
            scaling = (take_float(sc, "factor"), take_float(sc, "low"), take_float(sc, "high"),
                       take_float(sc, "original"))
            if scaling[2] == scaling[1]:
                raise ConfigError(f"config.json: {where}scaling.high must differ from scaling.low")
        return cls(dims=dims, base=take_float(d, "base"), scaling=scaling)


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int  # 0: every earlier token is visible
    keep_first: int  # tokens at the start of a sequence that stay visible behind the window
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "WindowAttentionConfig":
        heads = take_int(d, "heads")
        dim = take_int(d, "dim")
        mask = _section(d, "mask", where, optional=True)
        window = keep = 0
        if mask is not None:
            window = take_int(mask, "size")
            keep = take_int(mask, "keep_first", default=0, minimum=0)
        rot = _section(d, "rot", where, optional=True)
        cfg = cls(heads=heads, kv_heads=take_int(d, "kv_heads", default=heads), dim=dim,
                  vdim=take_int(d, "vdim", default=dim), scale=take_float(d, "scale", default=dim ** -0.5),
                  window=window, keep_first=keep,
                  rot=RotationConfig.from_dict(rot, where + "rot.", dim) if rot is not None else None)
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}{cfg.heads} heads are not a multiple of {cfg.kv_heads} kv_heads")
        return cfg


@dataclass(frozen=True)
class BolovikMlpConfig:
    kind: str  # "dense" | "moe"
    ff: int  # the dense width, or one expert's
    experts: int = 0
    top: int = 0
    group_count: int = 1
    group_keep: int = 1

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "BolovikMlpConfig":
        kind = d.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=take_int(d, "ff"))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind {kind!r} is not supported (dense, moe)")
        router = _section(d, "router", where)
        experts, top = take_int(router, "experts"), take_int(router, "top")
        groups = _section(router, "groups", where + "router.", optional=True)
        count = keep = 1
        if groups is not None:
            count = take_int(groups, "count")
            keep = take_int(groups, "keep", default=count)
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top {top} exceeds the {experts} experts")
        if experts % count or keep > count or keep * (experts // count) < top:
            raise ConfigError(f"config.json: {where}{experts} experts in {count} groups of which {keep} stay open "
                              f"cannot give {top} choices")
        return cls(kind="moe", ff=take_int(_section(d, "expert", where), "ff"), experts=experts, top=top,
                   group_count=count, group_keep=keep)


@dataclass(frozen=True)
class BolovikLayerConfig:
    type: str  # "delta" | "attention"
    mixer: Any  # DeltaConfig | WindowAttentionConfig
    mlp: Optional[BolovikMlpConfig]


@dataclass(frozen=True)
class BolovikConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[BolovikLayerConfig, ...]
    max_position: int = 32768
    architecture: str = "Bolovik"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BolovikConfig":
        if d.get("architecture") != "Bolovik":
            raise ConfigError(f"BolovikConfig cannot read architecture {d.get('architecture')!r}")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, ld in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(ld, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = ld.get("type")
            mixer_d = _section(ld, "mixer", where)
            if kind == "delta":
                mixer = DeltaConfig.from_dict(mixer_d, where + "mixer.")
            elif kind == "attention":
                mixer = WindowAttentionConfig.from_dict(mixer_d, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (delta, attention)")
            mlp_d = ld.get("mlp")
            if mlp_d is not None and not isinstance(mlp_d, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            mlp = BolovikMlpConfig.from_dict(mlp_d, where + "mlp.") if mlp_d is not None else None
            layers.append(BolovikLayerConfig(kind, mixer, mlp))
        norm = _section(d, "norm", "")
        width = take_int(d, "width")
        groups = take_int(norm, "groups", default=1)
        if width % groups:
            raise ConfigError(f"config.json: a width of {width} does not split in {groups} norm groups")
        return cls(vocab=take_int(d, "vocab"), width=width, norm_eps=take_float(norm, "eps"), norm_groups=groups,
                   layers=tuple(layers), max_position=take_int(d, "max_position", default=32768))
