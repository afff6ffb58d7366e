"""Typed configuration of the Vodatar decoder (``"architecture": "Vodatar"``).

config.json of this design is nested:

    architecture, vocab, width, residual_mult, norm.eps, norm.groups, canon.taps
    loop                                null or {start, stop, times}
    layers[i].type                      "attention" or "latent_attention"
    layers[i].mixer                     attention:        {heads, kv_heads, dim, vdim, scale, softcap, diff, conv,
                                                           rot: {dims, base}}
                                        latent_attention: {heads, dim, rot_dim, vdim, kv_rank, scale,
                                                           rot: {dims, base, scaling: {factor, original, fast, slow}}}
    layers[i].mlp                       null or {kind: "moe", expert: {ff}, router: {experts, top, identity},
                                                 shared: {ff}}

Every size and constant is read here and nowhere else.  Keys that a model leaves
out mean what their absence says: no ``loop`` - every layer runs once; no
``canon`` - sub-layers read the normed stream as it is; no ``conv`` - projections
are used as they are; no ``softcap`` - scores are not capped; no ``rot`` (or
``dims`` 0) - no rotation; no ``scaling`` - plain frequencies; no ``identity`` -
every router output has an expert; no ``shared`` - no expert that all tokens
use; ``kv_heads`` and ``vdim`` default to ``heads`` and ``dim``, ``scale`` to the
inverse root of the query's size, ``norm.groups`` and ``residual_mult`` to 1.  One
key is not the design's and optional: ``max_position`` bounds the scheduler's
default sequence length.
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
class RampScaling:
    """Frequencies divided by ``factor`` along a ramp over the pair index that
    runs between the pairs making ``fast`` and ``slow`` turns over ``original``
    positions; cosine and sine grow by ``0.1 ln(factor) + 1``."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class PairRotation:
    dims: int  # rotated dimensions, neighbours paired; 0: none
    base: float
    scaling: Optional[RampScaling]

    @classmethod
    def from_dict(cls, d: Optional[Mapping[str, Any]], where: str, limit: int) -> "PairRotation":
        if d is None:
            return cls(0, 10000.0, None)
        dims = take_int(d, "dims", default=limit, minimum=0)
        if dims % 2 or dims > limit:
            raise ConfigError(f"config.json: {where}dims {dims} must be even and at most {limit}")
        sc = _section(d, "scaling", where, optional=True)
        scaling = None
        if sc is not None:
            scaling = RampScaling(take_float(sc, "factor"), take_float(sc, "original"), take_float(sc, "fast"),
                                  take_float(sc, "slow"))
            if scaling.factor <= 0 or scaling.original <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                raise ConfigError(f"config.json: {where}scaling values must be positive")
        base = take_float(d, "base", default=10000.0)
        if base <= 1.0 and dims:
            raise ConfigError(f"config.json: {where}base must exceed 1")
        return cls(dims, base, scaling)


@dataclass(frozen=True)
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int  # of one score map's queries and keys
    vdim: int
    scale: float
    softcap: float  # 0: scores are not capped
    diff: float
    conv: int  # taps of the convolution on q, k, v; 0: none
    rot: PairRotation

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "DiffAttentionConfig":
        heads, dim = take_int(d, "heads"), take_int(d, "dim")
        cfg = cls(heads=heads, kv_heads=take_int(d, "kv_heads", default=heads), dim=dim,
                  vdim=take_int(d, "vdim", default=dim), scale=take_float(d, "scale", default=dim ** -0.5),
                  softcap=take_float(d, "softcap", default=0.0), diff=take_float(d, "diff", default=0.0),
                  conv=take_int(d, "conv", default=0, minimum=0),
                  rot=PairRotation.from_dict(_section(d, "rot", where, optional=True), where + "rot.", dim))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}{cfg.heads} heads are not a multiple of {cfg.kv_heads} kv_heads")
        if cfg.conv > 16:
            raise ConfigError(f"config.json: {where}a convolution of {cfg.conv} taps is beyond 16")
        if cfg.softcap < 0:
            raise ConfigError(f"config.json: {where}softcap must not be negative")
        if cfg.rot.dims and cfg.dim % 2:
            raise ConfigError(f"config.json: {where}rotated maps need an even dim")
        return cfg


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int  # unrotated query/key dimensions per head
    rot_dim: int  # rotated ones
    vdim: int
    kv_rank: int
    scale: float
    rot: PairRotation

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LatentConfig":
        dim, rot_dim = take_int(d, "dim", minimum=0), take_int(d, "rot_dim", default=0, minimum=0)
        if dim + rot_dim <= 0:
            raise ConfigError(f"config.json: {where}a head needs query dimensions")
        rot_d = _section(d, "rot", where, optional=True)
        rot = PairRotation.from_dict(rot_d, where + "rot.", rot_dim) if rot_dim else PairRotation(0, 10000.0, None)
        return cls(heads=take_int(d, "heads"), dim=dim, rot_dim=rot_dim, vdim=take_int(d, "vdim", default=max(dim, 1)),
                   kv_rank=take_int(d, "kv_rank"), scale=take_float(d, "scale", default=(dim + rot_dim) ** -0.5),
                   rot=rot)


@dataclass(frozen=True)
class VodatarMlpConfig:
    ff: int  # one expert's width
    experts: int
    top: int
    identity: int  # router outputs behind the experts that hand the input on
    shared_ff: int  # 0: no expert that every token uses

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "VodatarMlpConfig":
        kind = d.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind {kind!r} is not supported (moe)")
        router = _section(d, "router", where)
        experts, top = take_int(router, "experts"), take_int(router, "top")
        identity = take_int(router, "identity", default=0, minimum=0)
        if top > experts + identity:
            raise ConfigError(f"config.json: {where}router.top {top} exceeds the {experts + identity} router outputs")
        shared = _section(d, "shared", where, optional=True)
        return cls(ff=take_int(_section(d, "expert", where), "ff"), experts=experts, top=top,
                   identity=identity, shared_ff=take_int(shared, "ff") if shared is not None else 0)


@dataclass(frozen=True)
class VodatarLayerConfig:
    type: str  # "attention" | "latent_attention"
    mixer: Any  # DiffAttentionConfig | LatentConfig
    mlp: Optional[VodatarMlpConfig]


@dataclass(frozen=True)
class VodatarConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    canon_taps: int  # 0: no convolution on what a sub-layer reads
    loop: Optional[Tuple[int, int, int]]  # (start, stop, times)
    layers: Tuple[VodatarLayerConfig, ...]
    max_position: int = 32768
    architecture: str = "Vodatar"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VodatarConfig":
        if d.get("architecture") != "Vodatar":
            raise ConfigError(f"VodatarConfig cannot read architecture {d.get('architecture')!r}")
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
            if kind == "attention":
                mixer = DiffAttentionConfig.from_dict(mixer_d, where + "mixer.")
            elif kind == "latent_attention":
                mixer = LatentConfig.from_dict(mixer_d, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (attention, latent_attention)")
            mlp_d = ld.get("mlp")
            if mlp_d is not None and not isinstance(mlp_d, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            mlp = VodatarMlpConfig.from_dict(mlp_d, where + "mlp.") if mlp_d is not None else None
            layers.append(VodatarLayerConfig(kind, mixer, mlp))
        norm = _section(d, "norm", "")
        width = take_int(d, "width")
        groups = take_int(norm, "groups", default=1)
        if width % groups:
            raise ConfigError(f"config.json: a width of {width} does not split in {groups} norm groups")
        canon = _section(d, "canon", "", optional=True)
        taps = take_int(canon, "taps", default=0, minimum=0) if canon is not None else 0
        if taps > 16:
            raise ConfigError(f"config.json: canon.taps {taps} is beyond 16")
        loop_d = _section(d, "loop", "", optional=True)
        loop = None
        if loop_d is not None:
            loop = (take_int(loop_d, "start", minimum=0), take_int(loop_d, "stop", minimum=0),
                    take_int(loop_d, "times", default=1))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"config.json: loop {loop[0]}..{loop[1]} does not name a run of the {len(layers)} layers")
        return cls(vocab=take_int(d, "vocab"), width=width, norm_eps=take_float(norm, "eps"), norm_groups=groups,
                   residual_mult=take_float(d, "residual_mult", default=1.0), canon_taps=taps, loop=loop,
                   layers=tuple(layers), max_position=take_int(d, "max_position", default=32768))
