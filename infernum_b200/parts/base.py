"""Interfaces of the parts a decoder is put together from, and their registries.

A model is described by data (``ModelSpec``): a list of layers, each naming a
block arrangement, a mixer, a feed-forward and norms by *kind* with their
parameters, and a schedule that says in which order layers run and whose cache
each run uses.  The kinds are looked up in the registries below, so a new
mixer, feed-forward, norm, position encoding or block is added by registering
a class; nothing else in the package changes.  No part knows which model it is
in: it only sees its own parameters, its weights, the rows of the step and the
cache view it is handed.

The reference composes its decoder from the same pieces inside one graph
builder (infernum-llama/src/graph_builder.rs:399-549 for prefill, :756-921 for
paged decode); here they are separate objects chosen per layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..errors import ConfigError


# --------------------------------------------------------------------------
# Descriptions (plain data)
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part wants from the checkpoint.

    ``kind``: "float" tensors are kept in bfloat16 (float32 when the file
    stores them in 32-bit, or when the engine runs in float32); "int" tensors
    become int32 tables.  ``init`` drives the random-weights mode: "normal"
    draws N(0, std), "norm" draws 1 + U(-0.1, 0.1), "zeros" and "ones" are
    constant.
    """

    shape: Tuple[int, ...]
    kind: str = "float"
    init: str = "normal"
    std: float = 0.02
    # another tensor name to take when this one is absent from the checkpoint
    fallback: Optional[str] = None
    # True: the checkpoint may leave the tensor out; the part is then bound without
    # it and must cope (the random-weights mode always draws it)
    optional: bool = False
    # A dimension of -1 in ``shape`` is taken from the checkpoint (a size that no
    # configuration key names, the rank of a low-rank pair say); the random-weights
    # mode then draws ``draw_shape``.
    draw_shape: Optional[Tuple[int, ...]] = None

    def matches(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(w < 0 or w == g for w, g in zip(self.shape, shape))

    @property
    def concrete_shape(self) -> Tuple[int, ...]:
        """The shape to draw: ``shape``, or ``draw_shape`` when a dimension is free."""
        if any(d < 0 for d in self.shape):
            if self.draw_shape is None:
                raise ConfigError(f"a tensor of shape {list(self.shape)} has a free dimension and no size to draw")
            return tuple(self.draw_shape)
        return tuple(self.shape)


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which block arrangement and which parts fill it."""

    block: str
    parts: Dict[str, PartSpec]
    name: str = ""
    # the block arrangement's own constants (a residual scale, say)
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleItem:
    """One run of a layer.  ``cache_of`` names an earlier schedule position
    whose cache this run reads instead of owning one.  ``enter``: this run is
    the first of pass number ``enter`` through a run of layers that the model
    walks several times; the model's ``pass_entry`` part transforms the stream
    before it."""

    layer: int
    cache_of: Optional[int] = None
    enter: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleItem, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    max_position: int
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    # checkpoint tensors that may be present without being used
    ignorable: Tuple[str, ...] = ()
    # what happens to the stream where a schedule item has ``enter`` (an ENTRIES kind)
    pass_entry: Optional[PartSpec] = None


@dataclass(frozen=True)
class PagedCacheSpec:
    """What a mixer needs from the paged cache: keys and values of
    ``kv_heads`` x ``head_dim`` per token; ``window`` > 0 means only the last
    ``window`` tokens are ever read, so older pages can be given back.
    ``v_head_dim``: the size of a value when it differs from a key's; 0 means
    the mixer keeps no values of their own (a latent cache, where keys and
    values are made from the one cached vector): only the key pool exists.
    ``keep_first`` (with a window): the first so many tokens of a request stay
    visible however far back they lie, so the pages that hold them are kept."""

    kv_heads: int
    head_dim: int
    window: int = 0
    v_head_dim: Optional[int] = None
    keep_first: int = 0

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else int(self.v_head_dim)

    def elements_per_token(self) -> int:
        """Cached values per token and member layer."""
        return self.kv_heads * (self.head_dim + self.value_dim)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer (one tensor of this shape per
    request slot, zeroed when the slot is taken)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What every part needs to know about the engine it runs in."""

    device: torch.device
    dtype: torch.dtype  # activation / weight dtype: torch.bfloat16 or torch.float32
    err: Optional[torch.Tensor] = None  # device error word shared by the kernels
    options: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32

    def error_word(self) -> torch.Tensor:
        """The device error word, made on first use: every kernel of a step is
        given this one word, and the engine reads it after the step."""
        if self.err is None:
            from ..ops import core

            self.err = core.new_error_word(self.device)
        return self.err


# --------------------------------------------------------------------------
# Part interfaces
# --------------------------------------------------------------------------
class Part:
    """Base of all parts.  ``params`` are the part's own sizes and constants."""

    kind: str = ""
    # Recurring steps are recorded as CUDA graphs and replayed with new
    # contents in the step's device tensors.  A part whose ``forward`` cannot
    # run that way (it branches on values it reads back from the device, or on
    # host-side fields that differ between steps of one shape) sets this to
    # False, and an engine with such a part runs every step eagerly.
    replayable: bool = True

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        self.params = dict(params)
        self.rt = rt

    def all_replayable(self) -> bool:
        return bool(self.replayable)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Checkpoint tensor name -> what it must look like."""
        return {}

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        """Take the loaded tensors (on the device, already in their kept dtype)."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (for rooflines)."""
        return 0


class Norm(Part):
    """``forward(stream)`` folds the stream's pending delta into its residual
    and returns the normed rows in the activation dtype."""

    def forward(self, stream: "ResidualStream", row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """Norm of a plain float32 tensor of rows (no residual bookkeeping)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information for a mixer.  ``apply(q, k, positions)`` changes
    ``q`` [N, heads, hd] and ``k`` [N, kv_heads, hd] in place.  A mixer may use
    a fused route for encodings it knows (rotary) and this method otherwise."""

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        raise NotImplementedError


class Embedding(Part):
    """From token ids to the float32 residual stream.  ``forward_step(ctx,
    cache)`` returns the ``ResidualStream`` of the step's rows; an embedding
    that needs something of the request besides the step's tokens (the token
    before a portion, say) declares it with ``state_spec()`` and finds it in
    ``cache.state[slot]``."""

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_step(self, ctx: Any, cache: Any) -> "ResidualStream":
        return ResidualStream(self.forward(ctx.token_ids))


class Mixer(Part):
    """Token mixing (attention, or anything that moves information between
    positions).  ``forward(x, ctx, cache)``: ``x`` is [N, hidden] in the
    activation dtype, ``ctx`` the step's ``StepContext``, ``cache`` the
    ``LayerCache`` this run reads and writes.  Returns [N, hidden]."""

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Per-token transformation.  ``forward(x, ctx)`` -> [N, hidden]."""

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of a layer's parts around the residual stream."""

    def __init__(self, params: Dict[str, Any], rt: Runtime, parts: Dict[str, Part]):
        super().__init__(params, rt)
        self.parts = parts

    @property
    def mixer(self) -> Optional[Mixer]:
        m = self.parts.get("mixer")
        return m if isinstance(m, Mixer) else None

    def state_spec(self) -> Optional[StateSpec]:
        """Per-request state of the arrangement itself, beside its mixer's (the
        inputs a convolution on what the sub-layers read still needs, say); one
        flat float32 vector per slot and scheduled run, in ``cache.block_state``."""
        return None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts.values():
            specs.update(part.weight_specs())
        return specs

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        for part in self.parts.values():
            part.bind(weights)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts.values())

    def all_replayable(self) -> bool:
        return bool(self.replayable) and all(p.all_replayable() for p in self.parts.values())

    def forward(self, stream: "ResidualStream", ctx: Any, cache: Any) -> None:
        raise NotImplementedError


class ResidualStream:
    """The hidden state between parts: a float32 residual [N, hidden] and, at
    most, one pending delta in the activation dtype that the next norm (or
    ``flush``) adds to it.  Keeping the sum in 32-bit and fusing the add into
    the norm kernel saves one pass over the rows per sub-layer."""

    def __init__(self, residual: torch.Tensor, act: Optional[torch.Tensor] = None, streams: int = 1):
        self.residual = residual
        self.pending: Optional[torch.Tensor] = None
        # More than one stream per token (hyper-connections): ``residual`` is
        # [N, streams, hidden], and a pending delta comes with the coefficients that
        # write it into the streams: ``pending_write = (mix [S, S], out [S])`` for
        # ``x_t <- sum_s mix[s, t] x_s + out[t] * delta``.
        self.streams = int(streams)
        self.pending_write = None
        # The residual rounded to the activation dtype, for arrangements whose
        # sub-layers read the stream itself (norm after the sum); valid while
        # nothing is pending.  In a float32 engine it is the residual.
        self.act = act
        # For models whose stream between layers is a weighted sum of all layers'
        # results: float32 [slots, N, hidden], slot 0 the embedding's output, slot
        # j the result of layer j - 1; filled as the layers run.
        self.results: Optional[torch.Tensor] = None
        # The embedding's output (float32 [N, hidden]) for models whose layers meet
        # it again; never written over.
        self.origin: Optional[torch.Tensor] = None

    def push(self, delta: torch.Tensor, write=None) -> None:
        if self.pending is not None:
            self.flush()
        if (write is None) != (self.residual.dim() == 2):
            raise ConfigError("a stream of several copies takes a delta with its write coefficients, "
                              "a single one without")
        self.pending = delta
        self.pending_write = write

    def flush(self) -> None:
        if self.pending is not None:
            from ..ops import core

            if self.pending_write is not None:
                mix, out_coef = self.pending_write
                core.hc_norm(self.residual, self.pending, mix, out_coef, None, None, None, 1.0, None)
            else:
                core.residual_add(self.residual, self.pending)
            self.pending = None
            self.pending_write = None


# --------------------------------------------------------------------------
# Registries
# --------------------------------------------------------------------------
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, factory: Optional[Callable[..., Part]] = None):
        def deco(f):
            self._items[kind] = f
            try:
                f.kind = kind
            except (AttributeError, TypeError):
                pass
            return f

        return deco(factory) if factory is not None else deco

    def get(self, kind: str) -> Callable[..., Part]:
        try:
            return self._items[kind]
        except KeyError:
            raise ConfigError(
                f"unknown {self.what} kind {kind!r}; registered: {sorted(self._items)}"
            ) from None

    def kinds(self) -> List[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
ENTRIES = Registry("pass entry")

_ROLE_REGISTRY = {
    "mixer": MIXERS,
    "ffn": FEED_FORWARDS,
    "feed_forward": FEED_FORWARDS,
}


def registry_for_role(role: str, spec: PartSpec) -> Registry:
    """Which registry a named part of a layer comes from: by role name, norms
    by the ``norm`` prefix."""
    if role in _ROLE_REGISTRY:
        return _ROLE_REGISTRY[role]
    if role.startswith("norm") or role.endswith("norm"):
        return NORMS
    raise ConfigError(f"layer part {role!r}: cannot tell which registry it comes from")


def build_part(role: str, spec: PartSpec, rt: Runtime) -> Part:
    return registry_for_role(role, spec).get(spec.kind)(spec.params, rt)


def build_layer(spec: LayerSpec, rt: Runtime) -> Block:
    parts = {role: build_part(role, ps, rt) for role, ps in spec.parts.items()}
    return BLOCKS.get(spec.block)({**spec.params, "name": spec.name}, rt, parts)


def register_mixer(kind: str, factory=None):
    return MIXERS.register(kind, factory)


def register_feed_forward(kind: str, factory=None):
    return FEED_FORWARDS.register(kind, factory)


def register_norm(kind: str, factory=None):
    return NORMS.register(kind, factory)


def register_position_encoding(kind: str, factory=None):
    return POSITION_ENCODINGS.register(kind, factory)


def register_block(kind: str, factory=None):
    return BLOCKS.register(kind, factory)
