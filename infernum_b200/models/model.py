"""The generic decoder: built from a ``ModelSpec``, it owns the parts, runs
the schedule over a step's rows and returns logits for the wanted rows.

Order of a forward pass (infernum-llama/src/graph_builder.rs:442-536):
embedding -> scheduled layers -> final norm on the wanted rows only -> head.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from ..parts import (EMBEDDINGS, ENTRIES, HEADS, NORMS, Block, ModelSpec, PagedCacheSpec, ResidualStream,
                     Runtime, StateSpec, WeightSpec, build_layer)


@dataclass(frozen=True)
class CacheNeed:
    """What one scheduled run of a layer needs from the cache manager."""

    position: int  # index in the schedule
    paged: Optional[PagedCacheSpec]
    state: Optional[StateSpec]
    cache_of: Optional[int]  # reads the cache of this earlier schedule position
    block_state: Optional[StateSpec] = None  # state of the layer's arrangement itself, per run


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, rt)
        self.layers: List[Block] = [build_layer(ls, rt) for ls in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, rt)
        self.head = HEADS.get(spec.lm_head.kind)(spec.lm_head.params, rt)
        self.schedule = tuple(spec.schedule)
        self.pass_entry = ENTRIES.get(spec.pass_entry.kind)(spec.pass_entry.params, rt) if spec.pass_entry else None
        for pos, item in enumerate(self.schedule):
            if item.enter is not None and self.pass_entry is None:
                raise ConfigError(f"schedule[{pos}] begins a pass, the model names no pass entry")
            if not 0 <= item.layer < len(self.layers):
                raise ConfigError(f"schedule[{pos}] names layer {item.layer}, there are "
                                  f"{len(self.layers)}")
            if item.cache_of is not None and not 0 <= item.cache_of < pos:
                raise ConfigError(f"schedule[{pos}].cache_of must name an earlier position")
            if item.cache_of is not None and self.schedule[item.cache_of].cache_of is not None:
                raise ConfigError(f"schedule[{pos}].cache_of must name a run that owns its cache")
        self.bound = False

    # ---- declarations -------------------------------------------------------
    def _all_parts(self):
        extra = [self.pass_entry] if self.pass_entry is not None else []
        return [self.embedding, *extra, *self.layers, self.final_norm, self.head]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self._all_parts():
            for name, ws in part.weight_specs().items():
                if name in specs and tuple(specs[name].shape) != tuple(ws.shape):
                    raise ConfigError(f"tensor {name!r} is declared twice with different shapes")
                specs[name] = ws
        return specs

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        for part in self._all_parts():
            part.bind(weights)
        self.bound = True

    @property
    def replayable(self) -> bool:
        """Whether every part can run from a recorded CUDA graph."""
        return all(part.all_replayable() for part in self._all_parts())

    def cache_needs(self) -> List[CacheNeed]:
        """One need per schedule position and, when the embedding keeps state
        of a request, one more behind them (``caches[len(schedule)]``)."""
        needs = []
        for pos, item in enumerate(self.schedule):
            mixer = self.layers[item.layer].mixer
            paged = mixer.cache_spec() if mixer is not None else None
            state = mixer.state_spec() if mixer is not None else None
            needs.append(CacheNeed(pos, paged, state, item.cache_of, self.layers[item.layer].state_spec()))
        embed_state = self.embedding.state_spec() if hasattr(self.embedding, "state_spec") else None
        if embed_state is not None:
            needs.append(CacheNeed(len(self.schedule), None, embed_state, None))
        return needs

    def step_weight_bytes(self) -> int:
        """Bytes of weights that one step reads: every scheduled layer once, the
        final norm and the head; of the embedding only the rows looked up."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for item in self.schedule:
            total += self.layers[item.layer].weight_bytes()
            if item.enter is not None:
                total += self.pass_entry.weight_bytes()
        return total

    # ---- the forward pass of one step ---------------------------------------
    def forward(self, ctx, caches) -> Optional[torch.Tensor]:
        """Runs the step's rows through the schedule.  ``caches[i]`` is the
        ``LayerCache`` of schedule position i.  Returns float32 logits
        [wanted rows, vocab], or None when no row is wanted."""
        if not self.bound:
            raise ConfigError("the model has no weights bound")
        with core.step_stream(self.rt.device):
            # nothing of this step starts before what describes it (positions, tables) is complete
            core.step_fence(self.rt.device)
            if hasattr(self.embedding, "forward_step"):
                embed_cache = caches[len(self.schedule)] if len(caches) > len(self.schedule) else None
                stream = self.embedding.forward_step(ctx, embed_cache)
            else:
                stream = ResidualStream(self.embedding.forward(ctx.token_ids))
            for item, cache in zip(self.schedule, caches):
                if item.enter is not None:
                    self.pass_entry.forward(stream, item.enter)
                self.layers[item.layer].forward(stream, ctx, cache)
            if ctx.logit_rows is None or ctx.logit_rows.numel() == 0:
                return None
            normed = self.final_norm.forward(stream, row_idx=ctx.logit_rows)
            return self.head.forward(normed)
