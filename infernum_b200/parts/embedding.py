"""Token embedding and output head.

Embedding: ``h[t, :] = E[id_t, :]`` with no scaling
(infernum-llama/src/graph_builder.rs:442; infernum-cuda/kernels/embed.cu:36-50),
written straight into the float32 residual stream.

Head: ``logits = f . W_out^T`` on the rows whose logits are wanted, returned in
float32 from the 32-bit accumulator (the reference rounds them to bf16 first,
infernum-cuda/src/inner/cuda_graph_engine.rs:1297,1368).  ``tied_to`` makes the
head use the embedding table; otherwise a missing head tensor falls back to it
as in the reference (cuda_graph_engine.rs:225-232).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import EMBEDDINGS, HEADS, Embedding, Part, ResidualStream, Runtime, StateSpec, WeightSpec
from .linear import Linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """Parameters: ``vocab_size``, ``hidden_size``, ``weight``; ``act`` (True: the
    stream also carries its rounding to the activation dtype, for layers whose
    sub-layers read the stream itself); ``result_slots`` (n > 0: the stream keeps
    room for n results - the embedding's output, in slot 0, and every layer's -
    for layers that hand on a weighted sum of them); ``norm`` (a norm spec {"kind",
    "params"} with ``apply_f32``: the looked-up rows are normed, in 32-bit, before
    they become the stream); ``keep_origin`` (True: the stream keeps the embedding's
    output, as this part leaves it, in ``stream.origin``)."""

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.with_act = bool(params.get("act", False))
        self.result_slots = int(params.get("result_slots") or 0)
        self.keep_origin = bool(params.get("keep_origin", False))
        self.norm = None
        if params.get("norm"):
            from .base import NORMS

            self.norm = NORMS.get(params["norm"]["kind"])(params["norm"].get("params", {}), rt)
            if not hasattr(self.norm, "apply_f32"):
                raise ConfigError(f"token embedding: the {self.norm.kind!r} norm has no 32-bit form")
            if self.with_act or self.result_slots:
                raise ConfigError("token embedding: a normed embedding keeps no activation copy or results")
        self.weight: Optional[torch.Tensor] = None

    def forward_step(self, ctx, cache) -> ResidualStream:
        if self.norm is not None or self.keep_origin:
            x = self.forward(ctx.token_ids)
            if self.norm is not None:
                x = self.norm.apply_f32(x)
            stream = ResidualStream(x)
            if self.keep_origin:
                stream.origin = x
            return stream
        if not self.with_act and not self.result_slots:
            return ResidualStream(self.forward(ctx.token_ids))
        n, dev = ctx.token_ids.numel(), ctx.token_ids.device
        results = None
        if self.result_slots:
            results = torch.empty((self.result_slots, n, self.hidden_size), dtype=torch.float32, device=dev)
            out = results[0]
        else:
            out = torch.empty((n, self.hidden_size), dtype=torch.float32, device=dev)
        act = None
        if self.with_act and not self.rt.is_fp32:
            act = torch.empty((n, self.hidden_size), dtype=self.rt.dtype, device=dev)
        core.embed_dual(ctx.token_ids, self.weight, out, act, self.rt.err)
        stream = ResidualStream(out, (out if act is None else act) if self.with_act else None)
        stream.results = results
        return stream

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}
        if self.norm is not None:
            specs.update(self.norm.weight_specs())
        return specs

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()
        if self.norm is not None:
            self.norm.bind(weights)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden_size), dtype=torch.float32,
                          device=token_ids.device)
        core.embed(token_ids, self.weight, out, self.rt.err)
        return out


@EMBEDDINGS.register("hashed_bigram_embedding")
class HashedBigramEmbedding(Embedding):
    """``h[t] = E[id_t] + B[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]``;
    a sequence's first token takes the extra last row of ``B`` ([buckets + 1,
    hidden]).  The token before a portion's first is the request's state (one
    int32 per request slot), so that a prompt may be cut anywhere and a decoded
    token finds its predecessor on the device.  The stream gets the float32 sum
    and its rounding to the activation dtype.

    Parameters: ``vocab_size``, ``hidden_size``, ``weight``, ``bigram_weight``,
    ``buckets``, ``mul_prev``, ``mul_cur``.
    """

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.bigram_name = params["bigram_weight"]
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        self.weight: Optional[torch.Tensor] = None
        self.bigram: Optional[torch.Tensor] = None

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((1,), torch.int32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size)),
                self.bigram_name: WeightSpec((self.buckets + 1, self.hidden_size))}

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()
        self.bigram = weights[self.bigram_name].to(self.weight.dtype).contiguous()

    def forward_step(self, ctx, cache) -> ResidualStream:
        n = ctx.token_ids.numel()
        dev = ctx.token_ids.device
        out = torch.empty((n, self.hidden_size), dtype=torch.float32, device=dev)
        act = None if self.rt.is_fp32 else torch.empty((n, self.hidden_size), dtype=self.rt.dtype, device=dev)
        core.embed_hashed(ctx, cache.state.view(-1), self.weight, self.bigram, self.buckets, self.mul_prev,
                          self.mul_cur, out, act, self.rt.err)
        return ResidualStream(out, out if act is None else act)


@EMBEDDINGS.register("sinusoidal_embedding")
class SinusoidalEmbedding(Embedding):
    """``h[t] = E[id_t] + pe(p_t)`` with ``pe(p)[2i] = sin(p * base^(-2i/hidden))`` and
    ``pe(p)[2i+1] = cos`` of the same angle, ``p`` the token's position in its
    sequence.  The frequencies are rounded to float32 once (from float64); the
    angle is their 32-bit product with the position.  ``streams`` > 1 writes that
    many equal copies per token ([N, streams, hidden]) for layers that keep
    several residual streams.

    Parameters: ``vocab_size``, ``hidden_size``, ``weight``, ``base`` (default
    10000), ``streams`` (default 1: a plain [N, hidden] stream).
    """

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.base = float(params.get("base", 10000.0))
        self.streams = int(params.get("streams") or 0)
        self.weight: Optional[torch.Tensor] = None
        self.inv_freq: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()
        i2 = torch.arange(0, self.hidden_size, 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.base, dtype=torch.float64), -i2 / self.hidden_size)
        self.inv_freq = inv.to(torch.float32).to(self.weight.device)

    def forward_step(self, ctx, cache) -> ResidualStream:
        n = ctx.token_ids.numel()
        S = max(self.streams, 1)
        out = torch.empty((n, S, self.hidden_size), dtype=torch.float32, device=ctx.token_ids.device)
        core.embed_sinusoid(ctx.token_ids, ctx.positions, self.weight, self.inv_freq, out, self.rt.err)
        if self.streams >= 1:
            return ResidualStream(out, streams=S)
        return ResidualStream(out.view(n, self.hidden_size))


@HEADS.register("linear_head")
class LinearHead(Part):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.tied_to = params.get("tied_to")
        self.fallback = params.get("fallback")
        # logits <- softcap * tanh(logits / softcap) when given
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        # logits <- logits * scale when given
        self.scale = float(params["scale"]) if params.get("scale") is not None else None
        self.proj: Optional[Linear] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.tied_to:
            return {}
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size),
                                             fallback=self.fallback)}

    def bind(self, weights) -> None:
        self.proj = Linear(weights[self.tied_to or self.weight_name], self.rt)

    def weight_bytes(self) -> int:
        return self.proj.nbytes

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.proj(x, out_dtype=torch.float32)
        if self.scale is not None and self.scale != 1.0:
            core.scale_inplace(logits, self.scale)
        if self.softcap is not None:
            core.softcap(logits, self.softcap)
        return logits
