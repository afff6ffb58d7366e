"""Grouped-query causal attention over the paged cache.

Per layer (infernum-llama/src/graph_builder.rs:456-483 for prefill, :819-864
for paged decode): q, k, v projections without bias; q -> [N, heads, hd],
k, v -> [N, kv_heads, hd]; position encoding on q and k; the new k and v are
written to the request's pages at the token's absolute position; query head a
reads kv head a / (heads / kv_heads); scores scaled by 1/sqrt(hd); causal
softmax in 32-bit; output projection.

The three projections are one product with the row-concatenated weight
``[Wq; Wk; Wv]`` (the reference does this for decode,
infernum-llama/src/graph_builder.rs:819-827); only the fused copy is kept.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
``position`` (a position-encoding spec: {"kind", "params"}, or None),
``window`` (0 = all keys), ``scale`` (default 1/sqrt(head_dim)),
``prefix`` (checkpoint prefix, e.g. "model.layers.0.self_attn."),
``kv_shared`` (True: the layer has no k/v projection and reads the cache of
another run named by the schedule).

Options beyond the Llama layer, all off by default:
``names`` (the tensors' names behind the prefix: ``q``, ``k``, ``v``, ``o``);
``qk_norm`` ({"q": name, "k": name, "eps": e}): queries and keys are divided by
their root mean square per head and multiplied by a weight of ``head_dim``
values that all heads share, before the scores;
``value_from_key`` (True: there is no value projection; a token's value is its
key as projected, before any norm);
``sink`` (a tensor name: one learned logit per head whose exponential is added
to the softmax's denominator; it has no key and no value and is not scaled);
``gate`` (a tensor name: the concatenated heads are multiplied by
``sigmoid(W_gate x)`` before the output projection);
``v_head_dim`` (the size of a value head when it differs from a key's);
``biases`` ({"q": name, "k": name, "v": name}: biases of the three projections);
``unit_norm`` ({"eps": e, "value": bool}: after the rotation, queries and keys are
divided by their root mean square per head, without a weight; with ``value`` each
value head likewise before it is written to the pages); may be combined with a rotary ``position``;
``keep_first`` (with a window: the first so many tokens of a request stay visible
to every later query, at their own positions).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import attention as attn_ops
from ..ops import core
from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedCacheSpec, Runtime, WeightSpec
from .linear import Linear
from .rope import RotaryEmbedding


@MIXERS.register("attention")
class Attention(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params.get("num_kv_heads", self.num_heads))
        self.head_dim = int(params["head_dim"])
        self.window = int(params.get("window") or 0)
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.prefix = params.get("prefix", "")
        self.kv_shared = bool(params.get("kv_shared", False))
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(
                f"attention: {self.num_heads} heads are not a multiple of "
                f"{self.num_kv_heads} key/value heads")
        pos = params.get("position")
        self.position = None
        if pos:
            self.position = POSITION_ENCODINGS.get(pos["kind"])(pos.get("params", {}), rt)
        names = params.get("names") or {}
        self.names = {k: self.prefix + names.get(k, f"{k}_proj.weight") for k in ("q", "k", "v", "o")}
        qk_norm = params.get("qk_norm")
        self.qk_norm = None
        if qk_norm:
            self.qk_norm = {"q": self.prefix + qk_norm["q"], "k": self.prefix + qk_norm["k"],
                            "eps": float(qk_norm["eps"])}
        self.value_from_key = bool(params.get("value_from_key", False))
        self.v_head_dim = int(params.get("v_head_dim") or self.head_dim)
        self.keep_first = int(params.get("keep_first") or 0) if self.window > 0 else 0
        biases = params.get("biases")
        self.bias_names = {k: self.prefix + biases[k] for k in ("q", "k", "v")} if biases else None
        unit = params.get("unit_norm")
        self.unit_norm = {"eps": float(unit["eps"]), "value": bool(unit.get("value", False))} if unit else None
        self.fused_prep = bool(self.bias_names or self.unit_norm or self.v_head_dim != self.head_dim)
        self.bias = None
        self.sink_name = self.prefix + params["sink"] if params.get("sink") else None
        self.gate_name = self.prefix + params["gate"] if params.get("gate") else None
        if (self.qk_norm or self.value_from_key) and self.position is not None:
            raise ConfigError("attention: normed queries and keys, or values taken from keys, "
                              "are not combined with a position encoding")
        if self.fused_prep and (self.qk_norm or self.value_from_key or self.kv_shared or self.gate_name):
            raise ConfigError("attention: biases, weightless norms after the rotation or values of another size "
                              "are not combined with weighted norms, values taken from keys, a gate or a shared cache")
        if self.fused_prep and self.position is not None and not isinstance(self.position, RotaryEmbedding):
            raise ConfigError("attention: biases and weightless norms go with a rotary position encoding or none")
        if (self.qk_norm or self.value_from_key) and self.kv_shared:
            raise ConfigError("attention: normed keys or values taken from keys need a cache of the layer's own")
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_norm_w = self.k_norm_w = self.sink = None

    # ---- declarations -----------------------------------------------------
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        if self.v_head_dim != self.head_dim or self.keep_first:
            return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim,
                                  keep_first=self.keep_first)
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        qd, kvd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        vd, od = self.num_kv_heads * self.v_head_dim, self.num_heads * self.v_head_dim
        specs = {
            self.names["q"]: WeightSpec((qd, self.hidden_size)),
            self.names["o"]: WeightSpec((self.hidden_size, od)),
        }
        if not self.kv_shared:
            specs[self.names["k"]] = WeightSpec((kvd, self.hidden_size))
            if not self.value_from_key:
                specs[self.names["v"]] = WeightSpec((vd, self.hidden_size))
        if self.bias_names:
            for k, n in ((("q"), qd), ("k", kvd), ("v", vd)):
                specs[self.bias_names[k]] = WeightSpec((n,), init="normal", std=0.1)
        if self.qk_norm:
            specs[self.qk_norm["q"]] = WeightSpec((self.head_dim,), init="norm")
            specs[self.qk_norm["k"]] = WeightSpec((self.head_dim,), init="norm")
        if self.sink_name:
            specs[self.sink_name] = WeightSpec((self.num_heads,), init="normal", std=1.0)
        if self.gate_name:
            specs[self.gate_name] = WeightSpec((qd, self.hidden_size))
        return specs

    def bind(self, weights) -> None:
        keys = ["q"] + ([] if self.kv_shared else (["k"] if self.value_from_key else ["k", "v"]))
        mats = [weights[self.names[n]] for n in keys]
        if self.gate_name:
            mats.append(weights[self.gate_name])  # the gate rides in the same product, behind q, k (and v)
        if len({m.dtype for m in mats}) != 1:
            raise ConfigError(f"{self.prefix}: q/k/v projections are stored in different dtypes")
        self.qkv = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0], self.rt)
        self.o = Linear(weights[self.names["o"]], self.rt)
        if self.qk_norm:
            self.q_norm_w = weights[self.qk_norm["q"]].to(torch.float32).contiguous()
            self.k_norm_w = weights[self.qk_norm["k"]].to(torch.float32).contiguous()
        if self.sink_name:
            self.sink = weights[self.sink_name].to(torch.float32).contiguous()
        if self.bias_names:
            self.bias = torch.cat([weights[self.bias_names[k]].to(torch.float32).view(-1)
                                   for k in ("q", "k", "v")]).contiguous()

    def weight_bytes(self) -> int:
        return self.qkv.nbytes + self.o.nbytes

    # ---- the step -----------------------------------------------------------
    def project(self, x: torch.Tensor) -> torch.Tensor:
        """The fused product: rows of q | k | (v) | (gate)."""
        return self.qkv(x)

    @property
    def projected_rows(self) -> int:
        return self.qkv.out_features

    def forward(self, x: torch.Tensor, ctx, cache, projected: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``projected``: the fused product when the caller has already made it
        (as part of a wider one); a view of wider rows is fine."""
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = projected if projected is not None else self.qkv(x)  # [N, (nh + 2 nkv) hd (+ gate)], or [N, nh hd] when the cache is shared
        tables = ctx.block_tables[cache.group]
        if self.fused_prep:
            if not cache.owner:
                raise ConfigError("attention with biases or weightless norms must own its cache")
            rotary = self.position
            core.rope_norm_append(qkv, self.bias, rotary.inv_freq if rotary else None,
                                  rotary.rotary_dim if rotary else 0, self.unit_norm is not None,
                                  bool(self.unit_norm and self.unit_norm["value"]),
                                  self.unit_norm["eps"] if self.unit_norm else 1e-6, nh, nkv, hd, ctx.positions,
                                  ctx.row_entry, tables, cache.k_pool, cache.v_pool, self.rt.err)
            return self._attend(qkv, ctx, cache, tables)
        if self.qk_norm or self.value_from_key:
            if not cache.owner:
                raise ConfigError("attention with normed keys must own its cache")
            v_off = -1 if self.value_from_key else (nh + nkv) * hd
            core.qk_norm_append(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm["eps"] if self.qk_norm else 1e-6,
                                nh, nkv, hd, v_off, ctx.positions, ctx.row_entry, tables, cache.k_pool, cache.v_pool,
                                self.rt.err)
            return self._attend(qkv, ctx, cache, tables)
        writes = cache.owner and not self.kv_shared
        if self.kv_shared and cache.owner:
            raise ConfigError("a kv_shared attention layer must be scheduled with cache_of")
        rotary = self.position if isinstance(self.position, RotaryEmbedding) else None
        if self.position is not None and rotary is None:
            n = qkv.shape[0]
            q3 = qkv[:, : nh * hd].unflatten(1, (nh, hd))
            k3 = qkv[:, nh * hd: (nh + nkv) * hd].unflatten(1, (nkv, hd)) if writes else None
            self.position.apply(q3, k3, ctx.positions)
        core.rope_append(
            qkv, ctx.positions,
            rotary.inv_freq if rotary else None, rotary.rotary_dim if rotary else 0,
            nh, nkv if writes else 0, hd,
            ctx.row_entry if writes else None, tables if writes else None,
            cache.k_pool if writes else None, cache.v_pool if writes else None, self.rt.err)
        return self._attend(qkv, ctx, cache, tables)

    def _attend(self, qkv: torch.Tensor, ctx, cache, tables) -> torch.Tensor:
        nh, hd = self.num_heads, self.head_dim
        out = torch.empty((qkv.shape[0], nh * self.v_head_dim), dtype=qkv.dtype, device=qkv.device)
        attn_ops.paged_attention(qkv, cache.k_pool, cache.v_pool, out, ctx, tables, nh,
                                 self.scale, self.window, self.rt, sink=self.sink, keep_first=self.keep_first)
        if self.gate_name:
            g0 = self.qkv.out_features - nh * hd
            core.pointwise(out, qkv[:, g0: g0 + nh * hd], "sigmoid_gate")
        return self.o(out)
