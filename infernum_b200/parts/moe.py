"""Mixture of experts: ``experts`` small gated feed-forwards without biases, of
which each token uses the ``top`` with the largest router logits,
``z = W_r x + b_r`` in 32-bit; the chosen experts' weights are the softmax over
the chosen logits only, and the output is the weighted sum of their outputs,
``sum_k w_k Wd_k (act(Wg_k x) * (Wu_k x))``.

How it runs: routing stays on the device (``moe_route``: ids and weights per
token, and the dense row ``gate[N, experts]`` that is 0 for experts not chosen),
so a recorded step replays.  The experts' gate/up weights are kept as one
stacked matrix ``[experts * 2 ff, hidden]`` and their down weights side by side
as ``[hidden, experts * ff]``; one product gives every expert's gate and up
values, the activation kernel multiplies each expert's run of ``ff`` outputs by
the token's weight for that expert (0 where it was not chosen), and the down
product sums over all experts at once: ``sum_e Wd_e (w_e a_e)`` is one product
with the concatenated vector.  Every expert is computed for every token; what
a token did not choose is multiplied by an exact 0.

Parameters: ``hidden_size``, ``expert_size`` (ff), ``experts``, ``top``,
``activation`` ("silu" | "gelu_tanh"), ``prefix``, ``expert_names`` (format of
an expert's tensors behind the prefix, default "e{e}.{w}" with w in gate, up,
down), ``router`` and ``router_bias`` (names behind the prefix; bias None for
none); ``scoring``: "softmax_top" (default, as above) or "sigmoid": the scores
are ``sigmoid(z)``, the ``top`` largest are chosen and are the weights as they
are (``renormalize``: divided by their sum); with ``groups`` ({"count", "keep",
"top": 2}) expert e belongs to group ``e // (experts // count)``, a group is
scored by the sum of the ``top`` largest scores in it, and the experts outside
the ``keep`` best-scored groups are struck out before the choice;
"softmax_all": the router has ``experts + identity`` outputs, the scores are the
softmax over all of them, the ``top`` largest ``score + correction`` (a tensor,
name in ``correction``, or None) are chosen, and their weights are the scores
without the correction over the chosen ones' sum (+ 1e-20); the last
``identity`` outputs have no expert and no tensors: choosing one adds the
weight times the token's input.  ``shared`` ({"size", "prefix", "gate"}): one more
gated feed-forward that every token uses, added times ``sigmoid(w_gate . x)``
(one number per token; ``gate`` names the [1, hidden] tensor behind the shared
expert's prefix, None: no gate).  When its width is a multiple of an expert's, it
runs as further columns of the experts' two products, its gate in the dense row
of weights; otherwise as a feed-forward of its own.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import FEED_FORWARDS, FeedForward, Runtime, WeightSpec
from .linear import Linear


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.expert_size = int(params["expert_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        if not 0 < self.top <= self.experts + int(params.get("identity") or 0):
            raise ConfigError(f"mixture of experts: top {self.top} must be within 1..{self.experts} (+ the outputs "
                              f"without an expert)")
        self.activation = params.get("activation", "silu")
        if self.activation not in core.ACTIVATIONS:
            raise ConfigError(f"mixture of experts: unknown activation {self.activation!r}")
        self.prefix = params.get("prefix", "")
        self.expert_names = params.get("expert_names", "e{e}.{w}")
        self.router_name = self.prefix + params.get("router", "router")
        bias = params.get("router_bias", "router.b")
        self.bias_name = self.prefix + bias if bias else None
        self.scoring = params.get("scoring", "softmax_top")
        if self.scoring not in ("softmax_top", "sigmoid", "softmax_all"):
            raise ConfigError(f"mixture of experts: unknown scoring {self.scoring!r} (softmax_top, sigmoid, "
                              f"softmax_all)")
        self.identity = int(params.get("identity") or 0)
        corr = params.get("correction")
        self.correction_name = self.prefix + corr if corr else None
        shared = params.get("shared")
        self.shared = None
        if shared:
            self.shared = {"size": int(shared["size"]), "prefix": self.prefix + shared.get("prefix", "shared."),
                           "gate": shared.get("gate")}
        if (self.identity or self.correction_name or self.shared) and self.scoring != "softmax_all":
            raise ConfigError("mixture of experts: outputs without an expert, a correction of the choice and an "
                              "expert for every token go with softmax_all scoring")
        self.renormalize = bool(params.get("renormalize", False))
        groups = params.get("groups") or {}
        self.group_count = int(groups.get("count", 1))
        self.group_keep = int(groups.get("keep", self.group_count))
        self.group_top = int(groups.get("top", 2))
        if self.group_count > 1:
            if self.scoring != "sigmoid":
                raise ConfigError("mixture of experts: groups of experts go with sigmoid scoring")
            if self.experts % self.group_count or not 0 < self.group_keep <= self.group_count \
                    or self.group_keep * (self.experts // self.group_count) < self.top:
                raise ConfigError(f"mixture of experts: {self.experts} experts in {self.group_count} groups of which "
                                  f"{self.group_keep} stay open cannot give {self.top} choices")
            if self.experts // self.group_count > 64:
                raise ConfigError("mixture of experts: a group of more than 64 experts is beyond the routing kernel")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.router: Optional[torch.Tensor] = None
        self.router_bias: Optional[torch.Tensor] = None

    def _name(self, e: int, w: str) -> str:
        return self.prefix + self.expert_names.format(e=e, w=w)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, f = self.hidden_size, self.expert_size
        specs = {self.router_name: WeightSpec((self.experts + self.identity, h), std=0.5)}
        if self.bias_name:
            specs[self.bias_name] = WeightSpec((self.experts,), std=0.5)
        if self.correction_name:
            specs[self.correction_name] = WeightSpec((self.experts + self.identity,), std=0.02)
        if self.shared:
            sp, sf = self.shared["prefix"], self.shared["size"]
            specs[sp + "gate"], specs[sp + "up"], specs[sp + "down"] = WeightSpec((sf, h)), WeightSpec((sf, h)), \
                WeightSpec((h, sf))
            if self.shared["gate"]:
                specs[sp + self.shared["gate"]] = WeightSpec((1, h), std=0.3)
        for e in range(self.experts):
            specs[self._name(e, "gate")] = WeightSpec((f, h))
            specs[self._name(e, "up")] = WeightSpec((f, h))
            specs[self._name(e, "down")] = WeightSpec((h, f))
        return specs

    def bind(self, weights) -> None:
        E, f, h = self.experts, self.expert_size, self.hidden_size
        gates = [weights[self._name(e, "gate")] for e in range(E)]
        ups = [weights[self._name(e, "up")] for e in range(E)]
        downs = [weights[self._name(e, "down")] for e in range(E)]
        if len({t.dtype for t in gates + ups + downs}) != 1:
            raise ConfigError(f"{self.prefix}: the experts are stored in different dtypes")
        # one gated feed-forward of width E * ff: expert e owns outputs [e ff, (e + 1) ff); an expert that
        # every token uses, of k times an expert's width, is k more runs of columns behind them
        self.shared_runs = 0
        if self.shared and self.shared["size"] % f == 0:
            sp = self.shared["prefix"]
            extra = [weights[sp + "gate"], weights[sp + "up"], weights[sp + "down"]]
            if {t.dtype for t in extra} == {gates[0].dtype}:
                self.shared_runs = self.shared["size"] // f
                gates.append(extra[0])
                ups.append(extra[1])
                downs.append(extra[2])
        gate, up = torch.cat(gates, dim=0), torch.cat(ups, dim=0)
        I = (E + self.shared_runs) * f
        self.block = None
        if I % 64 == 0:
            fused = torch.stack([gate.view(I // 64, 64, h), up.view(I // 64, 64, h)], dim=1).reshape(2 * I, h)
            self.block = 64
        else:
            fused = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(fused, self.rt)
        self.down = Linear(torch.cat(downs, dim=1), self.rt)
        # the router is 32-bit arithmetic whatever the engine's dtype
        self.router = weights[self.router_name].contiguous()
        self.router_bias = weights[self.bias_name].to(torch.float32).contiguous() if self.bias_name else None
        self.correction = weights[self.correction_name].to(torch.float32).contiguous() if self.correction_name else None
        self.shared_ffn = None
        if self.shared:
            from .mlp import SwiGLU

            sp = self.shared["prefix"]
            if not self.shared_runs:
                self.shared_ffn = SwiGLU({"hidden_size": h, "intermediate_size": self.shared["size"], "prefix": sp,
                                          "names": {"gate": "gate", "up": "up", "down": "down"},
                                          "activation": self.activation}, self.rt)
                self.shared_ffn.bind(weights)
            if self.shared["gate"]:
                # the gate's logit is one more row of the router's product
                self.router = torch.cat([self.router, weights[sp + self.shared["gate"]].to(self.router.dtype)],
                                        dim=0).contiguous()

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes + self.router.numel() * self.router.element_size() \
            + (self.shared_ffn.weight_bytes() if self.shared_ffn is not None else 0)

    def route(self, x: torch.Tensor):
        """(ids [N, top] int32, weights [N, top] float32, gate [N, experts] float32)."""
        n, dev = x.shape[0], x.device
        logits = torch.empty((n, self.router.shape[0]), dtype=torch.float32, device=dev)
        core.router_logits(x, self.router, logits)  # 32-bit multiply-adds, a fixed order per row
        ids = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        gate = torch.empty((n, self.experts + getattr(self, "shared_runs", 0)), dtype=torch.float32, device=dev)
        if self.scoring == "softmax_all":
            self._extra = torch.empty((n, 2), dtype=torch.float32, device=dev)
            core.moe_route_softmax_all(logits, self.correction, self.experts + self.identity, self.experts, self.top,
                                       ids, wts, gate, self._extra)
        elif self.scoring == "sigmoid":
            core.moe_route_scored(logits, self.router_bias, self.top, ids, wts, gate, groups=self.group_count,
                                  keep=self.group_keep, group_top=self.group_top, renorm=self.renormalize)
        else:
            core.moe_route(logits, self.router_bias, self.top, ids, wts, gate)
        return ids, wts, gate

    def forward(self, x: torch.Tensor, ctx=None) -> torch.Tensor:
        _ids, _wts, gate = self.route(x)
        act = torch.empty((x.shape[0], gate.shape[1] * self.expert_size), dtype=x.dtype, device=x.device)
        fused = False
        if self.block == 64 and x.dtype == torch.bfloat16 and self.gate_up.weight.dtype == torch.bfloat16:
            from ..ops import gemm_tc

            # prompts: activation and the router's weights in the product's epilogue
            fused = gemm_tc.swiglu_route(x, self.gate_up.weight, act, self.gate_up.err, activation=self.activation,
                                         scale=gate, cols_per_scale=self.expert_size)
        if not fused:
            core.gated_act(self.gate_up(x), act, self.activation, block=self.block, scale=gate,
                           cols_per_scale=self.expert_size)
        routed = self.down(act)
        if self.scoring != "softmax_all" or not (self.identity or self.shared_ffn is not None):
            return routed  # (an expert for every token that ran as columns of the products is in there)
        # the input handed on by the outputs without an expert, and the expert that every token uses
        shared = self.shared_ffn.forward(x, ctx) if self.shared_ffn is not None else None
        out = torch.empty_like(routed)
        core.moe_combine(routed, x, shared, self._extra, out)
        return out
