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
the ``keep`` best-scored groups are struck out before the choice.
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
        if not 0 < self.top <= self.experts:
            raise ConfigError(f"mixture of experts: top {self.top} must be within 1..{self.experts}")
        self.activation = params.get("activation", "silu")
        if self.activation not in core.ACTIVATIONS:
            raise ConfigError(f"mixture of experts: unknown activation {self.activation!r}")
        self.prefix = params.get("prefix", "")
        self.expert_names = params.get("expert_names", "e{e}.{w}")
        self.router_name = self.prefix + params.get("router", "router")
        bias = params.get("router_bias", "router.b")
        self.bias_name = self.prefix + bias if bias else None
        self.scoring = params.get("scoring", "softmax_top")
        if self.scoring not in ("softmax_top", "sigmoid"):
            raise ConfigError(f"mixture of experts: unknown scoring {self.scoring!r} (softmax_top, sigmoid)")
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
        specs = {self.router_name: WeightSpec((self.experts, h), std=0.5)}
        if self.bias_name:
            specs[self.bias_name] = WeightSpec((self.experts,), std=0.5)
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
        # one gated feed-forward of width E * ff: expert e owns outputs [e ff, (e + 1) ff)
        gate, up = torch.cat(gates, dim=0), torch.cat(ups, dim=0)
        I = E * f
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

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes + self.router.numel() * self.router.element_size()

    def route(self, x: torch.Tensor):
        """(ids [N, top] int32, weights [N, top] float32, gate [N, experts] float32)."""
        n, dev = x.shape[0], x.device
        logits = torch.empty((n, self.experts), dtype=torch.float32, device=dev)
        core.router_logits(x, self.router, logits)  # 32-bit multiply-adds, a fixed order per row
        ids = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        gate = torch.empty((n, self.experts), dtype=torch.float32, device=dev)
        if self.scoring == "sigmoid":
            core.moe_route_scored(logits, self.router_bias, self.top, ids, wts, gate, groups=self.group_count,
                                  keep=self.group_keep, group_top=self.group_top, renorm=self.renormalize)
        else:
            core.moe_route(logits, self.router_bias, self.top, ids, wts, gate)
        return ids, wts, gate

    def forward(self, x: torch.Tensor, ctx=None) -> torch.Tensor:
        _ids, _wts, gate = self.route(x)
        act = torch.empty((x.shape[0], self.experts * self.expert_size), dtype=x.dtype, device=x.device)
        fused = False
        if self.block == 64 and x.dtype == torch.bfloat16 and self.gate_up.weight.dtype == torch.bfloat16:
            from ..ops import gemm_tc

            # prompts: activation and the router's weights in the product's epilogue
            fused = gemm_tc.swiglu_route(x, self.gate_up.weight, act, self.gate_up.err, activation=self.activation,
                                         scale=gate, cols_per_scale=self.expert_size)
        if not fused:
            core.gated_act(self.gate_up(x), act, self.activation, block=self.block, scale=gate,
                           cols_per_scale=self.expert_size)
        return self.down(act)
