"""Differential attention over the paged cache: two score maps per head over the
same values.

With ``h`` the mixer's input, H heads, G key/value heads (head a reads key/value
head a // (H / G)), maps of ``dim`` and values of ``vdim``:

    q = W_q h   [H, 2, dim]      k = W_k h   [G, 2, dim]      v = W_v h   [G, vdim]
    q, k, v <- causal convolution per channel over time (``conv`` taps, no bias)
    q_m, k_m <- rotated in their first ``rotary_dim`` dimensions, neighbours paired
    s_m(i, j) = cap * tanh(q_m(i) . k_m(j) * scale / cap)       for j <= i
    o = softmax(s_1) v - lam * softmax(s_2) v
    lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                (one number a layer)
    out = W_o concat_heads(o / sqrt(mean(o^2) + eps) * (1 - diff))

A token's cached key row holds both maps side by side ([pages, G, page_size, 2
dim]), its value row is [pages, G, page_size, vdim]; the last ``conv - 1``
projected rows of a request are the mixer's state.  Scores, softmax, the norm
and the angles are 32-bit.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim``, ``vdim``,
``scale``, ``softcap`` (0: none), ``diff``, ``conv`` (0: none), ``eps``,
``rotary`` (None or {"dims", "theta", "scaling"}), ``prefix``; tensors behind the
prefix: ``q, k, v, o``, ``q.conv, k.conv, v.conv``, ``lq1, lk1, lq2, lk2``.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import attention_diff, core
from .base import MIXERS, Mixer, PagedCacheSpec, Runtime, StateSpec, WeightSpec
from .linear import Linear
from .rope import rotary_inv_freq, rotary_magnitude


@MIXERS.register("diff_attention")
class DiffAttention(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        g = lambda k: int(params[k])  # noqa: E731
        self.hidden_size, self.heads = g("hidden_size"), g("num_heads")
        self.kv_heads = int(params.get("num_kv_heads") or self.heads)
        self.dim = g("dim")
        self.vdim = int(params.get("vdim") or self.dim)
        self.scale = float(params.get("scale") or self.dim ** -0.5)
        self.softcap = float(params.get("softcap") or 0.0)
        self.diff = float(params.get("diff") or 0.0)
        self.taps = int(params.get("conv") or 0)
        self.eps = float(params["eps"])
        self.prefix = params.get("prefix", "")
        if self.heads % self.kv_heads:
            raise ConfigError(f"differential attention: {self.heads} heads are not a multiple of "
                              f"{self.kv_heads} key/value heads")
        if not 0 <= self.taps <= 16:
            raise ConfigError(f"differential attention: a convolution of {self.taps} taps is outside 0..16")
        if self.vdim > 512:
            raise ConfigError(f"differential attention: values of {self.vdim} are beyond 512")
        rot = params.get("rotary") or {}
        self.rotary_dim = int(rot.get("dims") or 0)
        if self.rotary_dim % 2 or self.rotary_dim > self.dim or (self.rotary_dim and self.dim % 2):
            raise ConfigError(f"differential attention: {self.rotary_dim} rotated dimensions must be even and "
                              f"within an even map size, not {self.dim}")
        self.magnitude = rotary_magnitude(rot.get("scaling"))
        self.inv_freq = None
        if self.rotary_dim:
            freqs = rotary_inv_freq(self.rotary_dim, float(rot.get("theta", 10000.0)), rot.get("scaling"))
            self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.q_cols = self.heads * 2 * self.dim
        self.channels = self.q_cols + self.kv_heads * (2 * self.dim + self.vdim)
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.conv_w: Optional[torch.Tensor] = None
        self.lam = 0.0

    # ---- declarations -----------------------------------------------------
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(self.kv_heads, 2 * self.dim, 0, v_head_dim=self.vdim)

    def state_spec(self) -> Optional[StateSpec]:
        if self.taps <= 1:
            return None
        return StateSpec(((self.taps - 1) * self.channels,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        p, D = self.prefix, self.hidden_size
        kc, vc = self.kv_heads * 2 * self.dim, self.kv_heads * self.vdim
        specs = {p + "q": WeightSpec((self.q_cols, D)), p + "k": WeightSpec((kc, D)), p + "v": WeightSpec((vc, D)),
                 p + "o": WeightSpec((D, self.heads * self.vdim))}
        if self.taps:
            for name, rows in (("q", self.q_cols), ("k", kc), ("v", vc)):
                specs[p + name + ".conv"] = WeightSpec((rows, self.taps), init="normal", std=0.4)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[p + name] = WeightSpec((self.dim,), init="normal", std=0.1)
        return specs

    def bind(self, weights) -> None:
        p = self.prefix
        mats = [weights[p + n] for n in ("q", "k", "v")]
        if len({m.dtype for m in mats}) != 1:
            raise ConfigError(f"{p}: q/k/v projections are stored in different dtypes")
        self.qkv = Linear(torch.cat(mats, dim=0), self.rt)
        self.o = Linear(weights[p + "o"], self.rt)
        if self.taps:
            self.conv_w = torch.cat([weights[p + n + ".conv"] for n in ("q", "k", "v")], dim=0) \
                .to(torch.float32).contiguous()
        l = {n: weights[p + n].to(torch.float64).cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((l["lq1"] * l["lk1"]).sum())) - math.exp(float((l["lq2"] * l["lk2"]).sum())) \
            + self.diff

    def weight_bytes(self) -> int:
        return self.qkv.nbytes + self.o.nbytes

    # ---- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if not cache.owner:
            raise ConfigError("differential attention must own its cache")
        N = x.shape[0]
        tables = ctx.block_tables[cache.group]
        proj = self.qkv(x)
        q = torch.empty((N, self.q_cols), dtype=x.dtype, device=x.device)
        core.conv_rope_append(proj, self.conv_w, cache.state, 0, self.inv_freq, self.rotary_dim, self.magnitude,
                              self.heads, self.kv_heads, self.dim, self.vdim, ctx, tables, q, cache.k_pool,
                              cache.v_pool, self.rt.err)
        if self.taps > 1:
            core.conv_state_update(proj, self.taps, cache.state, 0, ctx)
        out = torch.empty((N, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        # bfloat16 with sizes that have a variant: the tensor-core kernel; everything else the plain 32-bit one
        if not attention_diff.run(q, cache.k_pool, cache.v_pool, out, ctx, tables, self.heads, self.scale, self.softcap,
                                  self.lam, self.eps, 1.0 - self.diff, self.rt):
            core.attention_diff(q, cache.k_pool, cache.v_pool, out, ctx, tables, self.heads, self.scale, self.softcap,
                                self.lam, self.eps, 1.0 - self.diff, self.rt.err)
        return self.o(out)
