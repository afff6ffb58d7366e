"""Attention through a low-rank latent, over a paged cache of latents.

Per layer, with ``h`` the mixer's input, H heads, per head ``dim`` unrotated and
``rot_dim`` rotated query/key dimensions, value size ``vdim``:

    c_q = rmsnorm(W_dq h) * g_q                  query latent   [q_rank]
    q   = W_uq c_q                               per head [dim | rot_dim]
    (c_raw | r_raw) = W_dkv h                    [kv_rank | rot_dim]
    c   = rmsnorm(c_raw) * g_kv                  key/value latent, cached
    r   = rotate(r_raw, position)                one rotated key part for all heads, cached
    k_h = W_uk,h c      v_h = W_uv,h c
    s_h(i, j) = (q_h,unrot(i) . k_h(j) + rotate(q_h,rot(i)) . r(j)) * scale
    j visible from i when 0 <= i - j < window;  softmax over the visible keys
    out = W_o concat_h(sum_j p_h(i, j) v_h(j))

Only ``c`` and ``r`` are cached: one vector of ``kv_rank + rot_dim`` per token
and layer, whatever the number of heads.  The keys and values are never made:
``q_h,unrot . (W_uk,h c) = (W_uk,h^T q_h,unrot) . c``, so each head's query is
taken into latent space once (a product per head with ``W_uk,h^T``), attention
runs for all heads over the one cached vector per token, whose first
``kv_rank`` elements are also its value, and the weighted sum of latents goes
through ``W_uv,h`` afterwards.  A step's result therefore does not depend on
where a prompt was cut: cached and new tokens are read the same way.

A layer with ``kv_shared`` has no ``W_dkv``: it is scheduled with ``cache_of``
and reads the latents another layer cached, with its own ``W_uk``, ``W_uv``,
queries and window.  The owner's ``cache_window`` must cover every reader's
window: pages are given back by it.

Norms, angles, scores and softmax are 32-bit.  Rotation pairs element i with
i + rotary_dim / 2 of the rotated part; ``rotary_dim`` <= ``rot_dim``.

Without a query latent (``q_rank`` 0 or None) the queries are a projection of
``h`` itself, ``q = W_q h`` (tensor ``q``), made in one product with ``W_dkv h``.
``rotary_pairing: "adjacent"`` rotates neighbours (2i, 2i + 1) instead;
``rotary_scaling`` rescales the frequencies (``rope.rotary_inv_freq``) and, for
"ramp" scaling, multiplies cosine and sine by its magnitude.

Parameters: ``hidden_size``, ``num_heads``, ``dim``, ``rot_dim``, ``vdim``,
``q_rank``, ``kv_rank``, ``scale``, ``window`` (0 = all keys), ``cache_window``
(default: window), ``eps``, ``rotary_dim`` (default rot_dim), ``theta``,
``kv_shared``, ``prefix`` and ``names`` (tensor names behind the prefix for
dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from ..ops import attention as attn_ops
from .base import MIXERS, Mixer, PagedCacheSpec, Runtime, WeightSpec
from .linear import Linear, batched_matmul_nt
from .rope import rotary_inv_freq, rotary_magnitude

_DEFAULT_NAMES = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                  "uk": "uk", "uv": "uv", "o": "o"}


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        g = lambda k: int(params[k])  # noqa: E731
        self.hidden_size, self.num_heads = g("hidden_size"), g("num_heads")
        self.dim, self.rot_dim, self.vdim = g("dim"), g("rot_dim"), g("vdim")
        self.q_rank, self.kv_rank = int(params.get("q_rank") or 0), g("kv_rank")
        self.scale = float(params["scale"])
        self.window = int(params.get("window") or 0)
        self.cache_window = int(params.get("cache_window", self.window) or 0)
        if self.cache_window and (self.window == 0 or self.window > self.cache_window):
            raise ConfigError("latent attention: the cache's window must cover the layer's")
        self.eps = float(params["eps"])
        self.rotary_dim = int(params.get("rotary_dim", self.rot_dim))
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.rot_dim:
            raise ConfigError(f"latent attention: rotary_dim {self.rotary_dim} must be even and within "
                              f"rot_dim {self.rot_dim}")
        self.kv_shared = bool(params.get("kv_shared", False))
        self.prefix = params.get("prefix", "")
        names = {**_DEFAULT_NAMES, **(params.get("names") or {})}
        self.names = {k: self.prefix + v for k, v in names.items()}
        scaling = params.get("rotary_scaling")
        self.adjacent = params.get("rotary_pairing", "half") == "adjacent"
        self.magnitude = rotary_magnitude(scaling)
        freqs = rotary_inv_freq(self.rotary_dim, float(params.get("theta", 10000.0)), scaling) if self.rotary_dim else []
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device) \
            if freqs else None
        self.width = self.kv_rank + self.rot_dim  # of a cached vector and of a query in latent space
        self.down: Optional[Linear] = None
        self.uq: Optional[Linear] = None
        self.o: Optional[Linear] = None

    # ---- declarations -----------------------------------------------------
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(1, self.width, self.cache_window, v_head_dim=0)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H, n = self.num_heads, self.names
        specs = {n["q"]: WeightSpec((H * (self.dim + self.rot_dim), self.hidden_size))} if not self.q_rank else {
            n["dq"]: WeightSpec((self.q_rank, self.hidden_size)),
            n["dq_norm"]: WeightSpec((self.q_rank,), init="norm"),
            n["uq"]: WeightSpec((H * (self.dim + self.rot_dim), self.q_rank)),
        }
        specs.update({
            n["uk"]: WeightSpec((H * self.dim, self.kv_rank)),
            n["uv"]: WeightSpec((H * self.vdim, self.kv_rank)),
            n["o"]: WeightSpec((self.hidden_size, H * self.vdim)),
        })
        if not self.kv_shared:
            specs[n["dkv"]] = WeightSpec((self.kv_rank + self.rot_dim, self.hidden_size))
            specs[n["dkv_norm"]] = WeightSpec((self.kv_rank,), init="norm")
        return specs

    def bind(self, weights) -> None:
        H, n = self.num_heads, self.names
        mats = [weights[n["dq"] if self.q_rank else n["q"]]] + ([] if self.kv_shared else [weights[n["dkv"]]])
        if len({m.dtype for m in mats}) != 1:
            raise ConfigError(f"{self.prefix}: the down projections are stored in different dtypes")
        # both down projections read the same input: one product [dq | c | r]
        self.down = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0], self.rt)
        self.uq = Linear(weights[n["uq"]], self.rt) if self.q_rank else None
        self.o = Linear(weights[n["o"]], self.rt)
        act = self.rt.dtype
        self.q_norm = weights[n["dq_norm"]].to(act).contiguous() if self.q_rank else None
        self.kv_norm = None if self.kv_shared else weights[n["dkv_norm"]].to(act).contiguous()
        # per head: W_uk,h^T [kv_rank, dim] takes a query into latent space, W_uv,h [vdim, kv_rank] a
        # weighted sum of latents to the head's output
        self.uk_t = weights[n["uk"]].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = weights[n["uv"]].view(H, self.vdim, self.kv_rank).contiguous()

    def weight_bytes(self) -> int:
        return self.down.nbytes + (self.uq.nbytes if self.uq is not None else 0) + self.o.nbytes \
            + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()

    # ---- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, W, N = self.num_heads, self.width, x.shape[0]
        writes = cache.owner and not self.kv_shared
        if self.kv_shared and cache.owner:
            raise ConfigError("a kv_shared latent attention layer must be scheduled with cache_of")
        tables = ctx.block_tables[cache.group]
        pool = cache.k_pool
        lat = self.down(x)
        if self.q_rank:
            cq = torch.empty((N, self.q_rank), dtype=x.dtype, device=x.device)
            core.latent_prepare(lat, self.q_rank, self.kv_rank, self.rot_dim, self.rotary_dim, self.q_norm,
                                self.kv_norm, self.eps, self.inv_freq, ctx.positions, ctx.row_entry,
                                tables if writes else None, cq, pool if writes else None, self.rt.err,
                                adjacent=self.adjacent, magnitude=self.magnitude)
            q = self.uq(cq)
        else:
            # the product's rows are [ q | c | r ]: the queries are used as they are
            hq = H * (self.dim + self.rot_dim)
            q = lat[:, :hq]
            if writes:
                core.latent_prepare(lat[:, hq:], 0, self.kv_rank, self.rot_dim, self.rotary_dim, None, self.kv_norm,
                                    self.eps, self.inv_freq, ctx.positions, ctx.row_entry, tables, None, pool,
                                    self.rt.err, adjacent=self.adjacent, magnitude=self.magnitude)
        # queries in latent space and the sums of latents are kept head by head ([H, N, .]):
        # the per-head products then read and write plain matrices
        q_abs = torch.empty((H, N, W), dtype=x.dtype, device=x.device)
        core.latent_q_rotate(q, H, self.dim, self.rot_dim, self.rotary_dim, self.inv_freq, ctx.positions,
                             q_abs.transpose(0, 1), self.kv_rank, adjacent=self.adjacent, magnitude=self.magnitude)
        q3 = q.unflatten(1, (H, self.dim + self.rot_dim))
        batched_matmul_nt(q3[:, :, : self.dim].transpose(0, 1), self.uk_t, q_abs[:, :, : self.kv_rank])
        o_lat = torch.empty((H, N, self.kv_rank), dtype=x.dtype, device=x.device)
        attn_ops.latent_attention(q_abs.transpose(0, 1), pool, o_lat.transpose(0, 1), self.kv_rank, ctx, tables,
                                  self.scale, self.window, self.rt)
        o = torch.empty((N, H, self.vdim), dtype=x.dtype, device=x.device)
        batched_matmul_nt(o_lat, self.uv, o.transpose(0, 1))
        return self.o(o.view(N, H * self.vdim))
