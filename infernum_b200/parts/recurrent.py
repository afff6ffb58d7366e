"""Recurrent mixers: a matrix-valued state per head and request, carried from
token to token in the request's state slot (32-bit), so that a prompt may be cut
anywhere and a decoded token goes on from where the prompt ended.

``wkv``: time mixing with a data-dependent decay per key channel.  With ``h'`` the
token before (the request's state for the first row of a step), five mixes
``m_s = h + (h' - h) * mu_s`` feed ``r, k, v`` (heads x dim), the gate
``silu(W_g m_g)`` and the decay ``w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))``.  Per
head ``o_t = (S + diag(u) k_t v_t^T)^T r_t`` and then ``S <- diag(w_t) S + k_t v_t^T``;
``o`` is divided by its root mean square per head, multiplied by ``norm`` and the
gate, and projected by ``W_o``.
Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``eps``, ``prefix``,
``decay_rank`` (None: taken from the checkpoint's ``w1``).
Tensors behind the prefix: ``mu.{r,k,v,g,w}`` [hidden], ``r, k, v, g`` [heads*dim,
hidden], ``w1`` [rank, hidden], ``w2`` [heads*dim, rank], ``w0`` [heads*dim], ``u``
[heads, dim], ``norm`` [heads*dim], ``o`` [hidden, heads*dim].

``ssd``: a selective state space layer with a scalar decay per head.  ``W_in h``
is laid out ``[z: inner | x: inner | B: groups*state | C: groups*state | dt: heads]``
(inner = heads * vdim); x, B and C pass a causal convolution per channel and SiLU;
``dt <- softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``
(``S`` is state x vdim), ``y = S^T C + D x``; ``y * silu(z)`` is RMS-normed in
``norm_groups`` equal parts, multiplied by ``norm`` and projected by ``W_o``.
Parameters: ``hidden_size``, ``num_heads``, ``vdim``, ``state``, ``groups``,
``conv`` (taps), ``norm_groups``, ``eps``, ``prefix``.
Tensors: ``in`` [2 inner + 2 groups state + heads, hidden], ``conv`` [channels,
taps], ``conv.b``, ``dt_bias``, ``A_log``, ``D`` [heads], ``norm`` [inner], ``o``
[hidden, inner].

``delta``: a gated delta rule.  ``q = W_q h`` and ``k = W_k h`` (kv_heads x dim), ``v =
W_v h`` (heads x vdim); value head a uses key head ``a // (heads / kv_heads)``.  Each of
q, k, v passes a causal convolution per channel (no bias) and SiLU; q and k are then
scaled to unit length per head (``x / sqrt(sum x^2 + 1e-6)``), q also by ``dim ** -0.5``.
``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` per head.
Per head ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q`` (``S`` is
dim x vdim); ``o`` is divided by its root mean square per head, multiplied by ``norm``
(vdim values shared by the heads) and by ``silu(W_g h)``, and projected by ``W_o``.
Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``vdim``,
``conv`` (taps; 0 or None: no convolution), ``eps``, ``prefix``.
Tensors: ``q, k`` [kv_heads*dim, hidden], ``v, g`` [heads*vdim, hidden], ``b, a`` [heads,
hidden], ``q.conv, k.conv, v.conv`` [channels, taps], ``A_log, dt_bias`` [heads], ``norm``
[vdim], ``o`` [hidden, heads*vdim].

The state tensor of a slot is flat float32: the heads' matrices, then what the
shift or the convolution needs of earlier tokens.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from ..ops import scan as scan_ops
from .base import MIXERS, Mixer, Runtime, StateSpec, WeightSpec
from .linear import Linear


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


@MIXERS.register("wkv")
class WkvMixer(Mixer):
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["head_dim"])
        self.eps = float(params["eps"])
        self.prefix = params.get("prefix", "")
        rank = params.get("decay_rank")
        self.decay_rank = int(rank) if rank else None
        self.hk = self.heads * self.dim
        if self.dim > scan_ops.MAX_ROWS:
            raise ConfigError(f"wkv: a head of {self.dim} channels is beyond {scan_ops.MAX_ROWS}")
        self.state_floats = self.heads * self.dim * self.dim
        self.off_prev = self.state_floats  # the token before, behind the heads' matrices

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats + self.hidden_size,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        p, D, HK = self.prefix, self.hidden_size, self.hk
        rank = self.decay_rank if self.decay_rank else -1
        draw = self.decay_rank or max(8, min(64, D // 16))
        specs = {p + "mu." + s: WeightSpec((D,), init="normal", std=0.3) for s in self.MIXES}
        for s in ("r", "k", "v", "g"):
            specs[p + s] = WeightSpec((HK, D))
        specs[p + "w1"] = WeightSpec((rank, D), draw_shape=(draw, D))
        specs[p + "w2"] = WeightSpec((HK, rank), draw_shape=(HK, draw))
        specs[p + "w0"] = WeightSpec((HK,), init="normal", std=0.5)
        specs[p + "u"] = WeightSpec((self.heads, self.dim), init="normal", std=0.3)
        specs[p + "norm"] = WeightSpec((HK,), init="norm")
        specs[p + "o"] = WeightSpec((D, HK))
        return specs

    def bind(self, weights) -> None:
        p = self.prefix
        self.mu = _f32(torch.stack([weights[p + "mu." + s] for s in self.MIXES]))
        self.proj = {s: Linear(weights[p + s], self.rt) for s in ("r", "k", "v", "g", "w1", "w2", "o")}
        if weights[p + "w1"].shape[0] != weights[p + "w2"].shape[1]:
            raise ConfigError(f"{p}: the decay's two matrices do not share a rank")
        self.w0 = _f32(weights[p + "w0"])
        self.u = _f32(weights[p + "u"]).view(-1)
        self.norm = _f32(weights[p + "norm"])

    def weight_bytes(self) -> int:
        return sum(l.nbytes for l in self.proj.values())

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, D = x.shape
        state = cache.state
        mixes = torch.empty((len(self.MIXES), N, D), dtype=x.dtype, device=x.device)
        core.token_shift(x, self.mu, state, self.off_prev, ctx, mixes)
        r = self.proj["r"](mixes[0])
        k = self.proj["k"](mixes[1])
        v = self.proj["v"](mixes[2])
        g = self.proj["g"](mixes[3])
        lw = self.proj["w1"](mixes[4])
        core.pointwise(lw, None, "tanh")
        z = self.proj["w2"](lw, out_dtype=torch.float32)
        o = torch.empty((N, self.hk), dtype=torch.float32, device=x.device)
        scan_ops.wkv_scan(r, k, v, z, self.w0, self.u, state, 0, ctx, o, self.heads, self.rt)
        y = torch.empty((N, self.hk), dtype=x.dtype, device=x.device)
        core.head_norm_gate(o, g, self.norm, self.heads, self.eps, y)
        return self.proj["o"](y)


@MIXERS.register("ssd")
class SsdMixer(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.vdim = int(params["vdim"])
        self.state_rows = int(params["state"])
        self.groups = int(params.get("groups", 1))
        self.taps = int(params["conv"])
        self.norm_groups = int(params.get("norm_groups", 1))
        self.eps = float(params["eps"])
        self.prefix = params.get("prefix", "")
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.state_rows
        self.in_rows = 2 * self.inner + 2 * self.groups * self.state_rows + self.heads
        if self.heads % self.groups:
            raise ConfigError(f"ssd: {self.heads} heads are not a multiple of {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ConfigError(f"ssd: {self.inner} channels do not split in {self.norm_groups} norm groups")
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"ssd: a convolution of {self.taps} taps is outside 1..16")
        if self.state_rows > scan_ops.MAX_ROWS:
            raise ConfigError(f"ssd: a state of {self.state_rows} rows is beyond {scan_ops.MAX_ROWS}")
        self.state_floats = self.heads * self.state_rows * self.vdim
        self.off_conv = self.state_floats  # the convolution's last taps-1 inputs, behind the matrices

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats + max(self.taps - 1, 1) * self.channels,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        p, D = self.prefix, self.hidden_size
        return {
            p + "in": WeightSpec((self.in_rows, D)),
            p + "conv": WeightSpec((self.channels, self.taps), init="normal", std=0.3),
            p + "conv.b": WeightSpec((self.channels,), init="normal", std=0.1),
            p + "dt_bias": WeightSpec((self.heads,), init="normal", std=0.5),
            p + "A_log": WeightSpec((self.heads,), init="normal", std=0.5),
            p + "D": WeightSpec((self.heads,), init="norm"),
            p + "norm": WeightSpec((self.inner,), init="norm"),
            p + "o": WeightSpec((D, self.inner)),
        }

    def bind(self, weights) -> None:
        p = self.prefix
        self.w_in = Linear(weights[p + "in"], self.rt)
        self.w_o = Linear(weights[p + "o"], self.rt)
        self.conv_w = _f32(weights[p + "conv"])
        self.conv_b = _f32(weights[p + "conv.b"])
        self.dt_bias = _f32(weights[p + "dt_bias"])
        self.a_log = _f32(weights[p + "A_log"])
        self.d_skip = _f32(weights[p + "D"])
        self.norm = _f32(weights[p + "norm"])

    def weight_bytes(self) -> int:
        return self.w_in.nbytes + self.w_o.nbytes

    def forward(self, x: torch.Tensor, ctx, cache, projected: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``projected``: ``W_in x`` when the caller has already made it (as part
        of a wider product); a view of wider rows is fine."""
        N = x.shape[0]
        state = cache.state
        zx = projected if projected is not None else self.w_in(x)
        z = zx[:, : self.inner]
        xbc_raw = zx[:, self.inner: self.inner + self.channels]
        dt = zx[:, self.inner + self.channels:]
        y = torch.empty((N, self.inner), dtype=torch.float32, device=x.device)
        # (the convolution runs in the pass that prepares the scan's inputs: its result stays 32-bit)
        scan_ops.ssd_scan(xbc_raw, dt, self.dt_bias, self.a_log, self.d_skip, state, 0, ctx, y, self.heads, self.groups,
                          self.state_rows, self.vdim, self.rt, conv=(self.conv_w, self.conv_b, self.off_conv))
        out = torch.empty((N, self.inner), dtype=x.dtype, device=x.device)
        core.gated_group_norm(y, z, self.norm, self.norm_groups, self.eps, out)
        return self.w_o(out)


@MIXERS.register("delta")
class DeltaMixer(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.kv_heads = int(params.get("num_kv_heads") or self.heads)
        self.dim = int(params["head_dim"])
        self.vdim = int(params.get("vdim") or self.dim)
        self.taps = int(params.get("conv") or 0)
        self.eps = float(params["eps"])
        self.prefix = params.get("prefix", "")
        if self.heads % self.kv_heads:
            raise ConfigError(f"delta: {self.heads} heads are not a multiple of {self.kv_heads} key heads")
        if self.dim > scan_ops.MAX_ROWS:
            raise ConfigError(f"delta: a key of {self.dim} channels is beyond {scan_ops.MAX_ROWS}")
        if not 0 <= self.taps <= 16:
            raise ConfigError(f"delta: a convolution of {self.taps} taps is outside 0..16")
        self.qk = self.kv_heads * self.dim
        self.inner = self.heads * self.vdim
        self.channels = 2 * self.qk + self.inner  # q | k | v: what the convolution runs over
        # rows of the one input product: q | k | v | gate | b | a
        self.off_gate = self.channels
        self.off_b = self.channels + self.inner
        self.off_a = self.off_b + self.heads
        self.in_rows = self.off_a + self.heads
        self.state_floats = self.heads * self.dim * self.vdim
        self.off_conv = self.state_floats  # the convolution's last taps-1 inputs, behind the matrices

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats + max(self.taps - 1, 1) * self.channels,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        p, D = self.prefix, self.hidden_size
        specs = {
            p + "q": WeightSpec((self.qk, D)), p + "k": WeightSpec((self.qk, D)), p + "v": WeightSpec((self.inner, D)),
            p + "g": WeightSpec((self.inner, D)), p + "b": WeightSpec((self.heads, D)),
            p + "a": WeightSpec((self.heads, D)),
            p + "A_log": WeightSpec((self.heads,), init="normal", std=0.5),
            p + "dt_bias": WeightSpec((self.heads,), init="normal", std=0.5),
            p + "norm": WeightSpec((self.vdim,), init="norm"),
            p + "o": WeightSpec((D, self.inner)),
        }
        if self.taps:
            for name, rows in (("q", self.qk), ("k", self.qk), ("v", self.inner)):
                specs[p + name + ".conv"] = WeightSpec((rows, self.taps), init="normal", std=0.4)
        return specs

    def bind(self, weights) -> None:
        p = self.prefix
        mats = [weights[p + n] for n in ("q", "k", "v", "g", "b", "a")]
        if len({m.dtype for m in mats}) != 1:
            raise ConfigError(f"{p}: the input projections are stored in different dtypes")
        self.w_in = Linear(torch.cat(mats, dim=0), self.rt)
        self.w_o = Linear(weights[p + "o"], self.rt)
        self.conv_w = _f32(torch.cat([weights[p + n + ".conv"] for n in ("q", "k", "v")], dim=0)) if self.taps else None
        self.a_log = _f32(weights[p + "A_log"])
        self.dt_bias = _f32(weights[p + "dt_bias"])
        self.norm = _f32(weights[p + "norm"]).repeat(self.heads)  # the heads share one weight

    def weight_bytes(self) -> int:
        return self.w_in.nbytes + self.w_o.nbytes

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N = x.shape[0]
        proj = self.w_in(x)
        o = torch.empty((N, self.inner), dtype=torch.float32, device=x.device)
        scan_ops.delta_scan(proj, 0, self.off_b, self.off_a, self.conv_w, self.a_log, self.dt_bias, cache.state, 0,
                            self.off_conv, ctx, o, self.heads, self.kv_heads, self.dim, self.vdim, self.rt)
        y = torch.empty((N, self.inner), dtype=x.dtype, device=x.device)
        core.head_norm_gate(o, proj[:, self.off_gate: self.off_gate + self.inner], self.norm, self.heads, self.eps, y)
        return self.w_o(y)
