"""A plain, slow implementation of the Bolovik decoder: whole sequences, no cache,
one function per mechanism, float64 unless asked otherwise.  It reads the same
nested configuration dictionary and the same tensor names as the engine, and
shares no code with it.

The decoder: token embedding; layers whose sub-layers read the stream itself and
whose results are normed before they are added (``x <- x + N1(mixer(x))``, then
``x <- x + N2(ff(x))``), N an RMS norm taken over equal consecutive parts of the
vector; after every layer the stream handed on is a learned weighted sum of the
embedding output and of all layers' results so far; mixers are either a gated
delta rule with short causal convolutions or sliding-window attention that also
keeps the first tokens; feed-forwards are gated GELU layers or mixtures of SiLU
experts routed by sigmoid scores inside the best groups of experts.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _t(w, dtype):
    return w.to(dtype)


def part_rms_norm(x: torch.Tensor, weight: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    """x [..., W] cut in ``parts`` equal consecutive pieces; each piece divided by
    sqrt(mean(piece^2) + eps); the whole times ``weight``."""
    shape = x.shape
    p = x.reshape(*shape[:-1], parts, shape[-1] // parts)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(shape) * weight


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension, no weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def depth_mix(results: List[torch.Tensor], coef: torch.Tensor) -> torch.Tensor:
    """sum_j coef[j] * results[j]."""
    out = torch.zeros_like(results[0])
    for j, r in enumerate(results):
        out = out + coef[j] * r
    return out


def causal_conv(x: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps_w [C, taps]; the last column multiplies the current token,
    the one before it the token before, zeros before the sequence."""
    T, C = x.shape
    taps = taps_w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back >= T:
            continue
        out[back:] = out[back:] + x[: T - back] * taps_w[:, j]
    return out


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def delta_rule(q, k, v, beta, g):
    """One head.  q, k [T, dk], v [T, dv], beta, g [T].  Per token:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    out = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.t() @ q[t]
    return out


def delta_mixer(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    dt = h.dtype
    H, dk = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", dk)
    T = h.shape[0]

    def conv_act(name):
        z = h @ _t(W[p + name], dt).t()
        if m.get("conv"):
            z = causal_conv(z, _t(W[p + name + ".conv"], dt))
        return silu(z)

    q, k, v = conv_act("q").reshape(T, G, dk), conv_act("k").reshape(T, G, dk), conv_act("v").reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ _t(W[p + "b"], dt).t())  # [T, H]
    a = h @ _t(W[p + "a"], dt).t() + _t(W[p + "dt_bias"], dt)
    g = torch.exp(-torch.exp(_t(W[p + "A_log"], dt)) * softplus(a))  # [T, H]
    gate = silu(h @ _t(W[p + "g"], dt).t()).reshape(T, H, dv)
    per = H // G
    outs = []
    for hd in range(H):
        o = delta_rule(q[:, hd // per], k[:, hd // per], v[:, hd], beta[:, hd], g[:, hd])
        o = unit_rms(o, eps) * _t(W[p + "norm"], dt)
        outs.append(o * gate[:, hd])
    y = torch.cat(outs, dim=-1)
    return y @ _t(W[p + "o"], dt).t()


def rotary_frequencies(rot: dict) -> List[float]:
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for fi in f:
        wl = 2.0 * math.pi / fi
        if wl < orig / high:
            out.append(fi)
        elif wl > orig / low:
            out.append(fi / factor)
        else:
            s = (orig / wl - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return out


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: List[float]) -> torch.Tensor:
    """x [T, heads, d]; the first 2 * len(freqs) dimensions of each head are
    rotated, dimension i paired with i + len(freqs); the rest pass."""
    half = len(freqs)
    if half == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]  # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half: 2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)


def visible(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention_mixer(h, W, p: str, m: dict, eps: float):
    dt = h.dtype
    H, dk = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", dk)
    T = h.shape[0]
    q = (h @ _t(W[p + "q"], dt).t() + _t(W[p + "q.b"], dt)).reshape(T, H, dk)
    k = (h @ _t(W[p + "k"], dt).t() + _t(W[p + "k.b"], dt)).reshape(T, G, dk)
    v = (h @ _t(W[p + "v"], dt).t() + _t(W[p + "v.b"], dt)).reshape(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        freqs = rotary_frequencies(rot)
        q, k = rotate(q, pos, freqs), rotate(k, pos, freqs)
    q, k, v = unit_rms(q, eps), unit_rms(k, eps), unit_rms(v, eps)
    mask = m.get("mask")
    if mask:
        see = visible(T, int(mask["size"]), int(mask.get("keep_first", 0)))
    else:
        see = visible(T, T + 1, 0)
    per = H // G
    outs = []
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // per].t()) * float(m.get("scale", dk ** -0.5))
        s = s.masked_fill(~see, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, hd // per])
    return torch.cat(outs, dim=-1) @ _t(W[p + "o"], dt).t()


def dense_ff(h, W, p: str):
    dt = h.dtype
    return (gelu_tanh(h @ _t(W[p + "gate"], dt).t()) * (h @ _t(W[p + "up"], dt).t())) @ _t(W[p + "down"], dt).t()


def route(h, router_w, r: dict):
    """Per token: (chosen expert ids, their weights).  Scores are sigmoids of the
    router's logits; expert e is in group e // (E // count); a group is scored by
    its two largest scores added up, and only the ``keep`` best-scored groups stay open; of
    those the ``top`` largest scores are chosen and are the weights as they are."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ router_w.t())  # [T, E]
    groups = r.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups:
        n = int(groups["count"])
        keep = int(groups.get("keep", n))
        per = E // n
        sg = s.reshape(-1, n, per)
        gscore = sg.topk(min(2, per), dim=-1).values.sum(-1)  # [T, n]
        best = gscore.topk(keep, dim=-1).indices
        gm = torch.zeros_like(gscore, dtype=torch.bool)
        gm.scatter_(1, best, True)
        allowed = gm[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    ids = masked.topk(top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def routing_margin(h, router_w, r: dict) -> torch.Tensor:
    """[T]: how far each token's routing is from going another way - the gap between
    the last chosen score and the best one left out among the open groups, and between
    the last open group's score and the best closed one - in units of the scores' spread
    (infinite where nothing is left out).  A small margin means that rounding may choose
    otherwise, with an equally valid result."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ router_w.t())
    T = s.shape[0]
    spread = (s.max(-1).values - s.min(-1).values).clamp_min(1e-9)
    margin = torch.full((T,), float("inf"), dtype=s.dtype)
    groups = r.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups:
        n = int(groups["count"])
        keep = int(groups.get("keep", n))
        per = E // n
        gscore = s.reshape(T, n, per).topk(min(2, per), dim=-1).values.sum(-1)
        order = gscore.sort(dim=-1, descending=True)
        if keep < n:
            margin = torch.minimum(margin, (order.values[:, keep - 1] - order.values[:, keep]) / spread)
        gm = torch.zeros_like(gscore, dtype=torch.bool)
        gm.scatter_(1, order.indices[:, :keep], True)
        allowed = gm[:, :, None].expand(-1, -1, per).reshape(T, E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    order = masked.sort(dim=-1, descending=True).values
    if top < E:
        gap = torch.where(order[:, top] >= 0, (order[:, top - 1] - order[:, top]) / spread,
                          torch.full_like(spread, float("inf")))
        margin = torch.minimum(margin, gap)
    return margin


def moe_ff(h, W, p: str, mlp: dict):
    dt = h.dtype
    ids, wts = route(h, _t(W[p + "router"], dt), mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t].tolist(), wts[t]):
            pe = f"{p}e{e}."
            y = (silu(_t(W[pe + "gate"], dt) @ h[t]) * (_t(W[pe + "up"], dt) @ h[t]))
            out[t] = out[t] + w * (_t(W[pe + "down"], dt) @ y)
    return out


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False,
            margins_out: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence (and, on request, the stream after
    every layer [layers, T, width]); ``margins_out`` collects the routing margins [T]
    of every mixture of experts."""
    eps, parts = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    x = _t(W["embed"], dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    results = [x]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "delta":
            y = delta_mixer(x, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention":
            y = attention_mixer(x, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + part_rms_norm(y, _t(W[p + "norm1"], dtype), parts, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, W, p + "mlp.", mlp)
            if mlp["kind"] != "dense" and margins_out is not None:
                margins_out.append(routing_margin(x, _t(W[p + "mlp.router"], dtype), mlp["router"]))
            x = x + part_rms_norm(y, _t(W[p + "norm2"], dtype), parts, eps)
        results.append(x)
        x = depth_mix(results, _t(W[p + "dwa"], dtype))
        after.append(x)
    logits = part_rms_norm(x, _t(W["final.norm"], dtype), parts, eps) @ _t(W["head"], dtype).t()
    if return_layers:
        return logits, torch.stack(after)
    return logits


def argmax(logits) -> int:
    return int(torch.argmax(logits).item())


def read_config(folder_or_dict) -> dict:
    import json
    import os

    if isinstance(folder_or_dict, dict):
        return folder_or_dict
    with open(os.path.join(folder_or_dict, "config.json")) as fh:
        return json.load(fh)


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    import os

    from safetensors.torch import load_file

    return {k: (v.to(torch.float64) if v.is_floating_point() else v) for k, v in
            load_file(os.path.join(folder, "model.safetensors")).items()}


class Plain:
    """The plain implementation over a model folder, logits cached by sequence."""

    def __init__(self, folder: Optional[str], config: Optional[dict] = None, weights=None):
        self.cfg = read_config(folder if folder is not None else config)
        self.weights = read_weights(folder) if folder is not None else weights
        self._cache: Dict[tuple, torch.Tensor] = {}
        self._margins: Dict[tuple, torch.Tensor] = {}

    def logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._cache:
            margins: list = []
            self._cache[key] = forward(self.cfg, self.weights, list(tokens), margins_out=margins).to(torch.float32)
            self._margins[key] = torch.stack(margins).min(0).values if margins else \
                torch.full((len(key),), float("inf"))
        return self._cache[key]

    def margins(self, tokens) -> torch.Tensor:
        """Per position the smallest routing margin over the layers."""
        self.logits(tokens)
        return self._margins[tuple(tokens)]
