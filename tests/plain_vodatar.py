"""The Vodatar decoder restated plainly: whole sequences, no cache, no batching,
one function per mechanism, float64 unless told otherwise.  It shares no code
with the package; the tests hold the package against it.

Notation: ``x`` [T, width] is one sequence's residual stream, ``W`` tensors are
stored [out, in] and applied as ``x @ W.T``; ``w`` is the dictionary of the
checkpoint's tensors by name, ``cfg`` the dictionary of config.json.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def part_norm(x: torch.Tensor, weight: Optional[torch.Tensor], parts: int, eps: float) -> torch.Tensor:
    """Each of ``parts`` equal consecutive pieces of the last axis divided by its own
    sqrt(mean(piece^2) + eps); then the whole times ``weight`` (None: no weight)."""
    shape = x.shape
    p = x.reshape(*shape[:-1], parts, shape[-1] // parts)
    p = p / torch.sqrt((p * p).mean(dim=-1, keepdim=True) + eps)
    y = p.reshape(shape)
    return y if weight is None else y * weight


def causal_conv(u: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """``y_t = sum_j taps_w[:, j] * u_(t - K + 1 + j)`` per channel, zeros before
    the sequence; ``u`` [T, C], ``taps_w`` [C, K]."""
    T, C = u.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + padded[j: j + T] * taps_w[:, j]
    return y


def rotary_frequencies(rot: Dict) -> (List[float], float):
    """(frequencies of the dims/2 pairs, magnitude that multiplies cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freqs, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], magnitude: float = 1.0) -> torch.Tensor:
    """Rotates the first ``2 len(freqs)`` elements of the last axis, element 2i
    with 2i + 1, by ``position * freqs[i]``; ``x`` [T, ..., d], the rest unchanged."""
    out = x.clone()
    n = len(freqs)
    if n == 0:
        return out
    f = torch.tensor(freqs, dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]  # [T, n]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang) * magnitude, torch.sin(ang) * magnitude
    a, b = x[..., 0: 2 * n: 2], x[..., 1: 2 * n: 2]
    out[..., 0: 2 * n: 2] = a * c - b * s
    out[..., 1: 2 * n: 2] = b * c + a * s
    return out


def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                             softcap: Optional[float] = None) -> torch.Tensor:
    """One head: ``q`` [T, d], ``k`` [T, d], ``v`` [T, e]; position i reads j <= i."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_attention(h: torch.Tensor, m: Dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The ``attention`` mixer: two score maps per head over shared values."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (causal_conv(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    pos = torch.arange(T)
    q = q.reshape(T, H, 2, d)
    k = k.reshape(T, G, 2, d)
    v = v.reshape(T, G, e)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        freqs, mag = rotary_frequencies(rot)
        q, k = rotate_pairs(q, pos, freqs, mag), rotate_pairs(k, pos, freqs, mag)
    lam = math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = causal_softmax_attention(q[:, a, 0], k[:, g, 0], v[:, g], float(m["scale"]), m.get("softcap"))
        a2 = causal_softmax_attention(q[:, a, 1], k[:, g, 1], v[:, g], float(m["scale"]), m.get("softcap"))
        o = a1 - lam * a2
        heads.append(part_norm(o, None, 1, eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, m: Dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The ``latent_attention`` mixer with explicit keys and values per head."""
    T = h.shape[0]
    H, d, r, e, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)
    down = h @ w[p + "dkv"].T
    c = part_norm(down[:, :R], w[p + "dkv.norm"], 1, eps)
    shared = down[:, R:]
    pos = torch.arange(T)
    rot = dict(m["rot"])
    freqs, mag = rotary_frequencies(rot) if int(rot["dims"]) > 0 else ([], 1.0)
    q_rot = rotate_pairs(q[:, :, d:], pos, freqs, mag)
    k_rot = rotate_pairs(shared, pos, freqs, mag)
    keys = (c @ w[p + "uk"].T).reshape(T, H, d)
    vals = (c @ w[p + "uv"].T).reshape(T, H, e)
    heads = []
    for a in range(H):
        qa = torch.cat([q[:, a, :d], q_rot[:, a]], dim=-1)
        ka = torch.cat([keys[:, a], k_rot], dim=-1)
        heads.append(causal_softmax_attention(qa, ka, vals[:, a], float(m["scale"])))
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gated_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, router: Dict, w: Dict[str, torch.Tensor], p: str, margins_out: Optional[list] = None):
    """(ids [T, top], weights [T, top]) over ``experts + identity`` outputs: softmax
    over all of them, the choice by score + correction (lowest index among equals),
    the weights the chosen scores over their sum.  ``margins_out`` collects, per
    token, by how much the last chosen output beat the best one left out."""
    z = h @ w[p + "router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    top = int(router["top"])
    order = torch.sort(choice, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :top]
    if margins_out is not None:
        margins_out.append(order.values[:, top - 1] - order.values[:, top] if top < choice.shape[1]
                           else torch.full((h.shape[0],), float("inf"), dtype=h.dtype))
    chosen = torch.gather(s, 1, ids)
    return ids, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def mixture(h: torch.Tensor, mlp: Dict, w: Dict[str, torch.Tensor], p: str, margins_out: Optional[list] = None) -> torch.Tensor:
    router = mlp["router"]
    E, I = int(router["experts"]), int(router.get("identity", 0))
    ids, wts = route(h, router, w, p, margins_out)
    out = torch.zeros_like(h)
    for e in range(E + I):
        share = (wts * (ids == e)).sum(dim=-1, keepdim=True)  # [T, 1], 0 where the token did not choose e
        if float(share.abs().sum()) == 0.0:
            continue
        # an output without an expert hands its input on
        out = out + share * (h if e >= E else gated_expert(h, w, f"{p}e{e}."))
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)  # [T, 1]
        out = out + gate * gated_expert(h, w, p + "shared.")
    return out


def layer(x: torch.Tensor, spec: Dict, cfg: Dict, w: Dict[str, torch.Tensor], p: str,
          margins_out: Optional[list] = None) -> torch.Tensor:
    eps, parts, mult = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1)), float(cfg.get("residual_mult", 1.0))
    canon = cfg.get("canon") or {}

    def sub(x, n, fn):
        h = part_norm(x, w[f"{p}norm{n}"], parts, eps)
        u = h + causal_conv(h, w[f"{p}canon{n}"]) if canon.get("taps") else h
        y = fn(u)
        if f"{p}rg{n}" in w:
            y = y * torch.sigmoid(h @ w[f"{p}rg{n}"].T + w[f"{p}rg{n}.b"])
        return x + mult * part_norm(y, w[f"{p}norm{n}b"], parts, eps)

    if spec["type"] == "attention":
        x = sub(x, 1, lambda u: differential_attention(u, spec["mixer"], w, p + "mix.", eps))
    else:
        x = sub(x, 1, lambda u: latent_attention(u, spec["mixer"], w, p + "mix.", eps))
    if spec.get("mlp"):
        x = sub(x, 2, lambda u: mixture(u, spec["mlp"], w, p + "mlp.", margins_out))
    return x


def run_order(cfg: Dict):
    """[(layer, pass number or None when the run does not begin a pass)]."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(n):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, L)]


def forward(tokens, cfg: Dict, weights: Dict[str, torch.Tensor], dtype=F, keep_layers: bool = False,
            margins_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence; with ``keep_layers`` also the stream after every run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, parts = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    x = part_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], parts, eps)
    x0 = x
    kept = []
    for i, begins in run_order(cfg):
        if begins is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][begins]
        x = layer(x, cfg["layers"][i], cfg, w, f"l{i}.", margins_out)
        kept.append(x)
    logits = part_norm(x, w["final.norm"], parts, eps) @ w["head"].T
    return (logits, torch.stack(kept)) if keep_layers else logits


def argmax(logits: torch.Tensor) -> int:
    """The lowest index among the largest values."""
    return int((logits == logits.max()).nonzero()[0])


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

    return {k: (v.to(F) if v.is_floating_point() else v) for k, v in
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
            with torch.no_grad():
                self._cache[key] = forward(list(tokens), self.cfg, self.weights, margins_out=margins).to(torch.float32)
            self._margins[key] = torch.stack(margins).min(0).values if margins else \
                torch.full((len(key),), float("inf"))
        return self._cache[key]

    def margins(self, tokens) -> torch.Tensor:
        """Per position the smallest routing margin over all runs of layers."""
        self.logits(tokens)
        return self._margins[tuple(tokens)]
