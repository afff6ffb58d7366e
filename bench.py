#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decoded tokens per second at the
Llama-3.1-8B layer sizes with random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

A "step" is one decode step of the whole batch.  The default run: batch 8,
prompts of 1,024 tokens, K timed decode steps after W untimed ones.  One JSON
line is printed:

  value      decoded tokens per second, timed on the device with CUDA events
             around K steps whose inputs stay on the device
  e2e        the same through the Python entry point (``Engine``): host tokens
             in (pinned memory, copied every step) and host tokens out
  prefill    one step over a 2,048-token prompt: tokens/s, time, and the
             fraction of the measured bf16 matmul peak its flops reach
  roofline   bytes a decode step must read (every weight once, the cache of
             the live requests) / its time, against the measured copy bandwidth
  points     decode tokens/s at batch 1 and at batch 64 (1,024-token prompts), and
             at batch 8 near the end of an 8,192-token context; and two runs
             through the scheduler at other layer sizes, each with a model of its
             own made after the headline runs: the Llama-3.2-1B sizes under a
             mixed workload (64 requests, prompts of 16 to 4,096 tokens fed 512
             at a time beside decoding requests, temperature 0.8), and the
             Llama-2-13B sizes with a page pool of 0.8 of the need, so that
             requests are preempted and recomputed (``pressure_13b_*``; some of
             them, the preempted ones first, are run again alone and compared)

Weights (15 GB) and cache are far larger than the 126 MB L2, so every timed
step streams its inputs from HBM; no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_8B = {
    "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        rows = [l for t, l in self.samples if t0 <= t <= t1] or [l for _, l in self.samples[-3:]]
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            parts = [x.strip() for x in l.split(",")]
            try:
                mhz.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def decode_bytes(model, cache, live_tokens: int, batch: int = 0) -> int:
    """Bytes one decode step has to move: every weight it uses once, the keys and
    values of the live requests (inside their windows), and the requests' fixed-size
    state, read and written."""
    per_token = 0
    el = 2 if model.rt.dtype != __import__("torch").float32 else 4
    per_request = live_tokens / max(batch, 1)
    for g in cache.groups:
        seen = min(per_request, g.spec.window) if g.spec.window > 0 and batch else per_request
        per_token += g.spec.elements_per_token() * el * len(g.positions) * (seen / per_request if per_request else 1)
    return int(model.step_weight_bytes() + per_token * live_tokens + 2 * batch * cache.state_bytes_per_request())


def prefill_flops(cfg: dict, T: int, layers: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2.0 * T * H * ((nh + 2 * nkv) * hd) + 2.0 * T * (nh * hd) * H + 2.0 * T * H * 2 * I + 2.0 * T * I * H
    attn = 2.0 * 2.0 * nh * hd * T * (T + 1) / 2.0  # causal: QK^T and PV
    return layers * (linear + attn) + 2.0 * 1 * H * V


def make_requests(runner, cache, batch, prompt_len, vocab, seed, chunk=2048):
    """Admits ``batch`` requests and runs their prompts through the step
    function in portions of at most ``chunk`` tokens.  Returns the caches and
    the first token selected for each."""
    import torch

    from infernum_b200.engine.step import StepEntry
    from infernum_b200.ops import core

    g = torch.Generator().manual_seed(seed)
    caches, first = [], []
    for b in range(batch):
        rc = cache.admit(("bench", seed, b))
        prompt = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        pos, logits = 0, None
        while pos < prompt_len:
            n = min(chunk, prompt_len - pos)
            logits = runner.step([StepEntry(rc, prompt[pos: pos + n], [n - 1] if pos + n == prompt_len else [])])
            pos += n
        out = torch.empty(1, dtype=torch.int32, device=logits.device)
        core.argmax(logits, out)
        caches.append(rc)
        first.append(int(out.item()))
    return caches, first


def time_decode(model, batch, prompt_len, steps, warmup, page_size, seed, clocks=None, graph=True):
    """Device-timed decode: K steps of a DecodeRunner that feeds itself."""
    import torch

    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner
    from infernum_b200.ops import core

    total = prompt_len + steps + warmup + 8
    pages = batch * (-(-total // page_size)) + 8
    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=pages, max_requests=batch,
                         dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=4096, max_entries=max(batch, 1))
    caches, first = make_requests(runner, cache, batch, prompt_len, model.spec.vocab_size, seed)
    session = DecodeRunner(runner, total + 8, use_graph=graph)
    session.pin(caches, first, steps + max(warmup, 3) + 2)
    for _ in range(max(warmup, 3)):
        session.step_pinned()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = core.LAUNCHES
    t0 = time.time()
    start.record()
    for _ in range(steps):
        session.step_pinned()
    end.record()
    torch.cuda.synchronize()
    t1 = time.time()
    runner.check_errors()
    ms = start.elapsed_time(end) / steps
    live = sum(rc.num_tokens for rc in caches) - batch * steps // 2  # mean over the timed steps
    result = {
        "ms_per_step": ms, "tokens_per_s": batch * 1000.0 / ms,
        "bytes_per_step": decode_bytes(model, cache, live, batch),
        "launches_per_step": session.last.launches_per_step,
        "graph": session.last.graph is not None,
        "clocks": clocks.summary(t0, t1) if clocks else None,
    }
    for rc in caches:
        cache.release(rc)
    del session, runner, cache
    torch.cuda.empty_cache()
    return result


def time_e2e(model, batch, prompt_len, steps, warmup, page_size, seed, launch_ahead=True):
    """The same through ``Engine``: requests are submitted as host token lists,
    every step copies its inputs from pinned memory and reads the selected
    tokens back.  With ``launch_ahead`` (the engine's default) a decode step is
    launched behind the one in flight and takes that one's tokens on the device;
    its positions, lengths and slots still come from the host every step.
    Without it every step is launched after the one before was read and gets
    its tokens from the host too."""
    import torch

    import infernum_b200 as ib

    total = prompt_len + steps + warmup + 8
    pages = batch * (-(-total // page_size)) + 8
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=batch, max_prefill_tokens=2048,
                                             block_size=page_size, num_blocks=pages,
                                             max_tokens_per_step=2048, max_model_len=total + 8,
                                             launch_ahead=launch_ahead))
    g = torch.Generator().manual_seed(seed)
    opts = ib.GenerateOptions(max_new_tokens=steps + warmup + 6, ignore_eos=True)
    handles = [engine.submit(torch.randint(0, model.spec.vocab_size, (prompt_len,), generator=g).tolist(), opts)
               for _ in range(batch)]
    while any(len(h.seq.generated_ids) < 1 for h in handles):
        engine.step()  # prompts
    for _ in range(max(warmup, 3)):
        engine.step()
    torch.cuda.synchronize()
    before = sum(len(h.seq.generated_ids) for h in handles)
    h2d0, d2h0 = engine.h2d_bytes, engine.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(h.seq.generated_ids) for h in handles) - before
    for h in handles:
        engine.cancel(h)
    engine.step()
    out = {"value": made / dt, "unit": "tokens/s", "ms_per_step": dt * 1000 / steps,
           "h2d_bytes_per_step": (engine.h2d_bytes - h2d0) / steps,
           "d2h_bytes_per_step": (engine.d2h_bytes - d2h0) / steps}
    del engine
    torch.cuda.empty_cache()
    return out


def time_prefill(model, cfg, layers, T, page_size, peaks, reps=3, recorded=False, flops=None):
    """One step over a whole prompt of ``T`` tokens, timed on the device.
    ``recorded``: the way ``Engine`` runs a prompt that comes alone - replayed from
    a recording made for the bucket of its length - with the host's own time for
    the step beside it (a step is bound by the device while that is the smaller)."""
    import torch

    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner, StepEntry

    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=-(-T // page_size) + 2,
                         max_requests=1, dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=T, max_entries=1)
    session = DecodeRunner(runner, T + 8) if recorded else None
    g = torch.Generator().manual_seed(5)
    times, host = [], []
    for i in range(reps + (3 if recorded else 2)):
        prompt = torch.randint(0, model.spec.vocab_size, (T,), generator=g).tolist()
        rc = cache.admit(("prefill", i))
        cache.extend(rc, T)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        if recorded:
            slot = session.prepare([], 0, portions=[(rc, T, True)])
            session.launch(slot, [], [], None, portions=[(rc, prompt, True)])
        else:
            runner.step([StepEntry(rc, prompt, [T - 1])])
        end.record()
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        if recorded:
            session.read_result(0, [0])
        if i >= (3 if recorded else 2):
            times.append(start.elapsed_time(end))
            host.append((t1 - t0) * 1e3)
        cache.release(rc)
    runner.check_errors()
    ms = sorted(times)[len(times) // 2]
    flops = flops(T) if flops is not None else prefill_flops(cfg, T, layers)
    peak = peaks["bf16_tflops_sustained"]
    del runner, cache
    torch.cuda.empty_cache()
    return {"value": T * 1000.0 / ms, "tokens": T, "ms": ms, "host_ms": sorted(host)[len(host) // 2],
            "frac": flops / (ms * 1e-3) / (peak * 1e12), "tflops": flops / (ms * 1e-3) / 1e12,
            "peak_tflops": peak,
            # the same against the burst rate of the library product (a kernel timed in isolation)
            "frac_of_burst": flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)}


# ---------------------------------------------------------------------------------------------
# --design rugesun: the Rugesun decoder beside the Llama decoder at equal sizes
# ---------------------------------------------------------------------------------------------
def rugesun_config(width, layers, heads, ff, vocab, q_rank, experts=16, top=4, window=4096,
                   dim=128, rot=64, vdim=128, kv_rank=512):
    """Layers in fours: two that keep a latent cache (a gated GELU feed-forward, then a
    mixture of experts) and two that read the second one's cache (the same feed-forwards).
    An expert has ff / top columns, so a token's chosen experts do a dense layer's work."""
    def mixer(kv_from=None):
        m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": (dim + rot) ** -0.5, "rot": {"base": 10000.0, "dims": rot}, "mask": {"size": window}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return m
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top}}
    out = []
    for i in range(layers):
        base = i - i % 4
        kv_from = base + 1 if i % 4 >= 2 else None
        out.append({"type": "latent_attention", "mixer": mixer(kv_from), "mlp": dense if i % 2 == 0 else moe})
    return {"architecture": "Rugesun", "vocab": vocab, "width": width, "postln_alpha": 1.0, "logit_softcap": 25.0,
            "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 37, "mul_cur": 19}},
            "layers": out, "max_position": 8192}


def rugesun_prefill_flops(cfg: dict, T: int) -> float:
    """Multiply-adds x 2 of one prompt step as the engine computes it (queries taken into
    latent space, attention over the cached latents), counting a token's chosen experts only."""
    D, total = cfg["width"], 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        H, d, r, v, kr, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        w = (m.get("mask") or {}).get("size", 0)
        down = qr + (0 if "kv_from" in m else kr + r)
        keys = sum(min(t + 1, w) if w else t + 1 for t in range(T))
        total += 2.0 * T * (D * down + qr * H * (d + r) + H * d * kr + H * kr * v + H * v * D)
        total += 2.0 * H * (2 * kr + r) * keys
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            total += 6.0 * T * D * mlp["ff"]
        elif mlp:
            total += 6.0 * T * D * mlp["expert"]["ff"] * mlp["router"]["top"] + 2.0 * T * D * mlp["router"]["experts"]
    return total + 2.0 * D * cfg["vocab"]


def nadozen_config(width, layers, heads, kv_heads, ff, vocab, window=4096, streams=4):
    """Layers in pairs, each with a gated SiLU feed-forward: sliding-window attention with a
    sink beside a state space layer (inner width = model width, heads of 64, a state of 128),
    then wkv time mixing (heads of 64); four residual streams."""
    par = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                    "mask": {"size": window}},
           "right": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1},
           "left_scale": 0.5, "right_scale": 0.5}
    wkv = {"heads": width // 64, "dim": 64, "decay_rank": 64}
    dense = {"kind": "dense", "ff": ff}
    out = [{"type": "parallel", "mixer": par, "mlp": dense} if i % 2 == 0 else
           {"type": "wkv", "mixer": wkv, "mlp": dense} for i in range(layers)]
    return {"architecture": "Nadozen", "vocab": vocab, "width": width, "logit_scale": 1.0, "norm": {"eps": 1e-6},
            "streams": streams, "layers": out, "max_position": 8192}


def nadozen_prefill_flops(cfg: dict, T: int) -> float:
    """Multiply-adds x 2 of one prompt step: the products, the attention inside its window,
    and the scans' updates and read-outs of their states."""
    D, total = cfg["width"], 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if layer["type"] == "wkv":
            hk, rank = m["heads"] * m["dim"], m.get("decay_rank") or 64
            total += 2.0 * T * (5 * D * hk + D * rank + rank * hk) + 2.0 * T * m["heads"] * m["dim"] ** 2 * 3
        else:
            a, r = m["left"], m["right"]
            w = (a.get("mask") or {}).get("size", 0)
            keys = sum(min(t + 1, w) if w else t + 1 for t in range(T))
            qd = a["heads"] * a["dim"]
            inner = r["heads"] * r["vdim"]
            rows_in = 2 * inner + 2 * r["groups"] * r["state"] + r["heads"]
            total += 2.0 * T * D * (3 * qd + a["kv_heads"] * a["dim"]) + 4.0 * a["heads"] * a["dim"] * keys
            total += 2.0 * T * D * (rows_in + inner) + 2.0 * T * r["heads"] * r["state"] * r["vdim"] * 2.5
        if layer.get("mlp"):
            total += 6.0 * T * D * layer["mlp"]["ff"]
    return total + 2.0 * D * cfg["vocab"]


def bolovik_config(width, layers, heads, kv_heads, ff, vocab, window=4096, keep_first=4, experts=16, top=4):
    """Layers in pairs: sliding-window attention that keeps the first tokens (heads of 128, half of
    each rotated) with a gated GELU feed-forward, then a gated delta rule (value heads of 128 over
    half as many key heads, a convolution of 4 taps) with a mixture of experts whose chosen experts
    do a dense layer's work (an expert has ff / top columns; four groups of which two stay open)."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
           "mask": {"size": window, "keep_first": keep_first},
           "rot": {"dims": 64, "base": 500000.0,
                   "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    dh = width // 128
    delta = {"heads": dh, "kv_heads": max(1, dh // 2), "dim": 128, "vdim": 128, "conv": 4}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // top},
           "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}}
    out = [{"type": "attention", "mixer": att, "mlp": dense} if i % 2 == 0 else
           {"type": "delta", "mixer": delta, "mlp": moe} for i in range(layers)]
    return {"architecture": "Bolovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4},
            "layers": out, "max_position": 8192}


def bolovik_prefill_flops(cfg: dict, T: int) -> float:
    """Multiply-adds x 2 of one prompt step: the products (a token's chosen experts only), the
    attention over the keys each query sees, and the delta rule's two reads and one write of its
    state per token."""
    D, total = cfg["width"], 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "delta":
            total += 2.0 * T * D * (2 * G * d + 2 * H * v + 2 * H) + 2.0 * T * H * v * D + 2.0 * T * H * d * v * 3
        else:
            mask = m.get("mask") or {}
            w, keep = mask.get("size", 0), mask.get("keep_first", 0)
            keys = sum(min(t + 1, w + min(keep, max(0, t + 1 - w))) if w else t + 1 for t in range(T))
            total += 2.0 * T * D * (H * d + G * d + G * v) + 2.0 * T * H * v * D + 2.0 * H * (d + v) * keys
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            total += 6.0 * T * D * mlp["ff"]
        elif mlp:
            total += 6.0 * T * D * mlp["expert"]["ff"] * mlp["router"]["top"] + 2.0 * T * D * mlp["router"]["experts"]
    return total + 2.0 * D * cfg["vocab"]


def vodatar_config(width, layers, heads, kv_heads, ff, vocab, experts=16, top=4, identity=1):
    """Layers in fours: attention through a latent (heads of 128 + 64 rotated, values of 128, a latent of
    512, frequencies on a ramp), then three layers of differential attention (half the heads, two maps
    of 128 each, values of 256, a convolution of 4 taps, scores capped at 50); every layer with a
    mixture of experts whose chosen experts do half a dense layer's work (an expert has ff / (2 top)
    columns; one more router output hands the input on) beside a shared expert that does the other
    half.  The first two layers are walked twice, so ``layers`` runs come from ``layers - 2`` layers."""
    lat = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
           "rot": {"dims": 64, "base": 10000.0,
                   "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
    att = {"heads": max(1, heads // 2), "kv_heads": max(1, kv_heads // 2), "dim": 128, "vdim": 256,
           "scale": 128 ** -0.5, "softcap": 50.0, "diff": 0.3, "conv": 4, "rot": {"dims": 128, "base": 500000.0}}
    moe = {"kind": "moe", "expert": {"ff": ff // (2 * top)},
           "router": {"experts": experts, "top": top, "identity": identity}, "shared": {"ff": ff // 2}}
    n = max(layers - 2, 2)
    out = [{"type": "latent_attention" if i % 4 == 0 else "attention", "mixer": lat if i % 4 == 0 else att, "mlp": moe}
           for i in range(n)]
    return {"architecture": "Vodatar", "vocab": vocab, "width": width, "residual_mult": 0.7,
            "norm": {"eps": 1e-6, "groups": 4}, "canon": {"taps": 3}, "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": out, "max_position": 8192}


def vodatar_prefill_flops(cfg: dict, T: int) -> float:
    """Multiply-adds x 2 of one prompt step: the products of every run of a layer (a token's chosen
    experts only, the shared expert, the gates of both sub-layers, the product that re-enters a pass),
    attention in latent space as the engine computes it, and both score maps over the keys a query sees."""
    D, total = cfg["width"], 0.0
    keys = T * (T + 1) / 2.0
    loop = cfg.get("loop")
    runs = list(range(len(cfg["layers"])))
    if loop:
        runs = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] \
            + list(range(loop["stop"], len(cfg["layers"])))
        total += 2.0 * T * D * 2 * D * loop["times"]
    for i in runs:
        layer = cfg["layers"][i]
        m = layer["mixer"]
        if layer["type"] == "attention":
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            total += 2.0 * T * D * (H * 2 * d + G * 2 * d + G * v) + 2.0 * T * H * v * D + 2.0 * H * (2 * d + 2 * v) * keys
        else:
            H, d, r, v, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            total += 2.0 * T * D * (H * (d + r) + kr + r) + 2.0 * T * H * (d + v) * kr + 2.0 * T * H * v * D \
                + 2.0 * H * (2 * kr + r) * keys
        total += 2.0 * T * D * D  # the mixer's gate
        mlp = layer.get("mlp")
        if mlp:
            r = mlp["router"]
            total += 6.0 * T * D * mlp["expert"]["ff"] * r["top"] + 2.0 * T * D * (r["experts"] + r.get("identity", 0)) \
                + 6.0 * T * D * (mlp.get("shared") or {}).get("ff", 0) + 2.0 * T * D * D
    return total + 2.0 * D * cfg["vocab"]


DESIGN_SIZES = {
    # name: (width, layers, heads, feed-forward, vocabulary, q_rank, llama kv heads)
    "2b-shape": (2048, 8, 16, 8192, 32000, 768, 4),
    "8b-shape": (4096, 8, 32, 14336, 32000, 1536, 8),
}


def design_compare(args, peaks) -> dict:
    """Prefill and decode of the chosen design at a few sizes, and of the decoder it is set beside
    (the Llama decoder; for Bolovik the Nadozen decoder, whose layers also alternate window
    attention and a recurrent state; for Vodatar the Rugesun decoder, which also has attention
    through a latent and mixtures of experts) at the same width, depth, heads, feed-forward width and
    vocabulary."""
    import gc

    import torch

    import infernum_b200 as ib

    opts = {"sm_count": torch.cuda.get_device_properties(0).multi_processor_count}
    out = {}
    for name, (width, layers, heads, ff, vocab, q_rank, kv_heads) in DESIGN_SIZES.items():
        if args.size and name != args.size:
            continue
        if args.layers:
            layers = args.layers
        llama = {"model_type": "llama", "num_hidden_layers": layers, "hidden_size": width,
                 "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
                 "intermediate_size": ff, "vocab_size": vocab, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
                 "tie_word_embeddings": False, "max_position_embeddings": 8192}
        beside, beside_cfg, beside_flops = "llama", llama, None
        if args.design == "nadozen":
            other = nadozen_config(width, layers, heads, kv_heads, ff, vocab)
            other_flops = nadozen_prefill_flops
        elif args.design == "bolovik":
            other = bolovik_config(width, layers, heads, kv_heads, ff, vocab)
            other_flops = bolovik_prefill_flops
            beside, beside_cfg, beside_flops = "nadozen", nadozen_config(width, layers, heads, kv_heads, ff, vocab), \
                nadozen_prefill_flops
        elif args.design == "vodatar":
            other = vodatar_config(width, layers, heads, kv_heads, ff, vocab)
            other_flops = vodatar_prefill_flops
            beside, beside_cfg, beside_flops = "rugesun", rugesun_config(width, layers, heads, ff, vocab, q_rank), \
                rugesun_prefill_flops
        else:
            other = rugesun_config(width, layers, heads, ff, vocab, q_rank)
            other_flops = rugesun_prefill_flops
        for label, cfg in ((args.design, other), (beside, beside_cfg)):
            if args.only_model and label != args.only_model:
                continue
            model = ib.random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0", options=dict(opts))
            row = {}
            if label == args.design:
                flops = lambda T, c=cfg: other_flops(c, T)  # noqa: E731
            elif beside_flops is not None:
                flops = lambda T, c=cfg: beside_flops(c, T)  # noqa: E731
            else:
                flops = lambda T, c=cfg: prefill_flops(c, T, layers)  # noqa: E731
            for T in (512, 2048):
                if args.only == "decode":
                    break
                r = time_prefill(model, cfg, layers, T, args.page_size, peaks, flops=flops)
                row[f"prefill_{T}_tok_s"] = round(r["value"], 1)
                row[f"prefill_{T}_ms"] = round(r["ms"], 3)
                row[f"prefill_{T}_frac_of_sustained_bf16"] = round(r["frac"], 4)
                if T == 512:
                    # the way Engine runs a prompt that comes alone: replayed from a recording
                    r = time_prefill(model, cfg, layers, T, args.page_size, peaks, flops=flops, recorded=True)
                    row["prefill_512_recorded_ms"] = round(r["ms"], 3)
                    row["prefill_512_recorded_host_ms"] = round(r["host_ms"], 3)
                    row["prefill_512_recorded_frac_of_sustained_bf16"] = round(r["frac"], 4)
            for b in (1, 8, 64):
                if args.only == "prefill":
                    break
                r = time_decode(model, b, args.prompt_len, min(args.steps, 64), max(args.warmup, 3), args.page_size,
                                args.seed + b, graph=not args.no_cuda_graph)
                row[f"decode_b{b}_tok_s"] = round(r["tokens_per_s"], 1)
                row[f"decode_b{b}_ms"] = round(r["ms_per_step"], 4)
                row[f"decode_b{b}_hbm_frac"] = round(
                    r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                row[f"decode_b{b}_launches"] = r["launches_per_step"]
            row["weight_gb"] = round(model.step_weight_bytes() / 1e9, 3)
            out[f"{name}/{label}"] = row
            del model
            gc.collect()
            torch.cuda.empty_cache()
    return out


def scheduler_workloads(seed: int) -> dict:
    """The mixed workload at the 1B layer sizes and the page-pressure workload at
    the 13B layer sizes, through ``Engine`` (``infernum_b200.cli.bench``), as
    flat entries for ``points``."""
    import gc
    from types import SimpleNamespace

    import torch

    from infernum_b200.cli import bench as cli

    out = {}
    base = dict(dtype="bf16", layers=None, seed=seed, block_size=16, requests=None, prompt_len=None,
                new_tokens=None, num_blocks=None, no_warmup=False, n_gen=128)
    args = SimpleNamespace(model="1b", workload="mixed", **base)
    model = cli.load(args)
    r = cli.run_mixed(model, args)
    out.update({"mixed_1b_tok_s": round(r["total_tok_s"], 1), "mixed_1b_decode_tok_s": round(r["decode_tok_s"], 1),
                "mixed_1b_prefill_tokens": r["prefill_tokens"], "mixed_1b_decode_tokens": r["decode_tokens"],
                "mixed_1b_steps": r["steps"], "mixed_1b_budget_use": round(r["budget_use"], 3),
                "mixed_1b_ms_per_step": round(r["ms_per_step"], 3),
                "mixed_1b_host_ms_per_step": round(r["host_ms_per_step"], 3),
                "mixed_1b_steps_replayed": r["steps_run"].get("replayed", 0),
                "mixed_1b_steps_launched_ahead": r.get("steps_launched_ahead", 0),
                "mixed_1b_preemptions": r["preemptions"]})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    args = SimpleNamespace(model="13b", workload="pressure", solo_checks=4, **base)
    model = cli.load(args)
    r = cli.run_pressure(model, args)
    out.update({"pressure_13b_tok_s": round(r["total_tok_s"], 1), "pressure_13b_decode_tok_s": round(r["decode_tok_s"], 1),
                "pressure_13b_layers": len(model.layers), "pressure_13b_num_blocks": r["num_blocks"],
                "pressure_13b_blocks_for_all": r["blocks_for_all"], "pressure_13b_preemptions": r["preemptions"],
                "pressure_13b_requests_preempted": r["requests_preempted"],
                "pressure_13b_solo_checked": r["solo_checked"],
                "pressure_13b_identical_to_solo": r["identical_to_solo"],
                "pressure_13b_first_difference_at": ",".join(str(i) for i in r["first_difference_at"]),
                # (bfloat16, random weights: a differing token must be a near-tie by the logits)
                "pressure_13b_largest_gap_at_difference": max(r["logit_gap_at_first_difference"] + [0.0])})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    # the same in true 32-bit, where a preempted request must reproduce its tokens exactly
    # (four layers and eight requests: the 32-bit products run on the FMA units)
    args = SimpleNamespace(model="13b", workload="pressure", solo_checks=4,
                           **dict(base, dtype="f32", layers=4, requests=8, prompt_len=1024, new_tokens=256))
    model = cli.load(args)
    r = cli.run_pressure(model, args)
    out.update({"pressure_13b_f32_layers": 4, "pressure_13b_f32_requests": 8, "pressure_13b_f32_prompt_len": 1024,
                "pressure_13b_f32_preemptions": r["preemptions"],
                "pressure_13b_f32_solo_checked": r["solo_checked"],
                "pressure_13b_f32_identical_to_solo": r["identical_to_solo"]})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--skip-extras", action="store_true", help="only the headline decode run")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print its numbers (for profiling)")
    ap.add_argument("--no-cuda-graph", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--design", choices=["rugesun", "nadozen", "bolovik", "vodatar"], default=None,
                    help="instead of the default workload: prefill and decode of this design at a few sizes,\n"
                         "beside the Llama decoder (bolovik: the Nadozen decoder; vodatar: the Rugesun decoder) at equal sizes; prints one JSON line {\"design\": ...}")
    ap.add_argument("--size", default=None, help="with --design: one of its sizes only")
    ap.add_argument("--only-model", default=None, help="with --design: the design's name, or the name of the one beside it, only")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "infernum-rs/infernum is a Rust workspace; neither cargo nor rustc is "
                          "installed here and it has no Python package to install offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import infernum_b200 as ib
    from infernum_b200.csrc.build import loaded_libraries

    peaks = load_peaks()
    if args.design:
        torch.cuda.set_device(0)
        print(json.dumps({"design": args.design, "dtype": "bf16", "data": "synthetic: seeded random weights",
                          "prompt_len": args.prompt_len, "peaks": peaks["source"],
                          "sizes": design_compare(args, peaks)}))
        return 0
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    model = ib.random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0",
                            options={"sm_count": torch.cuda.get_device_properties(0).multi_processor_count})
    if args.only == "decode":
        r = time_decode(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size, args.seed,
                        graph=not args.no_cuda_graph)
        print(json.dumps({"only": "decode", "batch": args.batch, **r}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", **time_prefill(model, cfg, layers, 2048, args.page_size, peaks)}))
        return 0
    clocks = ClockSampler(0)
    clocks.start()
    try:
        # The prompt step is bound by arithmetic and so by the SM clock, which sags under the
        # power cap once the decode runs have heated the part (decode is bound by HBM): it is
        # timed here, on the cool part, and again after the decode runs; the line carries the
        # later, slower figure and names the earlier one beside it.
        cool = None if args.skip_extras else time_prefill(model, cfg, layers, 2048, args.page_size, peaks)
        main_run = time_decode(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size,
                               args.seed, clocks)
        e2e = time_e2e(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size, args.seed + 1)
        e2e["tokens"] = "fed on the device to a step launched ahead; positions, lengths and slots from the host"
        if not args.skip_extras:
            fed = time_e2e(model, args.batch, args.prompt_len, min(args.steps, 64), warmup, args.page_size,
                           args.seed + 1, launch_ahead=False)
            e2e["value_host_fed"] = round(fed["value"], 2)  # every step launched after the one before was read
            e2e["h2d_bytes_per_step_host_fed"] = fed["h2d_bytes_per_step"]
        points = {}
        if not args.skip_extras:
            for b in (1, 64):
                r = time_decode(model, b, args.prompt_len, min(args.steps, 64), warmup, args.page_size,
                                args.seed + 2 + b)
                points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
                points[f"decode_b{b}_hbm_frac"] = round(
                    r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            # the same batch of 8 near the end of the 8,192-token context the configuration names
            r = time_decode(model, 8, 8192 - 128, 32, warmup, args.page_size, args.seed + 9)
            points["decode_b8_ctx8k"] = round(r["tokens_per_s"], 1)
            points["decode_b8_ctx8k_hbm_frac"] = round(
                r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        if not args.skip_extras:
            # short prompts, the way the engine runs a prompt that comes alone: device time, the
            # host's own time for the step, and the fraction of the sustained bf16 rate
            for T in (256, 512):
                r = time_prefill(model, cfg, layers, T, args.page_size, peaks, recorded=True)
                points[f"prefill_{T}_ms"] = round(r["ms"], 3)
                points[f"prefill_{T}_host_ms"] = round(r["host_ms"], 3)
                points[f"prefill_{T}_frac"] = round(r["frac"], 4)
        prefill = None
        if cool is not None:
            prefill = time_prefill(model, cfg, layers, 2048, args.page_size, peaks)
            prefill.update({"when": "after the decode runs", "ms_cool": cool["ms"], "frac_cool": cool["frac"],
                            "value_cool": cool["value"]})
        libraries = [os.path.basename(p) for p in loaded_libraries()]
        if not args.skip_extras and not args.layers:
            del model
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            points.update(scheduler_workloads(args.seed))
    finally:
        clocks.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s (Llama-3.1-8B layer sizes, random bf16 weights)",
        "value": round(main_run["tokens_per_s"], 2),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), seeded uniform token ids",
        "config": {
            "model": "llama-3.1-8b-shape", "layers": layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": args.prompt_len, "context_len": 8192,
            "page_size": args.page_size, "parallelism": "single-gpu",
            "l2": "inputs larger than L2 (15 GB of weights per step)",
            "cuda_graph": bool(main_run["graph"]),
        },
        "clocks": main_run["clocks"],
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main_run["launches_per_step"]) * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "peaks": peaks["source"]},
        "points": points,
        "kernel_libraries": libraries,
    }
    if prefill is not None:
        line["prefill"] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
