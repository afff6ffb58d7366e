"""The Vodatar decoder on the GPU against the plain implementation
(``plain_vodatar``): each mechanism alone; whole prompts, token-by-token decoding,
portions down to two tokens, mixed batches with pages and state slots used again,
long decoding; keys far away and at page borders made to stand out; the first
tokens of a sequence; sizes that are 1 or equal; layers without a feed-forward;
greedy generation through the engine."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vodatar as pv
from helpers import (ROOT, TOL, compare_trace, peak_tokens, random_tokens, run_trace_inprocess,
                     run_trace_subprocess, trace_mixed, trace_portions, trace_tail, trace_whole)
from vodatar_cases import CASES, PAGE_SIZES, make_folder, random_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [31, 45, 1, 2, 90, 17], "B": [23, 60, 3, 1, 41, 8], "C": [130, 75, 2, 200, 33, 64],
           "D": [150, 3, 67, 1, 40, 129], "E": [50, 2, 27, 1, 12]}
NAMES = ["A", "B", "C", "D", "E", "Asharp", "Dsharp"]
# In bfloat16 a router's score carries the rounding of everything before it; where the last chosen
# output lies within that of the best one left out, the engine may choose otherwise than the 64-bit
# plain implementation: a different, equally valid, result.  Such positions (by the plain
# implementation's own margin between choice values) are not compared in bfloat16.
ROUTING_MARGIN = 0.002
# The test models' projections are scaled up (so that a wrong key shows); rounding is scaled with them.
F32_SLACK = 3


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CASES.items()):
        folder = make_folder(str(tmp_path_factory.mktemp(f"vdt{name}")), cfg, seed=31 + i)
        out[name] = (folder, pv.Plain(folder))
        steady = make_folder(str(tmp_path_factory.mktemp(f"vdtsteady{name}")), cfg, seed=31 + i, gain=0.25,
                             correction=15.0)
        out[name + "/bfloat16"] = (steady, pv.Plain(steady))
        if name in ("A", "D"):
            sharp = make_folder(str(tmp_path_factory.mktemp(f"vdtsharp{name}")), cfg, seed=61 + i, sharpen=6.0)
            out[name + "sharp"] = (sharp, pv.Plain(sharp))
    return out


def sequences(name):
    key = name.replace("sharp", "")
    return {f"r{i}": random_tokens(n, CASES[key]["vocab"], 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def pick(models, name, dtype):
    """The model of a case for a dtype: in bfloat16 the one whose routers' choices rest mostly on their
    corrections and whose projections are scaled up less.  Rounding to 8 bits before a router changes a
    choice among experts in a few tokens of a hundred, and every later token reads those tokens' keys."""
    return models.get(f"{name}/{dtype}", models[name])


def replay(models, name, dtype, steps, tmp_path, max_tokens=None):
    folder, plain = pick(models, name, dtype)
    out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"), max_tokens or peak_tokens(steps),
                              PAGE_SIZES[name.replace("sharp", "")])
    return out, plain


def names_for(dtype):
    # (where attention is peaked, bfloat16 rounding of a score is multiplied on its way to the logits)
    return NAMES if dtype == "float32" else ["A", "B", "C", "D", "E"]


def compare(steps, out, seqs, plain, dtype, name, slack=1):
    """float32: every position within the tolerance.  bfloat16: a request's positions before its
    first near-tie of the routing (a token routed otherwise than in the plain implementation is another
    valid result, and every later token of the request reads its keys and values); of those at most
    one in ten may lie beyond the tolerance, the median at most half of it; every value is finite."""
    if dtype == "float32":
        return compare_trace(steps, out, seqs, plain, TOL[dtype] * F32_SLACK * (3 if "sharp" in name else 1) * slack)
    fed = {rid: 0 for rid in seqs}
    errs, skipped = [], 0
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            assert e["tokens"] == seqs[rid][fed[rid]: fed[rid] + n], "trace feeds wrong tokens"
            ref_all, margins = plain.logits(seqs[rid]), plain.margins(seqs[rid])
            for w in e.get("want", []):
                pos = fed[rid] + w
                got, ref = out[s["step"]][row], ref_all[pos].numpy()
                row += 1
                assert np.isfinite(got).all()
                close = (margins < ROUTING_MARGIN).nonzero().flatten()
                if len(close) and pos >= int(close[0]):
                    skipped += 1
                    continue
                errs.append(float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6)))
            fed[rid] += n
        for rid in s.get("end", []):
            fed[rid] = 0
    assert len(errs) >= min(3, (len(errs) + skipped) // 10), f"{len(errs)} positions compared, {skipped} left out"
    errs = np.sort(np.array(errs))
    tol = TOL[dtype] * slack
    over = int((errs > tol).sum())
    summary = f"{len(errs)} positions, median {np.median(errs):.3e}, worst {errs[-1]:.3e}, {over} beyond {tol:.1e}"
    assert over <= max(1, len(errs) // 10), summary
    assert np.median(errs) <= tol / 2, summary
    return summary


def runtime(dtype, **options):
    from infernum_b200.ops import core
    from infernum_b200.parts.base import Runtime
    return Runtime(DEV, dtype, err=core.new_error_word(DEV), options=options)


def rel_err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / max(ref.abs().max().item(), 1e-9))


PART_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


# ---- whole models through the trace runner -------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = sequences(name)
    steps = []
    for rid, seq in seqs.items():
        steps += trace_whole(rid, seq, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_most_in_one_step_then_token_by_token(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for rid, seq in seqs.items():
        steps += trace_tail(rid, seq, 40, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_a_prompt_token_by_token_from_its_first_token(models, name, dtype, tmp_path):
    """Every token a step of its own from position 0: the convolutions' states begin empty."""
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {"r0": sequences(name)["r0"][:24]}
    steps = [{"step": i, "entries": [{"id": "r0", "tokens": [t], "want": [0]}], "end": []}
             for i, t in enumerate(seqs["r0"])]
    steps[-1]["end"] = ["r0"]
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for i, (rid, seq) in enumerate(seqs.items()):
        sizes = [[7, 2, 5, 3, 11, 2], [2, 2, 13, 4, 2, 9], [5, 17, 2, 3, 40], [2]][i % 4]
        steps += trace_portions(rid, seq, sizes, step0=len(steps))
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = sequences(name)
    steps = trace_mixed(seqs, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    peak = peak_tokens(steps)
    assert peak < sum((len(v) + 63) // 64 * 64 for v in seqs.values())
    out, plain = replay(models, name, dtype, steps, tmp_path, max_tokens=peak)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "Dsharp"])
def test_long_decoding(models, name, dtype, tmp_path):
    if dtype == "bfloat16":
        name = {"A": "A", "Dsharp": "E"}[name]  # (E has no routers: every position is compared)
    key = name.replace("sharp", "")
    seqs = {"long": random_tokens(230, CASES[key]["vocab"], 3)}
    if dtype == "bfloat16":
        # the sequence, of a few, whose first near-tie of the routing comes latest: what lies before it is compared
        _, plain = pick(models, name, dtype)
        def clean(seq):
            close = (plain.margins(seq) < ROUTING_MARGIN).nonzero().flatten()
            return int(close[0]) if len(close) else len(seq)
        seqs = {"long": max((random_tokens(230, CASES[key]["vocab"], s) for s in range(3, 23)), key=clean)}
        assert clean(seqs["long"]) >= 40
    steps = trace_tail("long", seqs["long"], tail=226)
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("seed", [2, 3, 5, 8, 13, 21, 34, 55])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Sizes, orders and constants nobody chose by hand: mixed batches with pages and slots used again,
    then a long tail decoded token by token, in 32-bit against the plain implementation."""
    cfg = random_case(seed)
    folder = make_folder(str(tmp_path / "m"), cfg, seed=seed)
    plain = pv.Plain(folder)
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], 31 * i + n) for i, n in enumerate([150, 70, 2, 19 + seed, 129, 1])}
    for rid, seq in seqs.items():
        # a router whose two candidates lie within 32-bit rounding of each other may choose either:
        # the sequence ends before such a token
        close = (plain.margins(seq) < 1e-5).nonzero().flatten().tolist()
        if close:
            seqs[rid] = seq[:max(close[0], 1)]
    steps = trace_mixed(seqs, max_live=4, seed=seed)
    if len(seqs["r0"]) > 3:
        steps += trace_tail("r0", seqs["r0"], 140, step0=len(steps))
    out = run_trace_inprocess(folder, "float32", steps, str(tmp_path / "out"), max(peak_tokens(steps), 256), 16)
    compare_trace(steps, out, seqs, plain, TOL["float32"] * F32_SLACK)


@pytest.mark.parametrize("seed", [4, 9])
def test_configurations_drawn_at_random_in_bfloat16(seed, tmp_path):
    cfg = random_case(seed)
    folder = make_folder(str(tmp_path / "m"), cfg, seed=seed, gain=0.25, correction=15.0)
    plain = pv.Plain(folder)
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], 17 * i + n) for i, n in enumerate([90, 40, 2, 70, 1])}
    steps = trace_mixed(seqs, max_live=4, seed=seed)
    out = run_trace_inprocess(folder, "bfloat16", steps, str(tmp_path / "out"), max(peak_tokens(steps), 256), 16)
    compare(steps, out, seqs, plain, "bfloat16", "random")


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_and_batching_change_logits_by_rounding_only(models, dtype, tmp_path):
    folder, plain = pick(models, "D", dtype)
    seqs = sequences("D")
    seq = seqs["r0"]
    runs = []
    mixed = trace_mixed(seqs, max_live=4, seed=9)
    for i, steps in enumerate([trace_whole("r0", seq), trace_portions("r0", seq, [7, 2, 5, 3, 11, 2]),
                               trace_tail("r0", seq, 60), mixed]):
        out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / f"o{i}"), peak_tokens(steps) + 64, 16)
        rows, pos = {}, 0
        for s in steps:
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    if e["id"] == "r0":
                        rows[pos + w] = out[s["step"]][r]
                    r += 1
                if e["id"] == "r0":
                    pos += len(e["tokens"])
        runs.append(rows)
    scale = max(np.abs(v).max() for v in runs[0].values())
    tol = 2e-5 if dtype == "float32" else 4e-2
    margins = plain.margins(seq)
    for other in runs[1:]:
        assert other
        far = 0
        for pos, row in other.items():
            if dtype == "bfloat16" and float(margins[pos]) < ROUTING_MARGIN:
                continue
            if np.abs(row - runs[0][pos]).max() / scale > tol:
                far += 1
        assert far <= (0 if dtype == "float32" else max(1, len(other) // 10))


def test_the_stream_after_every_run_of_a_layer(models):
    """In 32-bit the stream after each run of a layer (a looped layer counts each time) equals the plain one."""
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.loading import load_model
    for name in ("A", "B", "C", "D", "E"):
        folder, plain = models[name]
        model = load_model(folder, dtype="float32")
        cache = CacheManager(model.cache_needs(), page_size=4, num_pages=64, max_requests=2,
                             dtype=model.rt.dtype, device=model.rt.device)
        runner = ModelRunner(model, cache, max_rows=256, max_entries=2)
        seen = []
        for blk in model.layers:
            def hooked(stream, ctx, c, orig=blk.forward):
                orig(stream, ctx, c)
                seen.append(stream.residual.clone())
            blk.forward = hooked
        seq = random_tokens(50, CASES[name]["vocab"], 77)
        _, want = pv.forward(seq, plain.cfg, plain.weights, keep_layers=True)
        runner.step([StepEntry(cache.admit("x"), seq, [])])
        runner.check_errors()
        assert len(seen) == len(want) == len(pv.run_order(plain.cfg))
        for i, (got, ref) in enumerate(zip(seen, want)):
            assert rel_err(got, ref) < 2e-5, f"case {name} run {i}"


def test_the_program_itself_in_a_subprocess(models, tmp_path):
    seqs = {k: v for k, v in sequences("A").items() if len(v) > 3}
    steps = trace_mixed(seqs, max_live=3, seed=3)
    for dtype in DTYPES:
        folder, plain = pick(models, "A", dtype)
        out = run_trace_subprocess(folder, dtype, steps, str(tmp_path / dtype), peak_tokens(steps))
        compare(steps, out, seqs, plain, dtype, "A")


# ---- generation through the engine -----------------------------------------------------
def check_greedy(plain, prompt, got, dtype):
    """Every generated token is the plain implementation's best, or within rounding of it; after
    a near-tie the two may part, so the comparison follows what was generated.  In bfloat16 a
    step behind a near-tie of the routing is not held to the logits' gap."""
    seq = list(prompt)
    for i, tok in enumerate(got):
        logits = plain.logits(seq)[-1]
        best = pv.argmax(logits)
        if tok != best:
            gap = float((logits[best] - logits[tok]) / logits.abs().max())
            routed_close = dtype == "bfloat16" and float(plain.margins(seq).min()) < ROUTING_MARGIN
            assert gap < (1e-4 if dtype == "float32" else 5e-2) or routed_close, \
                f"token {i}: {tok} against {best}, gap {gap:.4f}"
        seq.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_through_the_engine(models, name, dtype):
    import infernum_b200 as ib
    folder, plain = pick(models, name, dtype)
    model = ib.load_model(folder, dtype=dtype)
    page = PAGE_SIZES[name]
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=3, block_size=page, num_blocks=480 // page,
                                             max_prefill_tokens=24))
    vocab = CASES[name]["vocab"]
    prompts = [random_tokens(n, vocab, 7 * n) for n in (5, 41, 18, 2, 30)]
    n_new = 30
    outs = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=n_new))
    for prompt, got in zip(prompts, outs):
        assert len(got) == n_new
        check_greedy(plain, prompt, got, dtype)
    # recurring steps ran from recordings: the parts take entries, slots and positions from the device
    assert model.replayable
    if engine.decoder is not None:
        assert engine.decoder.counts["replayed"] > 0
    # once more on the same engine: slots and pages that were used before
    again = engine.generate_batch(prompts[:2], ib.GenerateOptions(max_new_tokens=8))
    for prompt, got in zip(prompts[:2], again):
        check_greedy(plain, prompt, got, dtype)


def test_generation_with_too_few_pages_preempts_and_recomputes(models):
    import infernum_b200 as ib
    folder, plain = models["A"]
    model = ib.load_model(folder, dtype="float32")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, block_size=4, num_blocks=34, max_prefill_tokens=16))
    prompts = [random_tokens(n, CASES["A"]["vocab"], 11 * n) for n in (20, 33, 25, 14)]
    outs = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=30))
    for prompt, got in zip(prompts, outs):
        check_greedy(plain, prompt, got, "float32")


def test_command_line_generate(models, tmp_path):
    """``bin/generate`` picks the architecture by config.json: from a model folder, and from a bare
    configuration with random weights."""
    folder, plain = models["E"]
    prompt = random_tokens(9, CASES["E"]["vocab"], 1)
    text = ",".join(map(str, prompt))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "-m", folder, text, "-n", "6",
                           "--greedy", "--dtype", "float32", "--block-size", "4"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith(text)][0]
    got = [int(t) for t in line.split()[1:]]
    assert len(got) == 6
    check_greedy(plain, prompt, got, "float32")
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CASES["B"]))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--config", str(cfg_path),
                           "--random-weights", "--weights-seed", "3", "1,2,3", "-n", "4", "--greedy",
                           "--block-size", "8"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert "Generated 4 tokens" in proc.stdout


# ---- mechanisms alone ------------------------------------------------------------------
class Step:
    """The device tensors of a step that the kernels read."""

    def __init__(self, rows_per_entry, slots, starts=None):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        cu = [0]
        for n in rows_per_entry:
            cu.append(cu[-1] + n)
        starts = starts or [0] * len(rows_per_entry)
        self.n_entries = len(rows_per_entry)
        self.n_rows = cu[-1]
        self.cu_rows = i32(cu)
        self.slot_ids = i32(slots)
        self.row_entry = i32([e for e, n in enumerate(rows_per_entry) for _ in range(n)])
        self.positions = i32([s + i for s, n in zip(starts, rows_per_entry) for i in range(n)])


def cuts_of(T, sizes):
    out, at, i = [], 0, 0
    while at < T:
        n = min(sizes[i % len(sizes)], T - at)
        out.append((at, n))
        at += n
        i += 1
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,parts", [(96, 3), (72, 1), (384, 6), (64, 64), (1024, 4), (30, 2)])
def test_gated_result_normed_in_parts_and_added_with_a_factor(dtype, W, parts):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(W + parts)
    N, eps, mult = 11, 3e-6, 0.7
    x = torch.randn(N, W, generator=g) * 2
    y = (torch.randn(N, W, generator=g) * 5).to(dtype)
    # one part of one row is tiny beside eps: the eps sits inside the root
    y[3, : W // parts] = (y[3, : W // parts].float() * 1e-3).to(dtype)
    gate = (torch.randn(N, 2 * W, generator=g) * 2).to(dtype)  # the gate's logits lie in wider rows
    bias = torch.randn(W, generator=g)
    w = torch.randn(W, generator=g)
    gated = y.double() * torch.sigmoid(gate[:, W:].double() + bias.double())
    ref = x.double() + mult * pv.part_norm(gated, w.double(), parts, eps)
    out = torch.empty(N, W, dtype=torch.float32, device=DEV)
    core.gated_norm_add(x.to(DEV), y.to(DEV), gate.to(DEV)[:, W:], bias.to(DEV), w.to(DEV), parts, eps, mult, out)
    assert rel_err(out, ref) < 1e-5
    # without a gate, and in place
    ref = x.double() + mult * pv.part_norm(y.double(), w.double(), parts, eps)
    xd = x.to(DEV)
    core.gated_norm_add(xd, y.to(DEV), None, None, w.to(DEV), parts, eps, mult, xd)
    assert rel_err(xd, ref) < 1e-5
    # the norm of 32-bit rows returned in 32-bit (the normed embedding)
    o32 = torch.empty(N, W, dtype=torch.float32, device=DEV)
    core.part_rmsnorm(x.to(DEV), w.to(DEV), parts, eps, o32)
    assert rel_err(o32, pv.part_norm(x.double(), w.double(), parts, eps)) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,taps,add,off,pad", [(40, 3, True, 11, 3), (7, 1, True, 11, 3), (130, 4, False, 11, 3),
                                                (64, 2, False, 11, 3), (33, 5, True, 11, 3), (40, 3, True, 16, 8),
                                                (64, 4, False, 32, 0), (8, 1, True, 16, 8), (256, 5, True, 16, 24)])
def test_causal_convolution_over_steps_and_slots(dtype, C, taps, add, off, pad):
    """Two sequences cut differently and fed in the same steps, their states in slots that are
    not neighbours; portions shorter than the taps; a slot used again after it was zeroed.  ``off``
    floats lie before the state in a slot and rows are ``pad`` wider than the channels: with multiples
    of 8 everywhere the bfloat16 kernel takes eight channels a thread."""
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(C * taps)
    w = torch.randn(C, taps, generator=g)
    T = [37, 22]
    u = [torch.randn(t, C, generator=g).to(dtype) for t in T]
    ref = [pv.causal_conv(x.double(), w.double()) + (x.double() if add else 0) for x in u]
    state = torch.zeros(5, off + max(taps - 1, 1) * C, dtype=torch.float32, device=DEV)
    state[:, :off] = 7.0  # what lies before the offset is not the convolution's
    for attempt in range(2):
        cuts = [cuts_of(T[0], [5, 1, 2, 9, 1, 1, 3]), cuts_of(T[1], [1, 1, 6, 2])]
        got = [torch.zeros(t, C, dtype=dtype) for t in T]
        for i in range(max(len(c) for c in cuts)):
            live = [s for s in range(2) if i < len(cuts[s])]
            rows = [cuts[s][i][1] for s in live]
            step = Step(rows, [[3, 1][s] for s in live])
            x = torch.cat([u[s][cuts[s][i][0]: cuts[s][i][0] + cuts[s][i][1]] for s in live]).to(DEV)
            wide = torch.zeros(x.shape[0], C + pad, dtype=dtype, device=DEV)  # rows wider than the channels
            wide[:, :C] = x
            out = torch.empty(x.shape[0], C, dtype=dtype, device=DEV)
            core.causal_conv(wide[:, :C], w.to(DEV), state, off, step, out, add_input=add)
            core.conv_state_update(wide[:, :C], taps, state, off, step)
            at = 0
            for s, n in zip(live, rows):
                got[s][cuts[s][i][0]: cuts[s][i][0] + n] = out[at: at + n].cpu()
                at += n
        for s in range(2):
            assert rel_err(got[s], ref[s]) < PART_TOL[dtype], f"sequence {s}, attempt {attempt}"
        assert float(state[:, :off].min()) == 7.0 and float(state[[0, 2, 4]].abs()[:, off:].max()) == 0.0
        state[[1, 3], off:] = 0.0  # the slots are given to new requests


def build_pools(keys, values, page_size, dtype, seed):
    """Pools [pages, G, page_size, .] filled through block tables whose pages lie in no order.
    ``keys`` / ``values``: per request [T, G, .]."""
    rng = np.random.default_rng(seed)
    need = [-(-k.shape[0] // page_size) for k in keys]
    pages = sum(need) + 3
    order = rng.permutation(pages - 1).tolist()
    G, kw, vw = keys[0].shape[1], keys[0].shape[2], values[0].shape[2]
    k_pool = torch.full((pages, G, page_size, kw), float("nan"), dtype=dtype)
    v_pool = torch.full((pages, G, page_size, vw), float("nan"), dtype=dtype)
    tables = torch.full((len(keys), max(need)), -1, dtype=torch.int32)
    for r, (k, v) in enumerate(zip(keys, values)):
        for b in range(need[r]):
            page = order.pop()
            tables[r, b] = page
            n = min(page_size, k.shape[0] - b * page_size)
            k_pool[page, :, :n] = k[b * page_size: b * page_size + n].transpose(0, 1).to(dtype)
            v_pool[page, :, :n] = v[b * page_size: b * page_size + n].transpose(0, 1).to(dtype)
    return k_pool.to(DEV), v_pool.to(DEV), tables.to(DEV)


def plain_two_maps(q, k, v, scale, cap, lam, eps, out_scale):
    """q [T, H, 2, d], k [T, G, 2, d], v [T, G, e] of one sequence -> [T, H, e]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = []
    for a in range(H):
        g = a // (H // G)
        o = pv.causal_softmax_attention(q[:, a, 0], k[:, g, 0], v[:, g], scale, cap) \
            - lam * pv.causal_softmax_attention(q[:, a, 1], k[:, g, 1], v[:, g], scale, cap)
        out.append(pv.part_norm(o, None, 1, eps) * out_scale)
    return torch.stack(out, dim=1)


def check_two_maps(dtype, H, G, d, e, page, lens, rows, run, tol):
    """Queries at the ends of sequences of several lengths (the last ``rows`` of each are one step's
    entries); for each sequence's last query one key - far back, at a page's first or last place, the
    sequence's first token, the query's own - is scaled so that it alone carries the first map, another
    one the second.  ``run(q, k_pool, v_pool, out, step, tables, cap)`` is the kernel under test."""
    g = torch.Generator().manual_seed(H * d + e)
    scale, cap, lam, eps, out_scale = 0.3, 25.0, 0.37, 1e-5, 0.8
    ks = [torch.randn(t, G, 2, d, generator=g).to(dtype).double() for t in lens]
    vs = [torch.randn(t, G, e, generator=g).to(dtype).double() for t in lens]
    qs = [torch.randn(t, H, 2, d, generator=g).to(dtype).double() for t in lens]
    places = [0, -1, page - 1, page, None, 3, 0]
    for r, t in enumerate(lens):
        at = places[r % len(places)]
        first = (t // 2 if at is None else at) % t
        for m, j in ((0, first), (1, (t * 7 // 9) % t)):
            ks[r][j, :, m] = (ks[r][j, :, m] * 0 + qs[r][t - 1].mean(0)[m] * 6).to(dtype).double()  # q(t-1) . k(j) large
    k_pool, v_pool, tables = build_pools([k.reshape(k.shape[0], G, 2 * d) for k in ks], vs, page, dtype, seed=e)
    step = Step(rows, list(range(len(lens))), [t - n for t, n in zip(lens, rows)])
    q = torch.cat([qq[t - n:] for qq, t, n in zip(qs, lens, rows)]).reshape(-1, H * 2 * d).to(dtype).to(DEV)
    for use_cap in (cap, None):
        refs = [plain_two_maps(qq, k, v, scale, use_cap, lam, eps, out_scale) for qq, k, v in zip(qs, ks, vs)]
        ref = torch.cat([rf[t - n:] for rf, t, n in zip(refs, lens, rows)]).reshape(-1, H * e)
        out = torch.full((q.shape[0], H * e), float("nan"), dtype=dtype, device=DEV)
        run(q, k_pool, v_pool, out, step, tables, (scale, use_cap or 0.0, lam, eps, out_scale))
        assert torch.isfinite(out).all()
        assert rel_err(out, ref) < tol, f"cap {use_cap}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,page", [(4, 2, 16, 24, 4), (1, 1, 12, 12, 8), (6, 3, 8, 80, 16), (8, 1, 32, 64, 16),
                                          (2, 2, 64, 130, 32), (3, 1, 10, 300, 16)])
def test_two_score_maps_over_paged_keys_with_one_key_that_stands_out(dtype, H, G, d, e, page):
    from infernum_b200.ops import core
    rt = runtime(dtype)

    def run(q, k_pool, v_pool, out, step, tables, consts):
        core.attention_diff(q, k_pool, v_pool, out, step, tables, H, *consts, rt.err)

    lens = [1, 2, page, page + 1, 5 * page - 1, 301, 64]
    check_two_maps(dtype, H, G, d, e, page, lens, [min(t, 5) for t in lens], run, 2e-5 if dtype == torch.float32 else 3e-2)
    assert int(rt.err.item()) == 0


@pytest.mark.parametrize("H,G,d,e,page", [(4, 2, 16, 32, 4), (1, 1, 16, 16, 8), (6, 3, 16, 80, 16), (8, 1, 32, 64, 16),
                                          (8, 2, 128, 256, 16), (3, 1, 64, 128, 32), (16, 2, 48, 96, 16)])
def test_two_score_maps_on_the_tensor_cores(H, G, d, e, page):
    """The same through the tensor-core kernel: whole prompts that fill several row tiles, portions
    behind cached keys, single decoded rows far into a sequence, an entry without rows in the middle."""
    from infernum_b200.ops import attention_diff
    rt = runtime(torch.bfloat16)
    assert attention_diff.supported(d, e)

    def run(q, k_pool, v_pool, out, step, tables, consts):
        step.max_rows_per_entry = max(rows)
        assert attention_diff.run(q, k_pool, v_pool, out, step, tables, H, *consts, rt)

    lens = [1, 2, page, page + 1, 150, 301, 64, 97, 33]
    rows = [1, 2, 1, page + 1, 150, 1, 40, 0, 33]
    check_two_maps(torch.bfloat16, H, G, d, e, page, lens, rows, run, 3e-2)
    assert int(rt.err.item()) == 0
    # steps of few rows with the keys cut in slices over CTAs: slices that end inside a sequence, slices
    # behind a sequence's last key, a slice of one tile, as many slices as there are tiles
    lens = [1, 2, 33, 64, 301, 300, 97, 129]
    rows = [1, 2, 1, 3, 1, 2, 0, 1]
    for plan in ((2, 160, 0), (5, 64, 0), (10, 32, 0), (3, 128, 0)):
        rt.options["diff_splits"] = plan
        check_two_maps(torch.bfloat16, H, G, d, e, page, lens, rows, run, 3e-2)
    assert int(rt.err.item()) == 0
    # entries of at most 16 packed rows and values a multiple of 64 wide: the keys walked once, both maps'
    # sums side by side, in one slice and in several
    from infernum_b200.ops.attention_diff import one_walk
    rows = [1, 2, 1, 16 // (H // G), 1, min(2, 16 // (H // G)), 0, 1]
    if one_walk(max(rows), H // G, e):
        for plan in ((1, 320, 1), (2, 160, 1), (5, 64, 1), (10, 32, 1)):
            rt.options["diff_splits"] = plan
            check_two_maps(torch.bfloat16, H, G, d, e, page, lens, rows, run, 3e-2)
        assert int(rt.err.item()) == 0


def test_slices_of_the_keys_are_chosen_for_steps_of_few_rows():
    from infernum_b200.ops.attention_diff import choose_splits
    assert choose_splits(300, 1, 4, 2, 300, 148, 300, 8, 64) == (1, 0)  # a short prompt
    splits, slice_len = choose_splits(2048, 1, 4, 2, 2048, 148, 2048, 8, 256)  # a prompt whose last rows see many keys
    assert splits == 4 and slice_len == 512
    assert choose_splits(16384, 4, 4, 2, 16384, 148, 65536, 8, 256) == (1, 0)  # row tiles enough, shares too large
    assert choose_splits(1, 128, 4, 4, 1024, 148) == (1, 0)          # many decoded rows: CTAs enough
    assert choose_splits(1, 8, 4, 2, 100, 148) == (1, 0)             # few keys
    for entries, kv_heads, keys in ((1, 2, 1024), (8, 2, 1024), (1, 1, 9000), (3, 4, 300)):
        splits, slice_len = choose_splits(1, entries, 4, kv_heads, keys, 148)
        assert splits > 1 and slice_len % 32 == 0 and splits * slice_len >= keys > (splits - 1) * slice_len


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,taps,rd", [(4, 2, 16, 24, 4, 8), (1, 1, 12, 12, 0, 12), (3, 3, 10, 6, 1, 0),
                                            (2, 1, 8, 40, 5, 4), (4, 2, 48, 64, 3, 48)])
def test_convolution_rotation_and_cache_write_of_two_map_attention(dtype, H, G, d, e, taps, rd):
    """A sequence fed in portions: queries, and the keys and values found in the pages afterwards,
    against the convolution and the rotation of neighbouring pairs applied to the whole sequence."""
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(H + d + taps)
    T, page, mag = 45, 4, 1.07
    C = (H + G) * 2 * d + G * e
    x = torch.randn(T, C, generator=g).to(dtype)
    w = torch.randn(C, taps, generator=g) if taps else None
    y = pv.causal_conv(x.double(), w.double()) if taps else x.double()
    freqs = [50.0 ** (-2.0 * i / rd) for i in range(rd // 2)] if rd else []
    pos = torch.arange(T)
    q_ref = pv.rotate_pairs(y[:, : H * 2 * d].reshape(T, H * 2, d), pos, freqs, mag).reshape(T, -1)
    k_ref = pv.rotate_pairs(y[:, H * 2 * d: (H + G) * 2 * d].reshape(T, G * 2, d), pos, freqs, mag).reshape(T, G, 2 * d)
    v_ref = y[:, (H + G) * 2 * d:].reshape(T, G, e)
    pages = -(-T // page)
    k_pool = torch.zeros(pages + 2, G, page, 2 * d, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages + 2, G, page, e, dtype=dtype, device=DEV)
    tables = torch.tensor([[pages - b for b in range(pages)]], dtype=torch.int32, device=DEV)
    state = torch.zeros(3, max(taps - 1, 1) * C, dtype=torch.float32, device=DEV)
    inv = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(DEV) if rd else None
    rt = runtime(dtype)
    q_got = []
    for at, n in cuts_of(T, [6, 1, 2, 11, 3]):
        step = Step([n], [2], [at])
        q = torch.empty(n, H * 2 * d, dtype=dtype, device=DEV)
        xs = x[at: at + n].to(DEV)
        core.conv_rope_append(xs, w.to(DEV) if taps else None, state if taps > 1 else None, 0, inv, rd, mag, H, G, d, e,
                              step, tables, q, k_pool, v_pool, rt.err)
        if taps > 1:
            core.conv_state_update(xs, taps, state, 0, step)
        q_got.append(q.cpu())
    assert int(rt.err.item()) == 0
    tol = PART_TOL[dtype]
    assert rel_err(torch.cat(q_got), q_ref) < tol
    for t in range(T):
        pg = int(tables[0, t // page])
        assert rel_err(k_pool[pg, :, t % page], k_ref[t]) < tol, f"key {t}"
        assert rel_err(v_pool[pg, :, t % page], v_ref[t]) < tol, f"value {t}"


@pytest.mark.parametrize("E,I,top", [(6, 2, 2), (1, 0, 1), (3, 1, 4), (16, 2, 4), (40, 0, 6), (2, 3, 3)])
def test_routing_by_a_softmax_over_all_outputs(E, I, top):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(E * 10 + I)
    N, A = 50, E + I
    z = torch.randn(N, A + 1, generator=g) * 1.5
    z[7, : A] = 0.25  # all scores equal: the lowest indices win
    corr = torch.randn(A, generator=g) * 0.05
    corr_rows = torch.zeros(A) if A == 1 else corr
    w = {"m.router": torch.eye(A + 1, dtype=torch.float64)[:A], "m.correction": corr_rows.double()}
    ids_ref, wts_ref = pv.route(z.double(), {"top": top}, w, "m.")
    ids = torch.empty(N, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(N, top, dtype=torch.float32, device=DEV)
    gate = torch.empty(N, E, dtype=torch.float32, device=DEV)
    extra = torch.empty(N, 2, dtype=torch.float32, device=DEV)
    core.moe_route_softmax_all(z.to(DEV), corr_rows.to(DEV), A, E, top, ids, wts, gate, extra)
    assert (ids.cpu().long() == ids_ref).all()
    assert rel_err(wts, wts_ref) < 1e-5
    dense = torch.zeros(N, A, dtype=torch.float64)
    dense.scatter_(1, ids_ref, wts_ref)
    assert rel_err(gate, dense[:, :E]) < 1e-5
    assert (extra[:, 0].cpu().double() - dense[:, E:].sum(1)).abs().max() < 1e-5
    assert rel_err(extra[:, 1], torch.sigmoid(z[:, A].double())) < 1e-5
    # a dense row wider than the experts carries the extra column's gate in its further columns
    wide = torch.empty(N, E + 3, dtype=torch.float32, device=DEV)
    core.moe_route_softmax_all(z.to(DEV), corr_rows.to(DEV), A, E, top, ids, wts, wide, extra)
    assert torch.equal(wide[:, :E], gate) and torch.equal(wide[:, E:], extra[:, 1:2].expand(N, 3))
    # without the extra column there is no gate to take; without a correction equal scores meet
    core.moe_route_softmax_all(z[:, :A].contiguous().to(DEV), None, A, E, top, ids, wts, gate, extra)
    assert float((extra[:, 1] - 1).abs().max()) == 0.0
    ids_ref, _ = pv.route(z.double(), {"top": top}, {"m.router": w["m.router"]}, "m.")
    assert (ids.cpu().long() == ids_ref).all()
    assert ids[7].tolist() == list(range(top))
