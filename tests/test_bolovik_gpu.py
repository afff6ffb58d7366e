"""The Bolovik decoder on the GPU against the plain implementation
(``plain_bolovik``): each mechanism alone; whole prompts, token-by-token decoding,
portions down to two tokens, mixed batches with pages and state slots used again,
long decoding past every window; keys at window and page edges, among the kept
first tokens and far away, made to stand out; sizes that are 1 or equal; layers
without a feed-forward; greedy generation through the engine."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bolovik as pb
from bolovik_cases import CASES, PAGE_SIZES, make_folder, random_case
from helpers import (ROOT, TOL, compare_trace, peak_tokens, random_tokens, run_trace_inprocess,
                     run_trace_subprocess, trace_mixed, trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [31, 45, 1, 2, 90, 17], "B": [23, 60, 3, 1, 41, 8], "C": [130, 75, 2, 200, 33, 64],
           "D": [50, 3, 27, 1, 12], "E": [40, 2, 19, 66, 1], "F": [70, 33, 2, 1, 48]}
NAMES = ["A", "B", "C", "D", "E", "F", "Asharp", "Csharp"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CASES.items()):
        folder = make_folder(str(tmp_path_factory.mktemp(f"blv{name}")), cfg, seed=23 + i)
        out[name] = (folder, pb.Plain(folder))
        mild = make_folder(str(tmp_path_factory.mktemp(f"blvmild{name}")), cfg, seed=23 + i, gain=0.0)
        out[name + "/bfloat16"] = (mild, pb.Plain(mild))
        if name in ("A", "C"):
            sharp = make_folder(str(tmp_path_factory.mktemp(f"blvsharp{name}")), cfg, seed=53 + i, sharpen=6.0)
            out[name + "sharp"] = (sharp, pb.Plain(sharp))
    return out


def sequences(name):
    key = name.replace("sharp", "")
    return {f"r{i}": random_tokens(n, CASES[key]["vocab"], 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def pick(models, name, dtype):
    """The model of a case for a dtype: in bfloat16 the one whose projections are scaled up less.
    A decay's input of size 100 rounded to 8 bits is off by a half, which no engine can help."""
    return models.get(f"{name}/{dtype}", models[name])


def replay(models, name, dtype, steps, tmp_path, max_tokens=None):
    folder, plain = pick(models, name, dtype)
    out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"), max_tokens or peak_tokens(steps),
                              PAGE_SIZES[name.replace("sharp", "")])
    return out, plain


def names_for(dtype):
    # (where attention is peaked, bfloat16 rounding of a score is multiplied on its way to the logits)
    return NAMES if dtype == "float32" else ["A", "B", "C", "D", "E", "F"]


# In bfloat16 a router logit carries the rounding of everything before it; where the last chosen
# expert (or the last open group) lies within that of the best one left out, the engine may choose
# otherwise than the 64-bit plain implementation: a different, equally valid, result at that
# position.  Such positions (by the plain implementation's own margin) are not compared in bfloat16.
ROUTING_MARGIN = 0.03
# The test models' mixer projections and decay inputs are scaled up (so that a lost state or a
# wrong key shows); 32-bit rounding before a softplus or a unit norm is scaled with them.
F32_SLACK = 3
# Case A's norm parts have 32 elements and its heads 8: a bfloat16 rounding is averaged over few.
BF16_SLACK = {"A": 2}


def compare(steps, out, seqs, plain, dtype, name, slack=1):
    """float32: every position within the tolerance.  bfloat16: the positions whose routing is
    not a near-tie; the layers norm a sub-layer's result, which passes its rounding on undamped,
    and a position behind a differently routed one inherits a little of it through the mixers'
    states, so at most one position in ten may lie beyond the tolerance, the median at most half
    of it, and every value is finite."""
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
                if float(margins[pos]) < ROUTING_MARGIN:
                    skipped += 1
                    continue
                errs.append(float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6)))
            fed[rid] += n
        for rid in s.get("end", []):
            fed[rid] = 0
    assert len(errs) > skipped, f"{len(errs)} positions compared, {skipped} left out"
    errs = np.sort(np.array(errs))
    tol = TOL[dtype] * slack * BF16_SLACK.get(name, 1)
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
def test_most_in_one_step_then_token_by_token_past_the_windows(models, name, dtype, tmp_path):
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for rid, seq in seqs.items():
        steps += trace_tail(rid, seq, 70, step0=len(steps))  # longer than every window of the cases
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
@pytest.mark.parametrize("name", ["A", "Csharp"])
def test_long_decoding(models, name, dtype, tmp_path):
    if dtype == "bfloat16":
        name = name.replace("sharp", "")
    key = name.replace("sharp", "")
    seqs = {"long": random_tokens(230, CASES[key]["vocab"], 3)}
    steps = trace_tail("long", seqs["long"], tail=226)
    out, plain = replay(models, name, dtype, steps, tmp_path)
    compare(steps, out, seqs, plain, dtype, name)


@pytest.mark.parametrize("seed", [2, 3, 5, 8, 13, 21])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Sizes, orders and constants nobody chose by hand: mixed batches with pages and slots used again,
    then a long tail decoded token by token, in 32-bit against the plain implementation."""
    cfg = random_case(seed)
    folder = make_folder(str(tmp_path / "m"), cfg, seed=seed, gain=0.0)
    plain = pb.Plain(folder)
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], 31 * i + n) for i, n in enumerate([150, 70, 2, 19 + seed, 129, 1])}
    for rid, seq in seqs.items():
        # a router whose two candidates lie within 32-bit rounding of each other (scores that
        # saturate) may choose either: the sequence ends before such a token
        close = (plain.margins(seq) < 1e-4).nonzero().flatten().tolist()
        if close:
            seqs[rid] = seq[:max(close[0], 1)]
    steps = trace_mixed(seqs, max_live=4, seed=seed)
    if len(seqs["r0"]) > 3:
        steps += trace_tail("r0", seqs["r0"], 140, step0=len(steps))
    out = run_trace_inprocess(folder, "float32", steps, str(tmp_path / "out"), max(peak_tokens(steps), 256), 16)
    compare_trace(steps, out, seqs, plain, TOL["float32"] * F32_SLACK)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_and_batching_change_logits_by_rounding_only(models, dtype, tmp_path):
    folder, plain = pick(models, "C", dtype)
    seqs = sequences("C")
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


def test_the_stream_after_every_layer(models):
    """In 32-bit the stream after each layer (the depth average taken) equals the plain one closely."""
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.loading import load_model
    for name in ("A", "B", "C", "D"):
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
        _, want = pb.forward(plain.cfg, plain.weights, seq, return_layers=True)
        runner.step([StepEntry(cache.admit("x"), seq, [])])
        runner.check_errors()
        assert len(seen) == len(want)
        for i, (got, ref) in enumerate(zip(seen, want)):
            assert rel_err(got, ref) < 2e-5, f"case {name} layer {i}"


def test_the_program_itself_in_a_subprocess(models, tmp_path):
    seqs = {k: v for k, v in sequences("A").items() if len(v) > 3}
    steps = trace_mixed(seqs, max_live=3, seed=3)
    for dtype in DTYPES:
        folder, plain = pick(models, "A", dtype)
        out = run_trace_subprocess(folder, dtype, steps, str(tmp_path / dtype), peak_tokens(steps))
        compare(steps, out, seqs, plain, dtype, "A")


# ---- generation through the engine -----------------------------------------------------
def check_greedy(plain, prompt, got, dtype):
    """Every generated token is the plain implementation's best, or within rounding of it;
    after a near-tie the two may part, so the comparison follows what was generated.  In
    bfloat16 a step behind a near-tie of the routing is not held to the logits' gap."""
    seq = list(prompt)
    for i, tok in enumerate(got):
        logits = plain.logits(seq)[-1]
        best = pb.argmax(logits)
        if tok != best:
            gap = float((logits[best] - logits[tok]) / logits.abs().max())
            routed_close = dtype == "bfloat16" and float(plain.margins(seq).min()) < ROUTING_MARGIN
            assert gap < (1e-4 if dtype == "float32" else 5e-2) or routed_close, \
                f"token {i}: {tok} against {best}, gap {gap:.4f}"
        seq.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "Csharp"])
def test_greedy_generation_through_the_engine(models, name, dtype):
    import infernum_b200 as ib
    if name not in names_for(dtype):
        pytest.skip("peaked attention is compared in 32-bit")
    folder, plain = pick(models, name, dtype)
    key = name.replace("sharp", "")
    model = ib.load_model(folder, dtype=dtype)
    page = PAGE_SIZES[key]
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=3, block_size=page, num_blocks=480 // page,
                                             max_prefill_tokens=24))
    vocab = CASES[key]["vocab"]
    prompts = [random_tokens(n, vocab, 7 * n) for n in (5, 41, 18, 2, 30)]
    n_new = 50  # past the windows of the cases
    outs = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=n_new))
    for prompt, got in zip(prompts, outs):
        assert len(got) == n_new
        check_greedy(plain, prompt, got, dtype)
    # recurring steps ran from recordings: the mixers take entries, slots and positions from the device
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
    """``bin/generate`` picks the architecture by config.json: from a model folder, and from
    a bare configuration with random weights."""
    folder, plain = models["D"]
    prompt = random_tokens(9, CASES["D"]["vocab"], 1)
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
    """The device tensors of a step that the recurrent kernels read."""

    def __init__(self, rows_per_entry, slots):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        cu = [0]
        for n in rows_per_entry:
            cu.append(cu[-1] + n)
        self.n_entries = len(rows_per_entry)
        self.n_rows = cu[-1]
        self.cu_rows = i32(cu)
        self.slot_ids = i32(slots)
        self.row_entry = i32([e for e, n in enumerate(rows_per_entry) for _ in range(n)])


def cuts_of(T, sizes):
    out, at, i = [], 0, 0
    while at < T:
        n = min(sizes[i % len(sizes)], T - at)
        out.append((at, n))
        at += n
        i += 1
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,parts", [(96, 3), (72, 1), (320, 5), (64, 64), (1024, 4), (30, 2)])
def test_part_norm_of_a_result_added_to_the_stream_and_the_depth_average(dtype, W, parts):
    from infernum_b200.ops import core
    g = torch.Generator().manual_seed(W + parts)
    N, eps = 11, 3e-6
    x = torch.randn(N, W, generator=g) * 2
    y = (torch.randn(N, W, generator=g) * 5).to(dtype)
    # one part of one row is tiny beside eps: the eps sits inside the root
    y[3, : W // parts] = (y[3, : W // parts].float() * 1e-3).to(dtype)
    w = torch.randn(W, generator=g)
    ref = x.double() + pb.part_rms_norm(y.double(), w.double(), parts, eps)
    out = torch.empty(N, W, dtype=torch.float32, device=DEV)
    act = torch.empty(N, W, dtype=dtype, device=DEV) if dtype != torch.float32 else None
    core.sub_norm_add(x.to(DEV), y.to(DEV), w.to(DEV), parts, eps, out, act)
    assert rel_err(out, ref) < 1e-5
    if act is not None:
        assert rel_err(act, ref) < PART_TOL[dtype]
    # with earlier results: the sum is kept as result `slot`, the stream is the weighted sum of all
    for slot in (1, 2, 5):
        results = torch.randn(slot + 2, N, W, generator=g)
        coef = torch.randn(slot + 1, generator=g)
        res_dev = results.to(DEV)
        x_in = res_dev[0] if slot == 1 else x.to(DEV)
        base = results[0] if slot == 1 else x
        out = torch.empty(N, W, dtype=torch.float32, device=DEV)
        core.sub_norm_add(x_in, y.to(DEV), w.to(DEV), parts, eps, out, act, results=res_dev, slot=slot,
                          coef=coef.to(DEV))
        new = base.double() + pb.part_rms_norm(y.double(), w.double(), parts, eps)
        assert rel_err(res_dev[slot], new) < 1e-5
        assert torch.equal(res_dev[slot + 1].cpu(), results[slot + 1])  # the slot behind is not touched
        mixed = pb.depth_mix([results[j].double() for j in range(slot)] + [new], coef.double())
        assert rel_err(out, mixed) < 1e-5
        if act is not None:
            assert rel_err(act, mixed) < PART_TOL[dtype]
    # the norm alone, of chosen rows
    rows = torch.tensor([4, 0, 4, 10], dtype=torch.int32, device=DEV)
    xs = (torch.randn(N, W, generator=g) * 3)
    o = torch.empty(4, W, dtype=dtype, device=DEV)
    core.part_rmsnorm(xs.to(DEV), w.to(DEV), parts, eps, o, row_idx=rows)
    assert rel_err(o, pb.part_rms_norm(xs.double()[[4, 0, 4, 10]], w.double(), parts, eps)) < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_into_the_stream_and_its_rounding(dtype):
    from infernum_b200.ops import core
    table = torch.randn(37, 40).to(dtype).to(DEV)
    ids = torch.tensor([5, 0, 36, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 40, dtype=torch.float32, device=DEV)
    act = torch.empty(5, 40, dtype=dtype, device=DEV)
    err = core.new_error_word(DEV)
    core.embed_dual(ids, table, out, act, err)
    assert torch.equal(out, table[ids.long()].float()) and torch.equal(act, table[ids.long()])
    assert int(err.item()) == 0


def delta_reference(d, heads, kv_heads, dim, vdim, conv_w, a_log, dt_bias, off):
    """Outputs [T, heads * vdim] of one sequence from its projected rows, by the recurrence."""
    qk = kv_heads * dim
    C = 2 * qk + heads * vdim
    ch = d[:, off["c"]: off["c"] + C].double()
    if conv_w is not None:
        ch = pb.causal_conv(ch, conv_w.double())
    ch = pb.silu(ch)
    T = ch.shape[0]
    q = ch[:, :qk].reshape(T, kv_heads, dim)
    k = ch[:, qk: 2 * qk].reshape(T, kv_heads, dim)
    v = ch[:, 2 * qk:].reshape(T, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(d[:, off["b"]: off["b"] + heads].double())
    g = torch.exp(-torch.exp(a_log.double()) * pb.softplus(d[:, off["a"]: off["a"] + heads].double() + dt_bias.double()))
    per = heads // kv_heads
    return torch.cat([pb.delta_rule(q[:, a // per], k[:, a // per], v[:, a], beta[:, a], g[:, a])
                      for a in range(heads)], dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 16, 24, 4), (1, 1, 28, 10, 1), (3, 3, 12, 6, 0),
                                                           (2, 1, 128, 16, 3), (6, 2, 64, 32, 2), (2, 2, 8, 40, 7),
                                                           (4, 1, 32, 128, 4)])
def test_delta_scan_in_portions_and_batches_against_the_recurrence(dtype, heads, kv_heads, dim, vdim, taps):
    """Slow decays, so that what a token wrote still counts at the end; portions shorter than the
    convolution, whose last inputs are carried in the state; two requests side by side in slots
    that are not neighbours; then a slot that is used again."""
    from infernum_b200.ops import scan
    g = torch.Generator().manual_seed(heads * dim + vdim + taps)
    T = {"a": 75, "b": 22}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
    qk, inner = kv_heads * dim, heads * vdim
    C = 2 * qk + inner
    off = {"c": 3, "b": 3 + C + 5, "a": 3 + C + 5 + heads + 1}
    cols = off["a"] + heads + 2
    data = {}
    for r, n in T.items():
        d = rnd(n, cols) * 1.5
        d[:, off["b"]: off["b"] + heads] *= 2.0  # write strengths from weak to full
        data[r] = d.to(dtype)
    a_log, dt_bias = (rnd(heads) * 0.5 - 4.0).float(), (rnd(heads) * 0.5).float()
    conv_w = (rnd(C, taps) * 0.5).float() if taps else None
    ref = {r: delta_reference(data[r], heads, kv_heads, dim, vdim, conv_w, a_log, dt_bias, off) for r in T}
    # the first token still counts five portions later (small states forget by overwriting, however
    # slow the decay): without it that output differs clearly
    cut = delta_reference(data["a"][1:], heads, kv_heads, dim, vdim, conv_w, a_log, dt_bias, off)
    assert rel_err(cut[23], ref["a"][24]) > 1e-3
    rt = runtime(dtype)
    off_conv = heads * dim * vdim + 4
    state = torch.zeros(4, off_conv + max(taps - 1, 0) * C + 3, dtype=torch.float32, device=DEV)
    slot_of = {"a": 3, "b": 1}

    def run(plan, slots):
        got = {r: [] for r in plan}
        while any(plan.values()):
            live = [r for r in plan if plan[r]]
            cuts = [plan[r].pop(0) for r in live]
            rows = torch.cat([data[r][at: at + n] for r, (at, n) in zip(live, cuts)]).to(DEV)
            step = Step([n for _, n in cuts], [slots[r] for r in live])
            out = torch.full((step.n_rows, inner), float("nan"), dtype=torch.float32, device=DEV)
            scan.delta_scan(rows, off["c"], off["b"], off["a"], conv_w.to(DEV) if taps else None, a_log.to(DEV),
                            dt_bias.to(DEV), state, 0, off_conv, step, out, heads, kv_heads, dim, vdim, rt)
            at = 0
            for r, (_, n) in zip(live, cuts):
                got[r].append(out[at: at + n].cpu())
                at += n
        return {r: torch.cat(v) for r, v in got.items()}

    got = run({"a": cuts_of(T["a"], [2, 1, 16, 1, 3, 40]), "b": cuts_of(T["b"], [1, 1, 7, 20])}, slot_of)
    for r in T:
        assert rel_err(got[r], ref[r]) < 3e-5, r
    # the slots nobody had, the floats between the matrices and the convolution's inputs, and those behind them
    assert (state[0] == 0).all() and (state[2] == 0).all()
    assert (state[:, heads * dim * vdim: off_conv] == 0).all() and (state[:, -3:] == 0).all()
    # a request in a slot that another one left: its state starts from zero once the slot is cleared
    state[3].zero_()
    again = run({"b": cuts_of(T["b"], [22])}, {"b": 3})
    assert rel_err(again["b"], ref["b"]) < 3e-5
    # whole against token by token
    state.zero_()
    single = run({"a": cuts_of(T["a"], [1])}, slot_of)
    assert rel_err(single["a"], ref["a"]) < 3e-5
