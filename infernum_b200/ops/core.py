"""Python side of the ``core`` kernel module: argument checks and ctypes calls.

Every function here launches hand-written CUDA on the current stream of the
tensor's device.  There is no CPU or library fallback: a tensor that is not on
a CUDA device, or a missing/unbuildable extension, raises ``KernelError``.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_module
from ..errors import KernelError

CORE_SOURCES = ["elementwise.cu", "attention_plain.cu", "gemm_plain.cu", "sampling.cu", "layernorm.cu",
                "embed_hashed.cu", "latent.cu", "moe.cu", "hyper.cu", "recurrent.cu", "subnorm.cu", "shortconv.cu",
                "attention_diff.cu"]

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p
_c_ll = ctypes.c_longlong

FLAG_BAD_TOKEN = 1
FLAG_BAD_PAGE = 2
FLAG_WAIT_TIMEOUT = 4
# beside FLAG_WAIT_TIMEOUT, bit 8 + i says which wait gave up (common.cuh: IB_SITE_*)
TIMEOUT_SITES = ["product for few tokens: producer", "product for few tokens: MMA issuer",
                 "product for few tokens: epilogue", "product on SM pairs: producer",
                 "product on SM pairs: MMA issuer", "product on SM pairs: epilogue",
                 "prompt attention: producer", "prompt attention: MMA issuer", "prompt attention: softmax",
                 "prompt attention: shared memory window misplaced", "decode attention: producer",
                 "decode attention: computing warps"]


def describe_flags(flags: int) -> str:
    what = [name for bit, name in ((FLAG_BAD_TOKEN, "token id outside the vocabulary"),
                                   (FLAG_BAD_PAGE, "block-table entry outside the pool"),
                                   (FLAG_WAIT_TIMEOUT, "a device-side wait ran out")) if flags & bit]
    sites = [name for i, name in enumerate(TIMEOUT_SITES) if flags & (1 << (8 + i))]
    return "; ".join(what) + (" (" + ", ".join(sites) + ")" if sites else "")

_ERR_NAMES = {-1: "bad argument", -2: "unsupported configuration", -3: "size beyond the kernel's maximum",
              -4: "per-device set-up failed"}

_lib = None


def core_lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = load_module("core", CORE_SOURCES)
        lib.ib_wait_probe.argtypes = [_c_void_p, _c_ll, _c_int, _c_void_p]
        lib.ib_wait_probe.restype = _c_int
        lib.ib_step_fence.argtypes = [_c_void_p]
        lib.ib_step_fence.restype = _c_int
        lib.ib_embed.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                                 _c_void_p, _c_void_p]
        lib.ib_add_rmsnorm.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                       _c_void_p, _c_int, _c_int, _c_float, _c_int, _c_void_p]
        lib.ib_residual_add.argtypes = [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p]
        lib.ib_rope_append.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                       _c_void_p]
        lib.ib_silu_mul.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_attention_plain.argtypes = [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                           _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                           _c_float, _c_void_p, _c_void_p]
        lib.ib_gemm_plain.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                                      _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_argmax.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll,
                                  _c_void_p]
        lib.ib_sample.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                  _c_void_p, _c_void_p]
        lib.ib_decode_advance.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                          _c_void_p]
        lib.ib_feed_tokens.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p,
                                       _c_void_p]
        lib.ib_attention_plain_ex.argtypes = lib.ib_attention_plain.argtypes[:19] + [_c_int, _c_int, _c_int, _c_int,
                                                                                  _c_void_p, _c_void_p, _c_void_p]
        lib.ib_attention_plain_mask.argtypes = lib.ib_attention_plain.argtypes[:19] + [
            _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p]
        lib.ib_embed_dual.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                      _c_void_p, _c_void_p]
        lib.ib_sub_norm_add.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p, _c_int, _c_void_p,
                                        _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_part_rmsnorm.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int,
                                        _c_int, _c_void_p]
        lib.ib_delta_prepare.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p,
                                         _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                         _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_rope_norm_append.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                            _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        lib.ib_moe_route_scored.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p]
        for fn in ("ib_attention_plain_mask", "ib_embed_dual", "ib_sub_norm_add", "ib_part_rmsnorm", "ib_delta_prepare",
                   "ib_rope_norm_append", "ib_moe_route_scored"):
            getattr(lib, fn).restype = _c_int
        lib.ib_gemm_plain_batched.argtypes = [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_ll,
                                              _c_void_p, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int,
                                              _c_void_p]
        lib.ib_gated_act.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int,
                                     _c_void_p]
        lib.ib_scale_add_norm.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                          _c_void_p, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_void_p]
        lib.ib_softcap.argtypes = [_c_void_p, _c_ll, _c_float, _c_void_p]
        lib.ib_embed_hashed.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                        _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                        _c_ll, _c_ll, _c_ll, _c_void_p, _c_void_p]
        lib.ib_latent_prepare.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                                          _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                          _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        lib.ib_latent_q_rotate.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                                           _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_moe_route.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                     _c_int, _c_void_p]
        lib.ib_router_logits.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                                         _c_int, _c_void_p]
        lib.ib_router_logits.restype = _c_int
        lib.ib_hc_norm.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                   _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p]
        lib.ib_embed_sinusoid.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                                          _c_int, _c_int, _c_void_p, _c_void_p]
        lib.ib_scale_inplace.argtypes = [_c_void_p, _c_ll, _c_float, _c_void_p]
        lib.ib_token_shift.argtypes = [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p,
                                       _c_void_p, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_head_norm_gate.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                                          _c_int, _c_float, _c_void_p]
        lib.ib_gated_group_norm.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                                            _c_int, _c_float, _c_void_p]
        lib.ib_qk_norm_append.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p,
                                          _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                          _c_int, _c_int, _c_void_p, _c_void_p]
        lib.ib_ssd_prepare.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
                                       _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                       _c_void_p]
        lib.ib_wkv_prepare.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_ssd_prepare.restype = _c_int
        lib.ib_wkv_prepare.restype = _c_int
        lib.ib_pointwise.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float,
                                     _c_void_p]
        for fn in ("ib_hc_norm", "ib_embed_sinusoid", "ib_scale_inplace", "ib_token_shift",
                   "ib_head_norm_gate", "ib_gated_group_norm", "ib_qk_norm_append", "ib_pointwise"):
            getattr(lib, fn).restype = _c_int
        for fn in ("ib_attention_plain_ex", "ib_gemm_plain_batched", "ib_gated_act", "ib_scale_add_norm",
                   "ib_softcap", "ib_embed_hashed", "ib_latent_prepare", "ib_latent_q_rotate", "ib_moe_route"):
            getattr(lib, fn).restype = _c_int
        lib.ib_latent_prepare_ex.argtypes = lib.ib_latent_prepare.argtypes[:22] + [_c_int, _c_float, _c_void_p, _c_void_p]
        lib.ib_latent_q_rotate_ex.argtypes = lib.ib_latent_q_rotate.argtypes[:14] + [_c_int, _c_float, _c_void_p]
        lib.ib_moe_route_softmax_all.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                                 _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p]
        lib.ib_moe_combine.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                       _c_int, _c_void_p]
        lib.ib_gated_norm_add.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float,
                                          _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_concat_round.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_add_row.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p]
        lib.ib_causal_conv.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll, _c_void_p, _c_void_p,
                                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_conv_state_update.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_int,
                                             _c_int, _c_int, _c_void_p]
        lib.ib_conv_rope_append.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p,
                                            _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                            _c_float, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                            _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        lib.ib_attention_diff.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                          _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                          _c_float, _c_float, _c_float, _c_float, _c_float, _c_void_p, _c_void_p]
        for fn in ("ib_latent_prepare_ex", "ib_latent_q_rotate_ex", "ib_moe_route_softmax_all", "ib_moe_combine",
                   "ib_gated_norm_add", "ib_concat_round", "ib_add_row", "ib_causal_conv", "ib_conv_state_update",
                   "ib_conv_rope_append", "ib_attention_diff"):
            getattr(lib, fn).restype = _c_int
        for fn in ("ib_decode_advance", "ib_feed_tokens", "ib_embed", "ib_add_rmsnorm", "ib_residual_add", "ib_rope_append",
                   "ib_silu_mul", "ib_attention_plain", "ib_gemm_plain", "ib_argmax", "ib_sample"):
            getattr(lib, fn).restype = _c_int
        _lib = lib
    return _lib


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


_step_stream: Optional[int] = None  # the stream of the step being launched, looked up once per step


def stream_ptr(t: torch.Tensor) -> int:
    if _step_stream is not None:
        return _step_stream
    return torch.cuda.current_stream(t.device).cuda_stream


class step_stream:
    """While a model step is being launched, every kernel goes to the stream that
    was current at its start; looking it up for each launch costs as much as a
    small launch itself."""

    def __init__(self, device):
        self.device = device

    def __enter__(self):
        global _step_stream
        self.previous = _step_stream
        _step_stream = torch.cuda.current_stream(self.device).cuda_stream
        return self

    def __exit__(self, *exc):
        global _step_stream
        _step_stream = self.previous
        return False


LAUNCHES = 0  # kernels of this package launched so far (benchmarks report the count)

# ---------------------------------------------------------------------------
# INFERNUM_PROFILE=1: the device time of every operation, summed per operation
# and printed as a table when the process ends (the reference does this for its
# CPU executor: infernum-cpu/src/executor.rs:24-62).  A CUDA event is recorded
# before and behind every launch.  For the time between the two to be the
# operation's, the kernels must not overlap and must be launched one by one:
# in this mode programmatic dependent launch is off and the engine replays no
# recordings.  What the table shows is therefore not what a step costs in
# service, where kernels start under their predecessor's tail: it shows where
# the time goes.  A kernel that starts on an idle stream pays its launch
# (some 10 to 15 us between the two events even for the smallest kernel), and
# the first call of a library product pays the library's set-up: read the
# shares of the large operations here, and a kernel's own duration from
# ``ncu`` or ``python -m infernum_b200.cli.kernel_bench``.
# ---------------------------------------------------------------------------
PROFILE = os.environ.get("INFERNUM_PROFILE", "0") not in ("", "0")
_profile_marks: list = []  # (operation, event before, event after), in launch order
_profile_totals: dict = {}  # operation -> [calls, microseconds]
_profile_open = None  # the event before the operation being launched


def _profile_event():
    ev = torch.cuda.Event(enable_timing=True)
    ev.record(torch.cuda.current_stream() if _step_stream is None else torch.cuda.ExternalStream(_step_stream))
    return ev


def profile_begin() -> None:
    """The start of an operation (profile mode only): every wrapper passes here
    on its way in (``require_cuda``); ``profile_mark`` closes it."""
    global _profile_open
    if PROFILE and _profile_open is None:
        _profile_open = _profile_event()


def profile_mark(what: str) -> None:
    """The end of operation ``what`` on the current stream (profile mode only).
    Its time runs from ``profile_begin``, or from the end of the operation
    before it when one wrapper launches two kernels."""
    global _profile_open
    if not PROFILE:
        return
    after = _profile_event()
    before = _profile_open if _profile_open is not None else (_profile_marks[-1][2] if _profile_marks else after)
    _profile_open = None
    _profile_marks.append((what, before, after))
    if len(_profile_marks) >= 20000:
        profile_collect()


def profile_collect() -> dict:
    """Folds the marks so far into the totals and returns them: operation -> [calls, microseconds]."""
    if _profile_marks:
        torch.cuda.synchronize()
        for what, before, after in _profile_marks:
            row = _profile_totals.setdefault(what, [0, 0.0])
            row[0] += 1
            row[1] += before.elapsed_time(after) * 1000.0
        del _profile_marks[:]
    return _profile_totals


def profile_report(file=None) -> str:
    """The table of ``profile_collect``; printed to ``file`` when given."""
    totals = profile_collect()
    whole = sum(v[1] for v in totals.values()) or 1.0
    lines = [f"{'operation':28s} {'calls':>8s} {'total ms':>10s} {'mean us':>9s} {'share':>7s}"]
    for what, (calls, us) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{what:28s} {calls:8d} {us / 1000:10.2f} {us / max(calls, 1):9.2f} {100 * us / whole:6.1f}%")
    text = "\n".join(lines)
    if file is not None:
        print(text, file=file)
    return text


if PROFILE:
    import atexit
    import sys as _sys

    atexit.register(lambda: profile_report(_sys.stderr) if (_profile_marks or _profile_totals) else None)


def check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        if PROFILE:
            profile_mark(what)
        return
    if code < 0:
        raise KernelError(f"{what}: kernel refused its arguments ({_ERR_NAMES.get(code, code)})")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    if PROFILE:
        profile_begin()
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "infernum_b200 kernels run on a CUDA device only; got a tensor on "
                f"{t.device} (there is no CPU path)"
            )


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _int32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def new_error_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def wait_probe(err: torch.Tensor, limit_ms: float, site: int) -> None:
    """Runs a kernel whose one wait nothing ends: after ``limit_ms`` it sets the
    time-out flag with the bit of ``site`` in ``err`` and returns.  For testing
    that a wait that runs out is reported and leaves the device usable."""
    require_cuda(err)
    check(core_lib().ib_wait_probe(err.data_ptr(), int(limit_ms * 1e6), int(site), stream_ptr(err)),
          "wait_probe")


def step_fence(device) -> None:
    """The first launch of a step: an empty kernel launched the ordinary way, so
    that no kernel of the step starts before everything earlier in the stream -
    the copies and kernels that wrote the step's positions and tables - is
    complete (the package's other kernels start under their predecessor's tail
    and read those early)."""
    check(core_lib().ib_step_fence(torch.cuda.current_stream(device).cuda_stream), "step_fence")


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t, :] = table[ids[t], :] into a float32 residual stream."""
    require_cuda(ids, table, out, err)
    _int32(ids, "ids")
    n = ids.numel()
    V, H = table.shape
    if out.dtype != torch.float32 or out.shape != (n, H) or not out.is_contiguous():
        raise KernelError(f"embed: out must be contiguous float32 [{n}, {H}]")
    if not table.is_contiguous():
        raise KernelError("embed: table must be contiguous")
    check(core_lib().ib_embed(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                              out.data_ptr(), n, H, V, err.data_ptr(), stream_ptr(out)), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, row_idx: Optional[torch.Tensor] = None,
                write_residual: bool = True) -> None:
    """residual (+)= delta; out = rmsnorm(residual) * weight, in 32-bit.

    With ``row_idx`` only those rows are normed, ``out`` is compact and the
    residual is left as it was."""
    require_cuda(residual, delta, weight, out, row_idx)
    N, H = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("add_rmsnorm: residual must be contiguous float32")
    n_out = N if row_idx is None else row_idx.numel()
    _int32(row_idx, "row_idx")
    if row_idx is not None:
        write_residual = False
    if out.shape != (n_out, H) or not out.is_contiguous():
        raise KernelError(f"add_rmsnorm: out must be contiguous [{n_out}, {H}]")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype
                              or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and out's dtype")
    if weight.shape != (H,) or not weight.is_contiguous():
        raise KernelError(f"add_rmsnorm: weight must be [{H}]")
    check(core_lib().ib_add_rmsnorm(residual.data_ptr(), _ptr(delta), weight.data_ptr(),
                                    dtype_code(weight.dtype), out.data_ptr(),
                                    dtype_code(out.dtype), _ptr(row_idx), n_out, H, float(eps),
                                    1 if write_residual else 0, stream_ptr(out)), "add_rmsnorm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(residual, delta)
    if residual.dtype != torch.float32 or residual.shape != delta.shape \
            or not residual.is_contiguous() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes must match, residual float32, both contiguous")
    check(core_lib().ib_residual_add(residual.data_ptr(), delta.data_ptr(),
                                     dtype_code(delta.dtype), residual.numel(),
                                     stream_ptr(residual)), "residual_add")


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                rotary_dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                row_entry: Optional[torch.Tensor], block_tables: Optional[torch.Tensor],
                k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                err: torch.Tensor) -> None:
    """Rotate q and k of ``qkv`` in place; with pools, store k and v in the pages."""
    require_cuda(qkv, positions, inv_freq, row_entry, block_tables, k_pool, v_pool, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    N = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("rope_append: qkv must be 2-D with unit inner stride")
    write_kv = k_pool is not None
    page_size = num_pages = max_blocks = 0
    if write_kv:
        if k_pool.shape != v_pool.shape or k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype \
                or not k_pool.is_contiguous() or not v_pool.is_contiguous():
            raise KernelError("rope_append: pools must be contiguous, alike and of qkv's dtype")
        num_pages, nkv_pool, page_size, hd_pool = k_pool.shape
        if nkv_pool != n_kv_heads or hd_pool != head_dim:
            raise KernelError("rope_append: pool shape does not match the head counts")
        max_blocks = block_tables.shape[1]
    need = (n_heads + (2 * n_kv_heads if write_kv else n_kv_heads)) * head_dim
    if qkv.shape[1] < need:
        raise KernelError(f"rope_append: qkv rows hold {qkv.shape[1]} values, need {need}")
    if rotary_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32
                           or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_append: inv_freq must be float32 [rotary_dim / 2]")
    check(core_lib().ib_rope_append(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0),
                                    positions.data_ptr(), _ptr(row_entry), _ptr(block_tables),
                                    max_blocks, _ptr(inv_freq), _ptr(k_pool), _ptr(v_pool), N,
                                    n_heads, n_kv_heads, head_dim, rotary_dim, page_size,
                                    num_pages, 1 if write_kv else 0, err.data_ptr(),
                                    stream_ptr(qkv)), "rope_append")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: Optional[int] = None) -> None:
    """out = silu(gate) * up for rows [N, 2I].  ``block`` says where gates and
    ups sit in a row: None for [all gates | all ups], else pieces of ``block``
    gates followed by their ``block`` ups."""
    require_cuda(gate_up, out)
    N, two_i = gate_up.shape
    if two_i % 2 or out.shape != (N, two_i // 2) or out.dtype != gate_up.dtype \
            or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("silu_mul: gate_up [N, 2I] and out [N, I] must be contiguous, same dtype")
    I = two_i // 2
    blk = I if block is None else int(block)
    if blk <= 0 or I % blk:
        raise KernelError(f"silu_mul: block {blk} does not divide the width {I}")
    check(core_lib().ib_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), N, I,
                                 blk, stream_ptr(out)), "silu_mul")


def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    out: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor,
                    block_tables: torch.Tensor, n_heads: int, scale: float, window: int,
                    err: torch.Tensor, sink: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Causal attention of each row over its request's pages (32-bit arithmetic).

    ``q`` is [N, >= n_heads*hd] (a view into the qkv rows is fine), ``out`` is
    [N, n_heads*hdv]; the key pool is [pages, kv_heads, page_size, hd], the value
    pool the same with rows of hdv values (hdv may differ from hd).  ``sink``
    (float32 [n_heads]): a logit per head that is added to the softmax's
    denominator as exp(sink), with no key and no value behind it.
    ``keep_first``: behind a window, the keys at positions below it stay visible."""
    require_cuda(q, k_pool, v_pool, out, positions, row_entry, block_tables, err, sink)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    num_pages, nkv, page_size, hd = k_pool.shape
    hdv = v_pool.shape[3]
    N = q.shape[0]
    if v_pool.shape[:3] != k_pool.shape[:3] or not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention_plain: the pools must be contiguous and alike but for the value size")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < n_heads * hd \
            or out.shape[1] < n_heads * hdv:
        raise KernelError("attention_plain: q/out rows are too short or not unit-stride")
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("attention_plain: q, pools and out must share a dtype")
    if n_heads % nkv:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {nkv} kv heads")
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (n_heads,) or not sink.is_contiguous()):
        raise KernelError(f"attention_plain: sink must be contiguous float32 [{n_heads}]")
    if sink is not None or keep_first > 0 or hdv != hd:
        check(core_lib().ib_attention_plain_mask(q.data_ptr(), q.stride(0), k_pool.data_ptr(), v_pool.data_ptr(),
                                                 out.data_ptr(), out.stride(0), dtype_code(q.dtype),
                                                 positions.data_ptr(), row_entry.data_ptr(), block_tables.data_ptr(),
                                                 block_tables.shape[1], N, n_heads, nkv, hd, page_size, num_pages,
                                                 int(window), float(scale), hdv, hdv, hd, hdv, _ptr(sink),
                                                 int(keep_first), err.data_ptr(), stream_ptr(q)), "attention_plain")
        return
    check(core_lib().ib_attention_plain(q.data_ptr(), q.stride(0), k_pool.data_ptr(),
                                        v_pool.data_ptr(), out.data_ptr(), out.stride(0),
                                        dtype_code(q.dtype), positions.data_ptr(),
                                        row_entry.data_ptr(), block_tables.data_ptr(),
                                        block_tables.shape[1], N, n_heads, nkv, hd, page_size,
                                        num_pages, int(window), float(scale), err.data_ptr(),
                                        stream_ptr(q)), "attention_plain")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit fused multiply-adds in k order."""
    require_cuda(a, w, out)
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape != (M, N):
        raise KernelError(f"gemm_plain: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_plain: inner strides must be 1")
    check(core_lib().ib_gemm_plain(a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(),
                                   dtype_code(w.dtype), w.stride(0), out.data_ptr(),
                                   dtype_code(out.dtype), out.stride(0), M, N, K,
                                   stream_ptr(out)), "gemm_plain")


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """Greedy selection per row: the largest logit, the lowest index among equals."""
    require_cuda(logits, out)
    _int32(out, "out")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.numel() != R:
        raise KernelError("argmax: logits must be float32 [R, V], out int32 [R]")
    scratch_ptr, scratch_bytes = None, 0
    if V >= 16384:
        # partial results of the sliced kernel: 64 (value, index) pairs per row
        key = (logits.device, R)
        buf = _argmax_scratch.get(key)
        if buf is None:
            buf = torch.empty(R * 64 * 2, dtype=torch.int32, device=logits.device)
            _argmax_scratch[key] = buf
        scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel() * 4
    check(core_lib().ib_argmax(logits.data_ptr(), logits.stride(0), R, V, out.data_ptr(),
                               scratch_ptr, scratch_bytes, stream_ptr(logits)), "argmax")


SAMPLE_PARAM_FLOATS = 6  # temperature, top_p, penalty, u, n_recent (int bits), pad


def sample(logits: torch.Tensor, params: torch.Tensor, recent: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Temperature / nucleus / repetition-penalty sampling; ``params`` is a
    [R, 6] float32 tensor (see ``pack_sample_params``).  Logits are modified in
    place by the penalty."""
    require_cuda(logits, params, recent, out)
    _int32(out, "out")
    _int32(recent, "recent")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    if params.dtype != torch.float32 or params.shape != (R, SAMPLE_PARAM_FLOATS) \
            or not params.is_contiguous():
        raise KernelError("sample: params must be contiguous float32 [R, 6]")
    recent_ld = 0 if recent is None else recent.shape[1]
    check(core_lib().ib_sample(logits.data_ptr(), logits.stride(0), R, V, params.data_ptr(),
                               _ptr(recent), recent_ld, out.data_ptr(), stream_ptr(logits)),
          "sample")


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, selected: torch.Tensor,
                recent: Optional[torch.Tensor] = None, recent_pos: Optional[torch.Tensor] = None) -> None:
    """tokens[i] = selected[src[i]] where src[i] >= 0 (other rows keep theirs): the
    inputs of a step launched behind the step whose selection ``selected`` is.
    With ``recent`` [rows, width] and ``recent_pos`` [rows], the same token is
    also written to ``recent[i, recent_pos[i]]`` where that place is not
    negative (the row's recent tokens, for its repetition penalty)."""
    require_cuda(tokens, src, selected, recent, recent_pos)
    for t, name in ((tokens, "tokens"), (src, "src"), (selected, "selected"), (recent, "recent"),
                    (recent_pos, "recent_pos")):
        _int32(t, name)
    if src.numel() < tokens.numel():
        raise KernelError("feed_tokens: fewer sources than tokens")
    if recent is not None and (recent_pos is None or recent.dim() != 2 or recent.shape[0] < tokens.numel()
                               or recent_pos.numel() < tokens.numel()):
        raise KernelError("feed_tokens: the recent tokens need a row and a place per token")
    check(core_lib().ib_feed_tokens(tokens.data_ptr(), src.data_ptr(), selected.data_ptr(), selected.numel(),
                                    tokens.numel(), _ptr(recent), recent.shape[1] if recent is not None else 0,
                                    _ptr(recent_pos), stream_ptr(tokens)), "feed_tokens")


def decode_advance(tokens: torch.Tensor, selected: Optional[torch.Tensor], positions: torch.Tensor,
                   kv_len: torch.Tensor, slot_ids: Optional[torch.Tensor] = None, pad_slot: int = -1) -> None:
    """positions += 1, kv_len += 1, and tokens = selected when given; rows whose
    slot is ``pad_slot`` (they only fill up a batch bucket) are left alone."""
    require_cuda(tokens, selected, positions, kv_len, slot_ids)
    for t, name in ((tokens, "tokens"), (selected, "selected"), (positions, "positions"), (kv_len, "kv_len"),
                    (slot_ids, "slot_ids")):
        _int32(t, name)
    check(core_lib().ib_decode_advance(tokens.data_ptr(), _ptr(selected), positions.data_ptr(),
                                       kv_len.data_ptr(), _ptr(slot_ids), int(pad_slot), tokens.numel(),
                                       stream_ptr(tokens)),
          "decode_advance")


# ---------------------------------------------------------------------------
# Parts that several designs share beyond the Llama decoder: a norm of a scaled
# sum (post-norm layers, layer norm with bias), gated activations other than
# SiLU, a soft cap on logits, a hashed bigram embedding, attention over a latent
# cache, batched per-head products, and the routing of a mixture of experts.
# ---------------------------------------------------------------------------
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def scale_add_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                   bias: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor], alpha: float = 1.0,
                   centred: bool = True, store: bool = False, row_idx: Optional[torch.Tensor] = None) -> None:
    """y = norm(alpha * residual + delta) * weight + bias in 32-bit; ``centred``
    takes the mean off first (layer norm), else it is an RMS norm.  ``store``
    writes y over the float32 residual; ``out`` receives it in the activation
    dtype (compact when ``row_idx`` selects rows)."""
    require_cuda(residual, delta, weight, bias, out, row_idx)
    N, H = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("scale_add_norm: residual must be contiguous float32")
    _int32(row_idx, "row_idx")
    n_out = N if row_idx is None else row_idx.numel()
    if out is not None and (out.shape != (n_out, H) or not out.is_contiguous()):
        raise KernelError(f"scale_add_norm: out must be contiguous [{n_out}, {H}]")
    if out is None and not store:
        raise KernelError("scale_add_norm: nothing to write")
    act = out.dtype if out is not None else (delta.dtype if delta is not None else torch.float32)
    if delta is not None and (delta.shape != residual.shape or delta.dtype != act or not delta.is_contiguous()):
        raise KernelError("scale_add_norm: delta must match the residual's shape and the activation dtype")
    if weight.shape != (H,) or not weight.is_contiguous() or (
            bias is not None and (bias.shape != (H,) or bias.dtype != weight.dtype or not bias.is_contiguous())):
        raise KernelError(f"scale_add_norm: weight and bias must be [{H}] of one dtype")
    check(core_lib().ib_scale_add_norm(residual.data_ptr(), _ptr(delta), weight.data_ptr(), _ptr(bias),
                                       dtype_code(weight.dtype), _ptr(out), dtype_code(act), _ptr(row_idx), n_out,
                                       H, float(eps), float(alpha), 1 if centred else 0, 1 if store else 0,
                                       stream_ptr(residual)), "scale_add_norm")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    require_cuda(logits)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("softcap: logits must be contiguous float32")
    check(core_lib().ib_softcap(logits.data_ptr(), logits.numel(), float(cap), stream_ptr(logits)), "softcap")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", block: Optional[int] = None,
              scale: Optional[torch.Tensor] = None, cols_per_scale: int = 0) -> None:
    """out = act(gate) * up for rows [N, 2I] (``block`` as in ``silu_mul``); with
    ``scale`` [N, I / cols_per_scale] (float32) each run of ``cols_per_scale``
    outputs is multiplied by its scale."""
    require_cuda(gate_up, out, scale)
    N, two_i = gate_up.shape
    if two_i % 2 or out.shape != (N, two_i // 2) or out.dtype != gate_up.dtype \
            or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("gated_act: gate_up [N, 2I] and out [N, I] must be contiguous, same dtype")
    I = two_i // 2
    blk = I if block is None else int(block)
    if blk <= 0 or I % blk:
        raise KernelError(f"gated_act: block {blk} does not divide the width {I}")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
    if scale is not None and (scale.dtype != torch.float32 or not scale.is_contiguous() or cols_per_scale <= 0
                              or I % cols_per_scale or scale.shape != (N, I // cols_per_scale)):
        raise KernelError("gated_act: scale must be contiguous float32 [N, I / cols_per_scale]")
    check(core_lib().ib_gated_act(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), N, I, blk,
                                  ACTIVATIONS[activation], _ptr(scale), int(cols_per_scale), stream_ptr(out)),
          "gated_act")


def embed_hashed(ctx, prev_state: torch.Tensor, table: torch.Tensor, bigram: torch.Tensor, buckets: int,
                 mul_prev: int, mul_cur: int, out: torch.Tensor, out_act: Optional[torch.Tensor],
                 err: torch.Tensor) -> None:
    """out[t] = table[id_t] + bigram[hash(id_{t-1}, id_t)] (row ``buckets`` for a
    sequence's first token); ``prev_state`` [slots] int32 carries each request's
    last token from step to step."""
    ids = ctx.token_ids
    require_cuda(ids, prev_state, table, bigram, out, out_act, err)
    _int32(ids, "ids")
    _int32(prev_state, "prev_state")
    n = ids.numel()
    V, H = table.shape
    if bigram.shape != (buckets + 1, H) or bigram.dtype != table.dtype or not bigram.is_contiguous() \
            or not table.is_contiguous():
        raise KernelError(f"embed_hashed: the bigram table must be [{buckets + 1}, {H}] of the table's dtype")
    if out.dtype != torch.float32 or out.shape != (n, H) or not out.is_contiguous():
        raise KernelError(f"embed_hashed: out must be contiguous float32 [{n}, {H}]")
    if out_act is not None and (out_act.dtype != torch.bfloat16 or out_act.shape != (n, H)
                                or not out_act.is_contiguous()):
        raise KernelError("embed_hashed: the activation copy must be contiguous bfloat16")
    check(core_lib().ib_embed_hashed(ids.data_ptr(), ctx.positions.data_ptr(), ctx.row_entry.data_ptr(),
                                     ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(), prev_state.data_ptr(),
                                     prev_state.numel(), table.data_ptr(), bigram.data_ptr(),
                                     dtype_code(table.dtype), out.data_ptr(), _ptr(out_act), n, H, V, int(buckets),
                                     int(mul_prev), int(mul_cur), err.data_ptr(), stream_ptr(out)), "embed_hashed")


def latent_prepare(lat: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, rotary_dim: int,
                   wq: Optional[torch.Tensor], wkv: Optional[torch.Tensor], eps: float,
                   inv_freq: Optional[torch.Tensor], positions: torch.Tensor, row_entry: torch.Tensor,
                   block_tables: Optional[torch.Tensor], cq_out: Optional[torch.Tensor],
                   pool: Optional[torch.Tensor], err: torch.Tensor, adjacent: bool = False,
                   magnitude: float = 1.0) -> None:
    """From the down projections ``lat`` [N, q_rank + kv_rank + rot_dim] (float32 or
    the activation dtype; the norms and the rotation are 32-bit either way):
    the normed query latent into ``cq_out``, and - with ``pool`` - the normed
    key/value latent and the rotated shared key part into the token's place in
    the pool [pages, 1, page_size, kv_rank + rot_dim].  ``adjacent``: the rotation
    pairs neighbours (2i, 2i + 1) instead of (i, i + rotary_dim / 2); ``magnitude``
    multiplies cosine and sine."""
    require_cuda(lat, wq, wkv, inv_freq, positions, row_entry, block_tables, cq_out, pool, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    write_kv = pool is not None
    if lat.dim() != 2 or lat.stride(1) != 1:
        raise KernelError("latent_prepare: the down projections must be rows with unit inner stride")
    act = cq_out.dtype if cq_out is not None else pool.dtype
    for t, n, name in ((wq, q_rank, "query"), (wkv if write_kv else None, kv_rank, "key/value")):
        if t is not None and (t.shape != (n,) or t.dtype != act or not t.is_contiguous()):
            raise KernelError(f"latent_prepare: the {name} norm weight must be [{n}] in the activation dtype")
    if q_rank and (cq_out is None or cq_out.shape != (lat.shape[0], q_rank) or not cq_out.is_contiguous()):
        raise KernelError("latent_prepare: cq_out must be contiguous [N, q_rank]")
    page_size = num_pages = max_blocks = 0
    if write_kv:
        if pool.dim() != 4 or pool.shape[1] != 1 or pool.shape[3] != kv_rank + rot_dim or pool.dtype != act \
                or not pool.is_contiguous():
            raise KernelError("latent_prepare: the pool must be contiguous [pages, 1, page_size, kv_rank + rot_dim]")
        num_pages, _, page_size, _ = pool.shape
        max_blocks = block_tables.shape[1]
        if rotary_dim and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
            raise KernelError("latent_prepare: inv_freq must be float32 [rotary_dim / 2]")
    check(core_lib().ib_latent_prepare_ex(lat.data_ptr(), dtype_code(lat.dtype), lat.stride(0), int(q_rank), int(kv_rank), int(rot_dim),
                                       int(rotary_dim), _ptr(wq), _ptr(wkv), float(eps), _ptr(inv_freq),
                                       positions.data_ptr(), row_entry.data_ptr(), _ptr(block_tables), max_blocks,
                                       _ptr(cq_out), _ptr(pool), dtype_code(act), page_size, num_pages,
                                       1 if write_kv else 0, lat.shape[0], 1 if adjacent else 0, float(magnitude),
                                       err.data_ptr(), stream_ptr(lat)),
          "latent_prepare")


def latent_q_rotate(q: torch.Tensor, heads: int, dim: int, rot_dim: int, rotary_dim: int,
                    inv_freq: Optional[torch.Tensor], positions: torch.Tensor, q_abs: torch.Tensor,
                    offset: int, adjacent: bool = False, magnitude: float = 1.0) -> None:
    """The rotated part of each head of ``q`` [N, heads * (dim + rot_dim)], rotated
    by its row's position, into ``q_abs[N, heads, offset : offset + rot_dim]``."""
    require_cuda(q, inv_freq, positions, q_abs)
    _int32(positions, "positions")
    if q.dim() != 2 or q.stride(1) != 1 or q_abs.dim() != 3 or q_abs.stride(2) != 1 or q_abs.dtype != q.dtype \
            or q_abs.shape[0] != q.shape[0] or q_abs.shape[1] != heads or q_abs.shape[2] < offset + rot_dim:
        raise KernelError("latent_q_rotate: q [N, heads*(dim+rot)] and q_abs [N, heads, >= offset+rot] do not fit")
    check(core_lib().ib_latent_q_rotate_ex(q.data_ptr(), q.stride(0), int(heads), int(dim), int(rot_dim),
                                        int(rotary_dim), _ptr(inv_freq), positions.data_ptr(), q_abs.data_ptr(),
                                        q_abs.stride(0), q_abs.stride(1), int(offset), dtype_code(q.dtype),
                                        q.shape[0], 1 if adjacent else 0, float(magnitude), stream_ptr(q)),
          "latent_q_rotate")


def attention_latent_plain(q_abs: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, kv_rank: int,
                           positions: torch.Tensor, row_entry: torch.Tensor, block_tables: torch.Tensor,
                           scale: float, window: int, err: torch.Tensor) -> None:
    """Attention of all heads over one latent cache, in 32-bit: ``q_abs``
    [N, heads, width] holds each head's query in latent space followed by its
    rotated part, the pool [pages, 1, page_size, width] each token's latent
    followed by the shared rotated key; a token's value is its latent.  ``out``
    [N, heads, kv_rank]."""
    require_cuda(q_abs, pool, out, positions, row_entry, block_tables, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    num_pages, one, page_size, width = pool.shape
    N, heads, qw = q_abs.shape
    if one != 1 or qw != width or q_abs.stride(2) != 1 or out.stride(2) != 1 or out.shape != (N, heads, kv_rank) \
            or not (q_abs.dtype == pool.dtype == out.dtype) or not pool.is_contiguous():
        raise KernelError("attention_latent_plain: q_abs [N, heads, width], pool [pages, 1, page, width] and "
                          "out [N, heads, kv_rank] do not fit")
    check(core_lib().ib_attention_plain_ex(q_abs.data_ptr(), q_abs.stride(0), pool.data_ptr(), pool.data_ptr(),
                                           out.data_ptr(), out.stride(0), dtype_code(q_abs.dtype),
                                           positions.data_ptr(), row_entry.data_ptr(), block_tables.data_ptr(),
                                           block_tables.shape[1], N, heads, 1, width, page_size, num_pages,
                                           int(window), float(scale), int(kv_rank), width, q_abs.stride(1),
                                           out.stride(1), None, err.data_ptr(), stream_ptr(q_abs)),
          "attention_latent_plain")


def gemm_plain_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b, M, N] = a[b, M, K] @ w[b, N, K]^T member by member with the plain
    kernel's arithmetic.  Any batch and row strides (views of heads that lie
    side by side in a row are fine); inner strides 1."""
    require_cuda(a, w, out)
    B, M, K = a.shape
    if w.dim() != 3 or w.shape[0] != B or w.shape[2] != K or out.shape != (B, M, w.shape[1]):
        raise KernelError(f"gemm_plain_batched: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if a.stride(2) != 1 or w.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("gemm_plain_batched: inner strides must be 1")
    check(core_lib().ib_gemm_plain_batched(a.data_ptr(), dtype_code(a.dtype), a.stride(1), a.stride(0),
                                           w.data_ptr(), dtype_code(w.dtype), w.stride(1), w.stride(0),
                                           out.data_ptr(), dtype_code(out.dtype), out.stride(1), out.stride(0),
                                           B, M, w.shape[1], K, stream_ptr(out)), "gemm_plain_batched")


def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor,
              weights: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """The ``top`` largest of ``logits + bias`` per row (float32) with the softmax
    over those: ``ids`` / ``weights`` [N, top], and ``gate`` [N, E] dense."""
    require_cuda(logits, bias, ids, weights, gate)
    _int32(ids, "ids")
    N, E = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or ids.shape != (N, top) \
            or weights.shape != (N, top) or weights.dtype != torch.float32 or not weights.is_contiguous():
        raise KernelError("moe_route: logits float32 [N, E], ids int32 [N, top], weights float32 [N, top]")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (E,) or not bias.is_contiguous()):
        raise KernelError("moe_route: the bias must be float32 [E]")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != (N, E) or not gate.is_contiguous()):
        raise KernelError("moe_route: gate must be contiguous float32 [N, E]")
    check(core_lib().ib_moe_route(logits.data_ptr(), logits.stride(0), _ptr(bias), E, int(top), ids.data_ptr(),
                                  weights.data_ptr(), _ptr(gate), N, stream_ptr(logits)), "moe_route")


def router_logits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, e] = sum_k x[n, k] w[e, k] in 32-bit, for a handful of experts: one
    warp per (row, expert), a fixed order of additions."""
    require_cuda(x, w, out)
    N, K = x.shape
    E = w.shape[0]
    if w.shape[1] != K or out.shape != (N, E) or out.dtype != torch.float32 or not out.is_contiguous() \
            or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("router_logits: x [N, K], w [E, K] with unit inner strides, out contiguous float32 [N, E]")
    check(core_lib().ib_router_logits(x.data_ptr(), dtype_code(x.dtype), x.stride(0), w.data_ptr(),
                                      dtype_code(w.dtype), w.stride(0), out.data_ptr(), N, E, K, stream_ptr(out)),
          "router_logits")


# ---------------------------------------------------------------------------
# Several residual streams per token, a sinusoidal position vector on the
# embedding, recurrent mixers (token shift, causal convolution, the norms and
# gates behind their scans) and attention with normed queries and keys.
# ---------------------------------------------------------------------------
def _f32_vec(t: Optional[torch.Tensor], n: int, name: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise KernelError(f"{name} must be contiguous float32 with {n} values")


def hc_norm(x: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor],
            out_coef: Optional[torch.Tensor], read: Optional[torch.Tensor], weight: Optional[torch.Tensor],
            bias: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor], centred: bool = True,
            row_idx: Optional[torch.Tensor] = None) -> None:
    """Streams ``x`` [N, S, H] (float32): with ``y`` [N, H] the write of a
    sub-layer, ``x_t <- sum_s mix[s, t] x_s + out_coef[t] y``; with ``out`` the
    read ``u = sum_s read[s] x_s`` (``read`` None: the plain sum) and its norm
    with ``weight`` and ``bias`` into ``out``.  One pass, 32-bit.  With
    ``row_idx`` only those rows are read, ``out`` is compact and nothing is
    written back."""
    require_cuda(x, y, mix, out_coef, read, weight, bias, out, row_idx)
    if x.dim() != 3 or x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("hc_norm: the streams must be contiguous float32 [N, S, H]")
    N, S, H = x.shape
    _int32(row_idx, "row_idx")
    n_out = N if row_idx is None else row_idx.numel()
    _f32_vec(mix, S * S, "hc_norm: mix")
    _f32_vec(out_coef, S, "hc_norm: out_coef")
    _f32_vec(read, S, "hc_norm: read")
    if y is not None and (y.shape != (N, H) or not y.is_contiguous() or mix is None or out_coef is None):
        raise KernelError("hc_norm: y must be contiguous [N, H] and comes with mix and out_coef")
    if out is not None and (out.shape != (n_out, H) or not out.is_contiguous() or weight is None
                            or weight.shape != (H,) or not weight.is_contiguous()
                            or (bias is not None and (bias.shape != (H,) or bias.dtype != weight.dtype
                                                      or not bias.is_contiguous()))):
        raise KernelError(f"hc_norm: out must be contiguous [{n_out}, {H}], weight and bias [{H}] of one dtype")
    if y is not None and out is not None and y.dtype != out.dtype:
        raise KernelError("hc_norm: y and out share the activation dtype")
    act = out.dtype if out is not None else (y.dtype if y is not None else torch.float32)
    check(core_lib().ib_hc_norm(x.data_ptr(), _ptr(y), _ptr(mix), _ptr(out_coef), _ptr(read), _ptr(weight),
                                _ptr(bias), dtype_code(weight.dtype) if weight is not None else 0, _ptr(out),
                                dtype_code(act), _ptr(row_idx), n_out, S, H, float(eps), 1 if centred else 0,
                                stream_ptr(x)), "hc_norm")


def embed_sinusoid(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, inv_freq: torch.Tensor,
                   out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t, s, c] = table[ids[t], c] + (sin | cos)(positions[t] * inv_freq[c // 2])
    for every stream s (even c: sine, odd c: cosine); ``out`` float32 [N, S, H]."""
    require_cuda(ids, positions, table, inv_freq, out, err)
    _int32(ids, "ids")
    _int32(positions, "positions")
    n = ids.numel()
    V, H = table.shape
    if out.dim() != 3 or out.dtype != torch.float32 or out.shape[0] != n or out.shape[2] != H or not out.is_contiguous():
        raise KernelError(f"embed_sinusoid: out must be contiguous float32 [{n}, S, {H}]")
    _f32_vec(inv_freq, (H + 1) // 2, "embed_sinusoid: inv_freq")
    if not table.is_contiguous():
        raise KernelError("embed_sinusoid: table must be contiguous")
    check(core_lib().ib_embed_sinusoid(ids.data_ptr(), positions.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                                       inv_freq.data_ptr(), out.data_ptr(), n, H, V, out.shape[1], err.data_ptr(),
                                       stream_ptr(out)), "embed_sinusoid")


def scale_inplace(x: torch.Tensor, scale: float) -> None:
    """x <- x * scale (float32, in place)."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_inplace: x must be contiguous float32")
    check(core_lib().ib_scale_inplace(x.data_ptr(), x.numel(), float(scale), stream_ptr(x)), "scale_inplace")


def _state_view(state: torch.Tensor, offset: int):
    """(pointer to the state's element ``offset`` of slot 0, floats between slots)."""
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous():
        raise KernelError("a recurrent state must be contiguous float32 [slots, floats]")
    return state.data_ptr() + 4 * int(offset), state.stride(0)


def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, state_offset: int, ctx,
                out: torch.Tensor) -> None:
    """out[j, t] = x[t] + (x[t-1] - x[t]) * mu[j]; the row before an entry's first
    is the request's state (``state[slot, offset : offset + D]``), which takes the
    entry's last row.  ``mu`` float32 [M, D], ``out`` [M, N, D]."""
    require_cuda(x, mu, state, out)
    N, D = x.shape
    M = mu.shape[0]
    _f32_vec(mu, M * D, "token_shift: mu")
    if not x.is_contiguous() or out.shape != (M, N, D) or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("token_shift: x [N, D] and out [M, N, D] must be contiguous, one dtype")
    ptr, stride = _state_view(state, state_offset)
    check(core_lib().ib_token_shift(x.data_ptr(), dtype_code(x.dtype), mu.data_ptr(), ptr, stride,
                                    ctx.row_entry.data_ptr(), ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(),
                                    out.data_ptr(), N, D, M, stream_ptr(x)), "token_shift")


def head_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, heads: int, eps: float,
                   out: torch.Tensor) -> None:
    """out = o / rms_head(o) * weight * silu(gate): ``o`` float32 [N, heads * K], the
    root mean square taken over each head's K values."""
    require_cuda(o, gate, weight, out)
    N, HK = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or HK % heads or out.shape != (N, HK) \
            or not out.is_contiguous():
        raise KernelError("head_norm_gate: o contiguous float32 [N, heads * K], out contiguous of the same shape")
    _f32_vec(weight, HK, "head_norm_gate: weight")
    if gate is not None and (gate.shape != (N, HK) or gate.stride(1) != 1 or gate.dtype != out.dtype):
        raise KernelError("head_norm_gate: gate [N, heads * K] of out's dtype with unit inner stride")
    check(core_lib().ib_head_norm_gate(o.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                       dtype_code(out.dtype), weight.data_ptr(), out.data_ptr(), N, heads,
                                       HK // heads, float(eps), stream_ptr(o)), "head_norm_gate")


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float,
                     out: torch.Tensor) -> None:
    """v = y * silu(z); out = v / rms_group(v) * weight, the root mean square over
    each of ``groups`` equal parts of a row.  ``y`` float32 [N, inner]; ``z`` may
    be a view of wider rows."""
    require_cuda(y, z, weight, out)
    N, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or inner % groups or out.shape != (N, inner) \
            or not out.is_contiguous() or z.shape != (N, inner) or z.stride(1) != 1 or z.dtype != out.dtype:
        raise KernelError("gated_group_norm: y float32 [N, inner], z and out [N, inner] of the activation dtype")
    _f32_vec(weight, inner, "gated_group_norm: weight")
    check(core_lib().ib_gated_group_norm(y.data_ptr(), z.data_ptr(), z.stride(0), dtype_code(out.dtype),
                                         weight.data_ptr(), out.data_ptr(), N, inner, int(groups), float(eps),
                                         stream_ptr(y)), "gated_group_norm")


def qk_norm_append(x: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                   n_heads: int, n_kv_heads: int, head_dim: int, v_offset: int, positions: torch.Tensor,
                   row_entry: torch.Tensor, block_tables: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   err: torch.Tensor) -> None:
    """Rows of ``x`` hold ``n_heads`` query heads and then ``n_kv_heads`` key heads.
    Queries are RMS-normed per head in place (times ``q_weight`` [head_dim]); each
    key goes normed (times ``k_weight``) to its place in ``k_pool``, and the value
    pool gets the value head ``v_offset`` elements into the row, or - ``v_offset``
    negative - the key as it was projected."""
    require_cuda(x, q_weight, k_weight, positions, row_entry, block_tables, k_pool, v_pool, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    _f32_vec(q_weight, head_dim, "qk_norm_append: q_weight")
    _f32_vec(k_weight, head_dim, "qk_norm_append: k_weight")
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] < (n_heads + n_kv_heads) * head_dim:
        raise KernelError("qk_norm_append: x rows must hold the query and key heads with unit inner stride")
    num_pages, nkv_pool, page_size, hd_pool = k_pool.shape
    if k_pool.shape != v_pool.shape or nkv_pool != n_kv_heads or hd_pool != head_dim or k_pool.dtype != x.dtype \
            or v_pool.dtype != x.dtype or not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("qk_norm_append: pools must be contiguous [pages, kv_heads, page_size, head_dim] of x's dtype")
    check(core_lib().ib_qk_norm_append(x.data_ptr(), x.stride(0), dtype_code(x.dtype), _ptr(q_weight), _ptr(k_weight),
                                       float(eps), positions.data_ptr(), row_entry.data_ptr(), block_tables.data_ptr(),
                                       block_tables.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), x.shape[0],
                                       n_heads, n_kv_heads, head_dim, int(v_offset), page_size, num_pages,
                                       err.data_ptr(), stream_ptr(x)), "qk_norm_append")


_POINTWISE = {"sigmoid_gate": 0, "axpby": 1, "tanh": 2}


def pointwise(a: torch.Tensor, b: Optional[torch.Tensor], op: str, ca: float = 1.0, cb: float = 1.0) -> None:
    """In place on ``a`` [N, C] (contiguous): ``sigmoid_gate`` a * sigmoid(b);
    ``axpby`` ca * a + cb * b; ``tanh`` tanh(a).  ``b`` may be a view of wider rows."""
    require_cuda(a, b)
    if a.dim() != 2 or not a.is_contiguous() or op not in _POINTWISE:
        raise KernelError("pointwise: a must be contiguous [N, C]; ops: " + ", ".join(sorted(_POINTWISE)))
    if b is not None and (b.shape != a.shape or b.stride(1) != 1 or b.dtype != a.dtype):
        raise KernelError("pointwise: b must have a's shape and dtype with unit inner stride")
    check(core_lib().ib_pointwise(a.data_ptr(), _ptr(b), b.stride(0) if b is not None else 0, dtype_code(a.dtype),
                                  a.shape[0], a.shape[1], _POINTWISE[op], float(ca), float(cb), stream_ptr(a)),
          "pointwise_" + op)


# ---------------------------------------------------------------------------
# Layers that norm a sub-layer's result in parts before adding it, a stream that
# is a weighted sum of all layers' results, the pass before a delta rule's scan,
# attention whose queries, keys and values are normed after the rotation, and
# routing by sigmoid scores inside the best groups of experts.
# ---------------------------------------------------------------------------
def embed_dual(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, act: Optional[torch.Tensor],
               err: torch.Tensor) -> None:
    """out[t, :] = table[ids[t], :] into a float32 stream and, when given, into
    ``act`` in the activation dtype."""
    require_cuda(ids, table, out, act, err)
    _int32(ids, "ids")
    n = ids.numel()
    V, H = table.shape
    if out.dtype != torch.float32 or out.shape != (n, H) or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError(f"embed_dual: out must be contiguous float32 [{n}, {H}], the table contiguous")
    if act is not None and (act.shape != (n, H) or not act.is_contiguous()):
        raise KernelError(f"embed_dual: act must be contiguous [{n}, {H}]")
    check(core_lib().ib_embed_dual(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                   _ptr(act), dtype_code(act.dtype) if act is not None else 0, n, H, V,
                                   err.data_ptr(), stream_ptr(out)), "embed_dual")


def sub_norm_add(x_in: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, parts: int, eps: float,
                 out_res: torch.Tensor, out_act: Optional[torch.Tensor], results: Optional[torch.Tensor] = None,
                 slot: int = 0, coef: Optional[torch.Tensor] = None) -> None:
    """``X = x_in + n(y)`` with ``n`` the RMS norm over ``parts`` equal consecutive
    parts of a row times ``weight`` (float32).  Without ``results``: ``out_res = X``.
    With ``results`` (float32 [slots, N, W]): ``results[slot] = X`` and ``out_res =
    sum_{j <= slot} coef[j] results[j]``.  ``out_act`` gets ``out_res`` rounded to the
    activation dtype.  ``x_in`` and ``out_res`` may be one buffer."""
    require_cuda(x_in, y, weight, out_res, out_act, results, coef)
    N, W = x_in.shape
    for t, name in ((x_in, "x_in"), (out_res, "out_res")):
        if t.dtype != torch.float32 or t.shape != (N, W) or not t.is_contiguous():
            raise KernelError(f"sub_norm_add: {name} must be contiguous float32 [{N}, {W}]")
    if y.shape != (N, W) or not y.is_contiguous() or (out_act is not None and (
            out_act.shape != (N, W) or out_act.dtype != y.dtype or not out_act.is_contiguous())):
        raise KernelError("sub_norm_add: y and out_act must be contiguous [N, W] of one dtype")
    _f32_vec(weight, W, "sub_norm_add: weight")
    if parts <= 0 or W % parts:
        raise KernelError(f"sub_norm_add: a row of {W} does not split in {parts} parts")
    if results is not None:
        if results.dtype != torch.float32 or results.dim() != 3 or results.shape[1:] != (N, W) \
                or not results.is_contiguous() or not 1 <= slot < results.shape[0]:
            raise KernelError("sub_norm_add: results must be contiguous float32 [slots, N, W] with the slot inside")
        _f32_vec(coef, slot + 1, "sub_norm_add: coef")
    check(core_lib().ib_sub_norm_add(x_in.data_ptr(), y.data_ptr(), dtype_code(y.dtype), weight.data_ptr(), float(eps),
                                     _ptr(results), int(slot), _ptr(coef), out_res.data_ptr(), _ptr(out_act), N, W,
                                     int(parts), stream_ptr(y)), "sub_norm_add")


def part_rmsnorm(x: torch.Tensor, weight: torch.Tensor, parts: int, eps: float, out: torch.Tensor,
                 row_idx: Optional[torch.Tensor] = None) -> None:
    """out = n(x) for all rows of the float32 ``x`` or for those ``row_idx`` names."""
    require_cuda(x, weight, out, row_idx)
    _int32(row_idx, "row_idx")
    N, W = x.shape
    n_out = N if row_idx is None else row_idx.numel()
    if x.dtype != torch.float32 or not x.is_contiguous() or out.shape != (n_out, W) or not out.is_contiguous():
        raise KernelError(f"part_rmsnorm: x contiguous float32 [N, {W}], out contiguous [{n_out}, {W}]")
    _f32_vec(weight, W, "part_rmsnorm: weight")
    if parts <= 0 or W % parts:
        raise KernelError(f"part_rmsnorm: a row of {W} does not split in {parts} parts")
    check(core_lib().ib_part_rmsnorm(x.data_ptr(), _ptr(row_idx), weight.data_ptr(), float(eps), out.data_ptr(),
                                     dtype_code(out.dtype), n_out, W, int(parts), stream_ptr(x)), "part_rmsnorm")


def rope_norm_append(x: torch.Tensor, bias: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                     norm_qk: bool, norm_v: bool, eps: float, n_heads: int, n_kv_heads: int, head_dim: int,
                     positions: torch.Tensor, row_entry: torch.Tensor, block_tables: torch.Tensor,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, err: torch.Tensor) -> None:
    """Rows of ``x`` hold ``n_heads`` query heads and ``n_kv_heads`` key heads of
    ``head_dim`` and then ``n_kv_heads`` value heads of the value pool's width.  The
    bias (float32, one value per column of those) is added; queries and keys are
    rotated in their first ``rotary_dim`` dimensions and then, with ``norm_qk``,
    divided by their root mean square per head; values, with ``norm_v``, likewise.
    Queries are written back in place, keys and values to their pages."""
    require_cuda(x, bias, inv_freq, positions, row_entry, block_tables, k_pool, v_pool, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    num_pages, nkv_pool, page_size, hd_pool = k_pool.shape
    hdv = v_pool.shape[3]
    cols = (n_heads + n_kv_heads) * head_dim + n_kv_heads * hdv
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] < cols:
        raise KernelError("rope_norm_append: x rows must hold the query, key and value heads with unit inner stride")
    if nkv_pool != n_kv_heads or hd_pool != head_dim or v_pool.shape[:3] != k_pool.shape[:3] or k_pool.dtype != x.dtype \
            or v_pool.dtype != x.dtype or not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("rope_norm_append: pools must be contiguous [pages, kv_heads, page_size, size] of x's dtype")
    _f32_vec(bias, cols, "rope_norm_append: bias")
    if rotary_dim > 0:
        _f32_vec(inv_freq, rotary_dim // 2, "rope_norm_append: inv_freq")
        if inv_freq is None:
            raise KernelError("rope_norm_append: a rotation needs its frequencies")
    check(core_lib().ib_rope_norm_append(x.data_ptr(), x.stride(0), dtype_code(x.dtype), _ptr(bias), _ptr(inv_freq),
                                         int(rotary_dim), 1 if norm_qk else 0, 1 if norm_v else 0, float(eps),
                                         positions.data_ptr(), row_entry.data_ptr(), block_tables.data_ptr(),
                                         block_tables.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), x.shape[0],
                                         n_heads, n_kv_heads, head_dim, hdv, page_size, num_pages, err.data_ptr(),
                                         stream_ptr(x)), "rope_norm_append")


def moe_route_scored(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor,
                     weights: torch.Tensor, gate: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1,
                     group_top: int = 2, renorm: bool = False) -> None:
    """Routing by ``s = sigmoid(logits + bias)``: the experts form ``groups`` equal
    groups of neighbours, a group's score is the sum of its ``group_top`` largest
    scores, only experts of the ``keep`` best groups can be chosen; the ``top``
    largest scores among them are chosen and are the weights (``renorm``: divided
    by their sum).  Outputs as ``moe_route``."""
    require_cuda(logits, bias, ids, weights, gate)
    _int32(ids, "ids")
    N, E = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or ids.shape != (N, top) \
            or weights.shape != (N, top) or weights.dtype != torch.float32 or not weights.is_contiguous():
        raise KernelError("moe_route_scored: logits float32 [N, E], ids int32 [N, top], weights float32 [N, top]")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (E,) or not bias.is_contiguous()):
        raise KernelError("moe_route_scored: the bias must be float32 [E]")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != (N, E) or not gate.is_contiguous()):
        raise KernelError("moe_route_scored: gate must be contiguous float32 [N, E]")
    check(core_lib().ib_moe_route_scored(logits.data_ptr(), logits.stride(0), _ptr(bias), E, int(top), int(groups),
                                         int(keep), int(group_top), 1 if renorm else 0, ids.data_ptr(),
                                         weights.data_ptr(), _ptr(gate), N, stream_ptr(logits)), "moe_route_scored")


# ---------------------------------------------------------------------------
# Layers that norm what a sub-layer reads and what it returns, with a short
# convolution on the input and a gate on the result; a stream that re-enters a
# run of layers together with the embedding's output; attention with two score
# maps per head; routing by a softmax over all router outputs, some of which
# hand the input on.
# ---------------------------------------------------------------------------
def gated_norm_add(x_in: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor],
                   weight: torch.Tensor, parts: int, eps: float, mult: float, out_res: torch.Tensor,
                   out_act: Optional[torch.Tensor] = None) -> None:
    """``out_res = x_in + mult * n(y * sigmoid(gate + gate_bias))`` with ``n`` the RMS norm
    over ``parts`` equal consecutive parts of a row times ``weight`` (float32).
    ``gate`` None: the result is normed as it is; it may be a view of wider rows.
    ``x_in`` and ``out_res`` (float32) may be one buffer."""
    require_cuda(x_in, y, gate, gate_bias, weight, out_res, out_act)
    N, W = x_in.shape
    for t, name in ((x_in, "x_in"), (out_res, "out_res")):
        if t.dtype != torch.float32 or t.shape != (N, W) or not t.is_contiguous():
            raise KernelError(f"gated_norm_add: {name} must be contiguous float32 [{N}, {W}]")
    if y.shape != (N, W) or not y.is_contiguous() or (out_act is not None and (
            out_act.shape != (N, W) or out_act.dtype != y.dtype or not out_act.is_contiguous())):
        raise KernelError("gated_norm_add: y and out_act must be contiguous [N, W] of one dtype")
    if gate is not None and (gate.shape != (N, W) or gate.stride(1) != 1 or gate.dtype != y.dtype):
        raise KernelError("gated_norm_add: the gate must be [N, W] of y's dtype with unit inner stride")
    _f32_vec(weight, W, "gated_norm_add: weight")
    _f32_vec(gate_bias, W, "gated_norm_add: gate bias")
    if parts <= 0 or W % parts:
        raise KernelError(f"gated_norm_add: a row of {W} does not split in {parts} parts")
    check(core_lib().ib_gated_norm_add(x_in.data_ptr(), y.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                       _ptr(gate_bias), dtype_code(y.dtype), weight.data_ptr(), float(eps), float(mult),
                                       out_res.data_ptr(), _ptr(out_act), N, W, int(parts), stream_ptr(y)),
          "gated_norm_add")


def concat_round(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] = [a[n] | b[n]] rounded to ``out``'s dtype; ``a``, ``b`` float32 [N, W]."""
    require_cuda(a, b, out)
    N, W = a.shape
    if a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != (N, W) or not a.is_contiguous() \
            or not b.is_contiguous() or out.shape != (N, 2 * W) or not out.is_contiguous():
        raise KernelError("concat_round: a, b contiguous float32 [N, W], out contiguous [N, 2 W]")
    check(core_lib().ib_concat_round(a.data_ptr(), b.data_ptr(), out.data_ptr(), dtype_code(out.dtype), N, W,
                                     stream_ptr(a)), "concat_round")


def add_row(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[n, :] += v in place; ``x`` float32 [N, W], ``v`` float32 [W]."""
    require_cuda(x, v)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("add_row: x must be contiguous float32 [N, W]")
    _f32_vec(v, x.shape[1], "add_row: v")
    check(core_lib().ib_add_row(x.data_ptr(), v.data_ptr(), x.shape[0], x.shape[1], stream_ptr(x)), "add_row")


def causal_conv(x: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor], state_offset: int, ctx,
                out: torch.Tensor, add_input: bool = False) -> None:
    """Per channel ``out_t = (x_t if add_input) + sum_j weight[:, j] x_(t - taps + 1 + j)`` over each
    entry's rows in order; the ``taps - 1`` inputs before an entry's first row come from the request's
    state (``state[slot, offset : offset + (taps - 1) C]``, float32, oldest first).  ``x`` [N, C] may be
    a view of wider rows; ``weight`` float32 [C, taps].  The state is not changed: ``conv_state_update``
    does that once every row has read it."""
    require_cuda(x, weight, state, out)
    N, C = x.shape
    taps = weight.shape[1]
    if x.stride(1) != 1 or out.shape != (N, C) or out.stride(1) != 1 or out.dtype != x.dtype:
        raise KernelError("causal_conv: x and out must be [N, C] of one dtype with unit inner stride")
    if weight.dtype != torch.float32 or weight.shape != (C, taps) or not weight.is_contiguous():
        raise KernelError("causal_conv: the filters must be contiguous float32 [C, taps]")
    ptr, stride = _state_view(state, state_offset) if taps > 1 else (None, 0)
    check(core_lib().ib_causal_conv(x.data_ptr(), x.stride(0), dtype_code(x.dtype), weight.data_ptr(), ptr, stride,
                                    ctx.row_entry.data_ptr(), ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(),
                                    out.data_ptr(), out.stride(0), N, C, taps, 1 if add_input else 0, stream_ptr(x)),
          "causal_conv")


def conv_state_update(x: torch.Tensor, taps: int, state: torch.Tensor, state_offset: int, ctx) -> None:
    """The convolution's state after the step: the last ``taps - 1`` rows of (old state, then the entry's
    rows of ``x``), per entry; an entry without rows keeps its state."""
    if taps <= 1:
        return
    require_cuda(x, state)
    N, C = x.shape
    if x.stride(1) != 1:
        raise KernelError("conv_state_update: x must have unit inner stride")
    ptr, stride = _state_view(state, state_offset)
    check(core_lib().ib_conv_state_update(x.data_ptr(), x.stride(0), dtype_code(x.dtype), ptr, stride,
                                          ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(), ctx.n_entries, C, int(taps),
                                          stream_ptr(x)), "conv_state_update")


def conv_rope_append(x: torch.Tensor, weight: Optional[torch.Tensor], state: Optional[torch.Tensor], state_offset: int,
                     inv_freq: Optional[torch.Tensor], rotary_dim: int, magnitude: float, n_heads: int, n_kv_heads: int,
                     dim: int, vdim: int, ctx, block_tables: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor,
                     v_pool: torch.Tensor, err: torch.Tensor) -> None:
    """Rows of ``x``: ``n_heads`` query heads of two maps of ``dim``, ``n_kv_heads`` key heads of two maps,
    ``n_kv_heads`` values of ``vdim``, as projected.  Each channel goes through its short causal
    convolution (``weight`` float32 [C, taps]; None: none), every map of a query or key is rotated in its
    first ``rotary_dim`` dimensions (neighbours paired); queries go to ``q_out`` [N, n_heads * 2 dim], keys
    and values to their pages ([pages, n_kv_heads, page_size, 2 dim] and [.., vdim])."""
    require_cuda(x, weight, state, inv_freq, block_tables, q_out, k_pool, v_pool, err)
    _int32(block_tables, "block_tables")
    N = x.shape[0]
    C = (n_heads + n_kv_heads) * 2 * dim + n_kv_heads * vdim
    taps = 0 if weight is None else weight.shape[1]
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] < C:
        raise KernelError("conv_rope_append: x rows must hold queries, keys and values with unit inner stride")
    if weight is not None and (weight.dtype != torch.float32 or weight.shape != (C, taps) or not weight.is_contiguous()):
        raise KernelError("conv_rope_append: the filters must be contiguous float32 [C, taps]")
    num_pages, nkv_pool, page_size, kw = k_pool.shape
    if nkv_pool != n_kv_heads or kw != 2 * dim or v_pool.shape != (num_pages, n_kv_heads, page_size, vdim) \
            or k_pool.dtype != x.dtype or v_pool.dtype != x.dtype or not k_pool.is_contiguous() \
            or not v_pool.is_contiguous():
        raise KernelError("conv_rope_append: pools must be contiguous [pages, kv_heads, page_size, 2 dim | vdim] of x's dtype")
    if q_out.shape != (N, n_heads * 2 * dim) or q_out.dtype != x.dtype or not q_out.is_contiguous():
        raise KernelError("conv_rope_append: q_out must be contiguous [N, heads * 2 dim] of x's dtype")
    if rotary_dim:
        _f32_vec(inv_freq, rotary_dim // 2, "conv_rope_append: inv_freq")
        if inv_freq is None:
            raise KernelError("conv_rope_append: a rotation needs its frequencies")
    ptr, stride = _state_view(state, state_offset) if taps > 1 else (None, 0)
    check(core_lib().ib_conv_rope_append(x.data_ptr(), x.stride(0), dtype_code(x.dtype), _ptr(weight), taps, ptr, stride,
                                         ctx.positions.data_ptr(), ctx.row_entry.data_ptr(), ctx.cu_rows.data_ptr(),
                                         ctx.slot_ids.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                                         _ptr(inv_freq), int(rotary_dim), float(magnitude), n_heads, n_kv_heads, dim,
                                         vdim, q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_size,
                                         num_pages, N, err.data_ptr(), stream_ptr(x)), "conv_rope_append")


def attention_diff(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, ctx,
                   block_tables: torch.Tensor, n_heads: int, scale: float, softcap: float, lam: float, eps: float,
                   out_scale: float, err: torch.Tensor) -> None:
    """Two causal softmax maps per head over shared values, ``o = A_1 V - lam A_2 V``, each head's ``o``
    divided by its root mean square (``eps`` inside the root) and multiplied by ``out_scale``.  ``q``
    [N, n_heads * 2 dim] holds a head's two queries side by side, the key pool a key head's two keys
    ([pages, kv_heads, page_size, 2 dim]); scores are ``softcap * tanh(q . k * scale / softcap)``
    (``softcap`` 0: uncapped).  ``out`` [N, n_heads * vdim].  32-bit arithmetic."""
    require_cuda(q, k_pool, v_pool, out, block_tables, err)
    _int32(block_tables, "block_tables")
    N = q.shape[0]
    num_pages, nkv, page_size, kw = k_pool.shape
    vdim = v_pool.shape[3]
    if kw % 2 or q.shape != (N, n_heads * kw) or not q.is_contiguous() or out.shape != (N, n_heads * vdim) \
            or not out.is_contiguous() or q.dtype != k_pool.dtype or out.dtype != q.dtype or v_pool.dtype != q.dtype \
            or v_pool.shape[:3] != k_pool.shape[:3] or not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention_diff: q [N, heads * 2 dim], out [N, heads * vdim] and the pools do not fit")
    check(core_lib().ib_attention_diff(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                       dtype_code(q.dtype), ctx.positions.data_ptr(), ctx.row_entry.data_ptr(),
                                       block_tables.data_ptr(), block_tables.shape[1], N, n_heads, nkv, kw // 2, vdim,
                                       page_size, num_pages, float(scale), float(softcap or 0.0), float(lam), float(eps),
                                       float(out_scale), err.data_ptr(), stream_ptr(q)), "attention_diff")


def moe_route_softmax_all(logits: torch.Tensor, correction: Optional[torch.Tensor], outputs: int, experts: int, top: int,
                          ids: torch.Tensor, weights: torch.Tensor, gate: Optional[torch.Tensor],
                          extra: Optional[torch.Tensor]) -> None:
    """Routing by ``s = softmax(logits[:, :outputs])``: the ``top`` largest ``s + correction`` are chosen
    (lowest index among equals), their weights are ``s`` over the chosen ones' sum (+ 1e-20).  Outputs
    from ``experts`` on have no expert: their weight is summed into ``extra[:, 0]``.  ``gate`` [N, experts]
    gets the dense weights of the experts that exist.  When ``logits`` has one more column, ``extra[:, 1]``
    is its sigmoid, else 1; a ``gate`` wider than ``experts`` gets that number in its further columns."""
    require_cuda(logits, correction, ids, weights, gate, extra)
    _int32(ids, "ids")
    N, cols = logits.shape
    if cols not in (outputs, outputs + 1) or logits.dtype != torch.float32 or logits.stride(1) != 1 \
            or ids.shape != (N, top) or not ids.is_contiguous() or weights.shape != (N, top) \
            or weights.dtype != torch.float32 or not weights.is_contiguous():
        raise KernelError("moe_route_softmax_all: logits float32 [N, outputs (+ 1)], ids int32 and weights float32 [N, top]")
    _f32_vec(correction, outputs, "moe_route_softmax_all: correction")
    if gate is not None and (gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] != N
                             or gate.shape[1] < experts or not gate.is_contiguous()):
        raise KernelError("moe_route_softmax_all: gate must be contiguous float32 [N, >= experts]")
    if extra is not None and (extra.dtype != torch.float32 or extra.shape != (N, 2) or not extra.is_contiguous()):
        raise KernelError("moe_route_softmax_all: extra must be contiguous float32 [N, 2]")
    check(core_lib().ib_moe_route_softmax_all(logits.data_ptr(), logits.stride(0), _ptr(correction), int(outputs),
                                              int(experts), int(top), 1 if cols == outputs + 1 else 0, ids.data_ptr(),
                                              weights.data_ptr(), _ptr(gate), _ptr(extra),
                                              gate.shape[1] if gate is not None else int(experts), N, stream_ptr(logits)),
          "moe_route_softmax_all")


def moe_combine(routed: Optional[torch.Tensor], h: torch.Tensor, shared: Optional[torch.Tensor], extra: torch.Tensor,
                out: torch.Tensor) -> None:
    """out = routed + extra[:, 0] * h + extra[:, 1] * shared, row by row ([N, W]; ``h`` may be a view of
    wider rows; ``routed`` and ``shared`` may be None)."""
    require_cuda(routed, h, shared, extra, out)
    N, W = out.shape
    if h.shape != (N, W) or h.stride(1) != 1 or h.dtype != out.dtype or not out.is_contiguous():
        raise KernelError("moe_combine: h and out must be [N, W] of one dtype")
    for t in (routed, shared):
        if t is not None and (t.shape != (N, W) or t.dtype != out.dtype or not t.is_contiguous()):
            raise KernelError("moe_combine: routed and shared must be contiguous [N, W] of out's dtype")
    if extra.dtype != torch.float32 or extra.shape != (N, 2) or not extra.is_contiguous():
        raise KernelError("moe_combine: extra must be contiguous float32 [N, 2]")
    check(core_lib().ib_moe_combine(_ptr(routed), h.data_ptr(), h.stride(0), _ptr(shared), extra.data_ptr(), out.data_ptr(),
                                    dtype_code(out.dtype), N, W, stream_ptr(out)), "moe_combine")
