"""The scans of recurrent mixers (``scan.cu``): one compiled module per number
of rows of the per-head state matrix, built when a model first needs it.

``wkv_scan``, ``ssd_scan`` and ``delta_scan`` walk every entry's rows in order from the state in
the request's slot and leave the new state there; what they need to know about
the step (entries, slots) they read from the step's device tensors, so a
recorded step replays them for other requests.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from ..csrc.build import load_module
from ..errors import KernelError
from . import core

_c_int, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
_libs: Dict[int, ctypes.CDLL] = {}
MAX_ROWS = 512
SM_COUNT_FALLBACK = 148


def lib_for(rows: int) -> ctypes.CDLL:
    lib = _libs.get(rows)
    if lib is None:
        if not 1 <= rows <= MAX_ROWS:
            raise KernelError(f"recurrent scan: a state of {rows} rows per head is outside 1..{MAX_ROWS}")
        lib = load_module(f"scan_r{rows}", ["scan.cu"], [f"-DIB_ROWS={rows}"])
        lib.ib_wkv_scan.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p,
                                    _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_ssd_scan.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_ll, _c_void_p,
                                    _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_delta_scan.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p,
                                      _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        for fn in ("ib_wkv_scan", "ib_ssd_scan", "ib_delta_scan", "ib_scan_rows", "ib_scan_split"):
            getattr(lib, fn).restype = _c_int
        if lib.ib_scan_rows() != rows:
            raise KernelError(f"scan module for {rows} state rows was built for another size")
        _libs[rows] = lib
    return lib


def choose_col_slices(n_entries: int, heads: int, cols: int, split: int, sm_count: int) -> int:
    """Into how many CTAs the columns of a head's state are cut.  The warps of a
    scan are as many as its columns times the lanes of a column, whatever the
    slicing; slices only spread them over the SMs.  Every CTA fetches the whole of
    its head's per-token factors, so a head is cut no further than it takes to give
    most SMs a CTA, and a CTA keeps at least one warp, at most 512 threads and at
    most 128 columns (whose values it stages in shared memory).
    The result does not change any number: a column's arithmetic is the same in
    every slicing."""
    slices = 1
    while cols % (slices * 2) == 0 and (
            (cols // slices) * split > 512 or cols // slices > 128
            or (4 * n_entries * heads * slices < 3 * sm_count and (cols // (slices * 2)) * split >= 32)):
        slices *= 2
    if (cols // slices) * split > 512 or cols // slices > 128:
        # (no power of two cuts it small enough: take the smallest divisor that does)
        for s in range(slices + 1, cols + 1):
            if cols % s == 0 and (cols // s) * split <= 512 and cols // s <= 128:
                return s
    return slices


def _state_ptr(state: torch.Tensor, offset: int):
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous():
        raise KernelError("a recurrent state must be contiguous float32 [slots, floats]")
    return state.data_ptr() + 4 * int(offset), state.stride(0)


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, w0: torch.Tensor, u: torch.Tensor,
             state: torch.Tensor, state_offset: int, ctx, out: torch.Tensor, heads: int, rt) -> None:
    """Per head, with S [K, K] from ``state[slot, offset:]`` (stored column by column):
    ``o_t = (S + diag(u) k_t v_t^T)^T r_t``, then ``S <- diag(w_t) S + k_t v_t^T``
    with ``w_t = exp(-exp(z_t + w0))``.  ``r, k, v`` [N, heads * K] (activation
    dtype, one row stride), ``z`` float32 [N, heads * K], ``out`` float32.
    Two kernels: a parallel pass that makes every token's factors in 32-bit, and
    the scan that walks each entry's tokens in order."""
    core.require_cuda(r, k, v, z, w0, u, state, out)
    N, HK = r.shape
    K = HK // heads
    if HK % heads or k.shape != r.shape or v.shape != r.shape or not (r.dtype == k.dtype == v.dtype) \
            or r.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1 or not (r.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("wkv_scan: r, k, v must be [N, heads * K] of one dtype and one row stride")
    if z.shape != (N, HK) or z.dtype != torch.float32 or not z.is_contiguous() \
            or out.shape != (N, HK) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("wkv_scan: z and out must be contiguous float32 [N, heads * K]")
    for t, name in ((w0, "w0"), (u, "u")):
        if t.dtype != torch.float32 or t.numel() != HK or not t.is_contiguous():
            raise KernelError(f"wkv_scan: {name} must be contiguous float32 with {HK} values")
    lib = lib_for(K)
    factors = torch.empty((N, HK, 4), dtype=torch.float32, device=r.device)
    v32 = torch.empty((N, HK), dtype=torch.float32, device=r.device)
    core.check(core.core_lib().ib_wkv_prepare(r.data_ptr(), k.data_ptr(), v.data_ptr(), r.stride(0),
                                              core.dtype_code(r.dtype), z.data_ptr(), w0.data_ptr(), u.data_ptr(),
                                              factors.data_ptr(), v32.data_ptr(), N, HK, K, core.stream_ptr(r)),
               "wkv_prepare")
    ptr, stride = _state_ptr(state, state_offset)
    sm = rt.options.get("sm_count") or SM_COUNT_FALLBACK
    slices = choose_col_slices(ctx.n_entries, heads, K, lib.ib_scan_split(), sm)
    core.check(lib.ib_wkv_scan(factors.data_ptr(), v32.data_ptr(), N, ptr, stride, ctx.cu_rows.data_ptr(),
                               ctx.slot_ids.data_ptr(), out.data_ptr(), ctx.n_entries, heads, K, slices,
                               core.stream_ptr(r)), "wkv_scan")


def ssd_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, state_offset: int, ctx, out: torch.Tensor, heads: int, groups: int,
             state_rows: int, vdim: int, rt, conv=None) -> None:
    """Per head, with S [state_rows, vdim] from ``state[slot, offset:]`` (stored column by column):
    ``S <- exp(-exp(a_log) dt) S + dt B_t x_t^T``, ``y_t = S^T C_t + d_skip x_t``,
    ``dt = softplus(dt_raw + dt_bias)``.  ``xbc`` [N, heads*vdim + 2*groups*state_rows]
    holds x, B and C side by side; ``dt`` [N, heads]; both may be views of wider
    rows; ``out`` float32 [N, heads * vdim].  ``conv`` = (weight [C, taps], bias
    [C] or None, offset of the convolution's inputs in the state): x, B and C
    first pass a causal convolution per channel and SiLU, whose last ``taps - 1``
    inputs are carried in the state.  Two kernels as for ``wkv_scan``: the parallel
    pass (with the convolution) and the scan."""
    core.require_cuda(xbc, dt, dt_bias, a_log, d_skip, state, out)
    N = xbc.shape[0]
    inner, gn = heads * vdim, groups * state_rows
    if xbc.shape[1] != inner + 2 * gn or xbc.stride(1) != 1 or dt.shape != (N, heads) \
            or dt.stride(1) != 1 or dt.dtype != xbc.dtype or heads % groups:
        raise KernelError("ssd_scan: xbc [N, inner + 2 groups state] and dt [N, heads] of one dtype do not fit")
    if out.shape != (N, inner) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("ssd_scan: out must be contiguous float32 [N, heads * vdim]")
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        if t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous():
            raise KernelError(f"ssd_scan: {name} must be contiguous float32 [{heads}]")
    lib = lib_for(state_rows)
    x32 = torch.empty((N, inner), dtype=torch.float32, device=xbc.device)
    bc = torch.empty((N, gn, 2), dtype=torch.float32, device=xbc.device)
    dd = torch.empty((N, heads, 2), dtype=torch.float32, device=xbc.device)
    w = b = None
    taps, conv_ptr, conv_stride = 1, None, 0
    if conv is not None:
        w, b, conv_offset = conv
        taps = w.shape[1]
        if w.dtype != torch.float32 or w.shape[0] != inner + 2 * gn or not w.is_contiguous() or (
                b is not None and (b.dtype != torch.float32 or b.numel() != inner + 2 * gn or not b.is_contiguous())):
            raise KernelError("ssd_scan: the convolution's weight [C, taps] and bias [C] must be contiguous float32")
        conv_ptr, conv_stride = _state_ptr(state, conv_offset)
    core.check(core.core_lib().ib_ssd_prepare(
        xbc.data_ptr(), xbc.stride(0), core.dtype_code(xbc.dtype), w.data_ptr() if w is not None else None,
        b.data_ptr() if b is not None else None, conv_ptr, conv_stride, ctx.row_entry.data_ptr(),
        ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(), dt.data_ptr(), dt.stride(0), dt_bias.data_ptr(),
        a_log.data_ptr(), x32.data_ptr(), bc.data_ptr(), dd.data_ptr(), N, ctx.n_entries, inner, gn, heads, state_rows,
        taps,
        core.stream_ptr(xbc)), "ssd_prepare")
    ptr, stride = _state_ptr(state, state_offset)
    sm = rt.options.get("sm_count") or SM_COUNT_FALLBACK
    slices = choose_col_slices(ctx.n_entries, heads, vdim, lib.ib_scan_split(), sm)
    core.check(lib.ib_ssd_scan(x32.data_ptr(), bc.data_ptr(), dd.data_ptr(), N, d_skip.data_ptr(), ptr, stride,
                               ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(), out.data_ptr(), ctx.n_entries, heads,
                               groups, vdim, slices, core.stream_ptr(xbc)), "ssd_scan")


def delta_scan(proj: torch.Tensor, c_off: int, b_off: int, a_off: int, conv_w: Optional[torch.Tensor],
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, state_offset: int, conv_offset: int,
               ctx, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, rt) -> None:
    """A gated delta rule.  Per value head, with S [dim, vdim] from ``state[slot, offset:]``
    (stored column by column) and the head's key head ``h // (heads / kv_heads)``:
    ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``.
    A row of ``proj`` holds, from column ``c_off``, the channels ``q | k`` (kv_heads x dim
    each) and ``v`` (heads x vdim), and at ``b_off`` / ``a_off`` the ``heads`` pre-activations
    of ``beta = sigmoid(.)`` and of ``g = exp(-exp(a_log) softplus(. + dt_bias))``.  The
    channels first pass a causal convolution (``conv_w`` float32 [channels, taps], last
    column the current token's; None: none) and SiLU; q and k are then scaled to unit
    length, q also by ``dim ** -0.5``.  The convolution's last ``taps - 1`` inputs are
    carried at ``conv_offset`` of the state.  ``out`` float32 [N, heads * vdim].
    Two kernels as for the other scans: the parallel pass and the scan."""
    core.require_cuda(proj, conv_w, a_log, dt_bias, state, out)
    N = proj.shape[0]
    C = 2 * kv_heads * dim + heads * vdim
    if proj.dim() != 2 or proj.stride(1) != 1 or heads % kv_heads or min(c_off, b_off, a_off) < 0 \
            or max(c_off + C, b_off + heads, a_off + heads) > proj.shape[1]:
        raise KernelError("delta_scan: the projected rows do not hold q | k | v and the two gate pre-activations")
    if out.shape != (N, heads * vdim) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("delta_scan: out must be contiguous float32 [N, heads * vdim]")
    for t, name in ((a_log, "a_log"), (dt_bias, "dt_bias")):
        if t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous():
            raise KernelError(f"delta_scan: {name} must be contiguous float32 [{heads}]")
    taps = 0
    if conv_w is not None:
        taps = conv_w.shape[1]
        if conv_w.dtype != torch.float32 or conv_w.shape[0] != C or not conv_w.is_contiguous():
            raise KernelError(f"delta_scan: the convolution's weight must be contiguous float32 [{C}, taps]")
    lib = lib_for(dim)
    dev = proj.device
    kq = torch.empty((kv_heads, N, dim, 2), dtype=torch.float32, device=dev)
    v32 = torch.empty((heads, N, vdim), dtype=torch.float32, device=dev)
    dd = torch.empty((heads, N, 4), dtype=torch.float32, device=dev)
    conv_ptr, conv_stride = _state_ptr(state, conv_offset)
    core.check(core.core_lib().ib_delta_prepare(
        proj.data_ptr(), proj.stride(0), core.dtype_code(proj.dtype), int(c_off), int(b_off), int(a_off),
        conv_w.data_ptr() if conv_w is not None else None, taps, conv_ptr, conv_stride, ctx.row_entry.data_ptr(),
        ctx.cu_rows.data_ptr(), ctx.slot_ids.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), kq.data_ptr(),
        v32.data_ptr(), dd.data_ptr(), N, ctx.n_entries, kv_heads, heads, dim, vdim, core.stream_ptr(proj)),
        "delta_prepare")
    ptr, stride = _state_ptr(state, state_offset)
    sm = rt.options.get("sm_count") or SM_COUNT_FALLBACK
    slices = choose_col_slices(ctx.n_entries, heads, vdim, lib.ib_scan_split(), sm)
    core.check(lib.ib_delta_scan(v32.data_ptr(), kq.data_ptr(), dd.data_ptr(), N, ptr, stride, ctx.cu_rows.data_ptr(),
                                 ctx.slot_ids.data_ptr(), out.data_ptr(), ctx.n_entries, heads, kv_heads, vdim, slices,
                                 core.stream_ptr(proj)), "delta_scan")
