"""The tensor-core kernel for differential attention (``attention_diff_mma.cu``),
one compiled module per (map size, value size), built when a model first needs it.

``run`` returns False when the sizes have no variant (bfloat16; map and value
sizes multiples of 16, at most 256) or ``rt.options["attention"] == "plain"``;
the caller then takes the plain 32-bit kernel (``core.attention_diff``).

A step whose entries all have few rows (decoded tokens) would run one CTA per
entry and key/value head; ``choose_splits`` then cuts the keys in slices over
several CTAs.  When every entry has at most 16 packed rows (rows x heads of a
group) and values are a multiple of 64 wide, a kernel that walks the keys once
with both maps' sums side by side takes the step (``one_walk``); otherwise the
two walks become two launches.  The plan and the scratch buffer are worked out
once per step and kept in ``ctx.scratch``.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from ..csrc.build import load_module
from ..errors import KernelError
from . import core

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_libs: Dict[Tuple[int, int], ctypes.CDLL] = {}


def supported(dim: int, vdim: int) -> bool:
    return dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 256 and 16 <= vdim <= 256


def lib_for(dim: int, vdim: int) -> ctypes.CDLL:
    lib = _libs.get((dim, vdim))
    if lib is None:
        lib = load_module(f"attn_diff_d{dim}_e{vdim}", ["attention_diff_mma.cu"], [f"-DDIFF_D={dim}", f"-DDIFF_E={vdim}"])
        lib.ib_attention_diff_mma.argtypes = [
            _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
            _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_float, _c_float, _c_void_p, _c_int, _c_int, _c_int,
            _c_void_p, ctypes.c_longlong, _c_void_p]
        lib.ib_attention_diff_mma.restype = _c_int
        lib.ib_attention_diff_mma_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        lib.ib_attention_diff_mma_scratch_bytes.restype = ctypes.c_longlong
        lib.ib_attention_diff_decode.argtypes = [
            _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
            _c_int, _c_int, _c_float, _c_float, _c_float, _c_float, _c_float, _c_void_p, _c_int, _c_int, _c_int,
            _c_void_p, ctypes.c_longlong, _c_void_p]
        lib.ib_attention_diff_decode.restype = _c_int
        lib.ib_attention_diff_decode_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        lib.ib_attention_diff_decode_scratch_bytes.restype = ctypes.c_longlong
        if lib.ib_attention_diff_mma_d() != dim or lib.ib_attention_diff_mma_e() != vdim:
            raise KernelError(f"differential attention module for ({dim}, {vdim}) was built for other sizes")
        _libs[(dim, vdim)] = lib
    return lib


SM_COUNT_FALLBACK = 148
ROW_TILE, KEY_TILE, MAX_SPLITS = 64, 32, 64


def choose_splits(max_rows_per_entry: int, n_entries: int, group: int, kv_heads: int, max_kv_len: int,
                  sm_count: int, n_rows: int = 0, heads: int = 0, vdim: int = 0) -> Tuple[int, int]:
    """(slices of the keys, keys per slice).  Steps of few rows (every entry fits one row tile): when
    the CTAs leave SMs idle and there are keys enough for slices of at least two tiles, as many slices
    as fill the SMs about four times (a CTA waits for its keys most of the time).  Prompts: the row
    tile at a prompt's end walks all its keys while the first walks one tile, and a prompt of a few
    thousand tokens has no more row tiles than the SMs hold at once; slices of at least 512 keys
    shorten that longest walk, as many as keep the slices' 32-bit shares (``n_rows x heads x vdim``
    floats each) within 96 MB."""
    tiles = -(-max_rows_per_entry * group // ROW_TILE)
    ctas = max(1, tiles * n_entries * kv_heads)
    if tiles > 1:
        share = max(1, n_rows * heads * vdim * 4)
        want = min(max_kv_len // 512, 8, (96 << 20) // share, 65535 // max(kv_heads, 1))
        if want < 2 or ctas >= 8 * sm_count:
            return 1, 0
    else:
        if ctas >= 2 * sm_count or max_kv_len < 4 * KEY_TILE:
            return 1, 0
        want = min(-(-4 * sm_count // ctas), max_kv_len // (2 * KEY_TILE), MAX_SPLITS, 65535 // max(kv_heads, 1))
        if want < 2:
            return 1, 0
    slice_len = -(-(-(-max_kv_len // want)) // KEY_TILE) * KEY_TILE
    return -(-max_kv_len // slice_len), slice_len


def one_walk(max_rows_per_entry: int, group: int, vdim: int) -> bool:
    """Whether the kernel that walks the keys once takes the step."""
    return max_rows_per_entry * group <= 16 and vdim % 64 == 0


def run(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, ctx, tables: torch.Tensor,
        n_heads: int, scale: float, softcap: float, lam: float, eps: float, out_scale: float, rt) -> bool:
    """Arguments as ``core.attention_diff``; entries and their rows come from ``ctx.cu_rows`` and
    ``ctx.positions`` (an entry's rows are consecutive positions)."""
    num_pages, nkv, page_size, kw = k_pool.shape
    dim, vdim = kw // 2, v_pool.shape[3]
    if q.dtype != torch.bfloat16 or rt.options.get("attention", "auto") == "plain" or not supported(dim, vdim):
        return False
    N = q.shape[0]
    if q.shape != (N, n_heads * kw) or not q.is_contiguous() or out.shape != (N, n_heads * vdim) \
            or not out.is_contiguous() or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or v_pool.shape[:3] != k_pool.shape[:3]:
        raise KernelError("attention_diff_mma: q [N, heads * 2 dim], out [N, heads * vdim] and the pools do not fit")
    core.require_cuda(q, k_pool, v_pool, out, tables)
    lib = lib_for(dim, vdim)
    key = ("diff_plan", n_heads, nkv, dim, vdim)
    plan = ctx.scratch.get(key) if hasattr(ctx, "scratch") else None
    if plan is None:
        forced = rt.options.get("diff_splits")
        plan = tuple(forced) if forced else choose_splits(
            ctx.max_rows_per_entry, ctx.n_entries, n_heads // nkv, nkv, getattr(ctx, "max_kv_len", 0),
            rt.options.get("sm_count") or SM_COUNT_FALLBACK, N, n_heads, vdim)
        if hasattr(ctx, "scratch"):
            ctx.scratch[key] = plan
    splits, slice_len = plan[:2]
    once = bool(plan[2]) if len(plan) > 2 else one_walk(ctx.max_rows_per_entry, n_heads // nkv, vdim)
    if once and (splits <= 1 and slice_len <= 0):
        # one slice over all keys any row of the step sees
        splits, slice_len = 1, max(KEY_TILE, -(-ctx.max_kv_len // KEY_TILE) * KEY_TILE)
    scratch_ptr, scratch_bytes = None, 0
    if splits > 1 or once:
        need = (lib.ib_attention_diff_decode_scratch_bytes if once else lib.ib_attention_diff_mma_scratch_bytes)(
            N, n_heads, splits)
        buf = ctx.scratch.get("diff_split") if hasattr(ctx, "scratch") else None
        if buf is None or buf.numel() * 4 < need:
            buf = torch.empty((need + 3) // 4, dtype=torch.float32, device=q.device)
            if hasattr(ctx, "scratch"):
                ctx.scratch["diff_split"] = buf
        scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel() * 4
    if once:
        code = lib.ib_attention_diff_decode(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), ctx.cu_rows.data_ptr(),
            ctx.positions.data_ptr(), tables.data_ptr(), tables.shape[1], ctx.n_entries, n_heads, nkv, page_size,
            num_pages, float(scale), float(softcap or 0.0), float(lam), float(eps), float(out_scale), rt.err.data_ptr(),
            N, splits, slice_len, scratch_ptr, scratch_bytes, core.stream_ptr(q))
        core.check(code, "attention_diff_decode")
        core.profile_mark("attention_diff_decode")
        return True
    code = lib.ib_attention_diff_mma(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), ctx.cu_rows.data_ptr(),
        ctx.positions.data_ptr(), tables.data_ptr(), tables.shape[1], ctx.n_entries, ctx.max_rows_per_entry, n_heads, nkv,
        page_size, num_pages, float(scale), float(softcap or 0.0), float(lam), float(eps), float(out_scale),
        rt.err.data_ptr(), N, splits, slice_len, scratch_ptr, scratch_bytes, core.stream_ptr(q))
    core.check(code, "attention_diff_mma")
    core.profile_mark("attention_diff_mma")
    return True
