"""The tensor-core kernel for differential attention (``attention_diff_mma.cu``),
one compiled module per (map size, value size), built when a model first needs it.

``run`` returns False when the sizes have no variant (bfloat16; map and value
sizes multiples of 16, at most 256) or ``rt.options["attention"] == "plain"``;
the caller then takes the plain 32-bit kernel (``core.attention_diff``).
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
            _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_float, _c_float, _c_void_p, _c_void_p]
        lib.ib_attention_diff_mma.restype = _c_int
        if lib.ib_attention_diff_mma_d() != dim or lib.ib_attention_diff_mma_e() != vdim:
            raise KernelError(f"differential attention module for ({dim}, {vdim}) was built for other sizes")
        _libs[(dim, vdim)] = lib
    return lib


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
    code = lib.ib_attention_diff_mma(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), ctx.cu_rows.data_ptr(),
        ctx.positions.data_ptr(), tables.data_ptr(), tables.shape[1], ctx.n_entries, ctx.max_rows_per_entry, n_heads, nkv,
        page_size, num_pages, float(scale), float(softcap or 0.0), float(lam), float(eps), float(out_scale),
        rt.err.data_ptr(), core.stream_ptr(q))
    core.check(code, "attention_diff_mma")
    core.profile_mark("attention_diff_mma")
    return True
