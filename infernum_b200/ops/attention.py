"""Chooses the attention kernel for a step.

``float32`` engines always take the plain kernel (one warp per row and head,
32-bit throughout).  ``bfloat16`` engines take the tensor-core prefill kernel
and the split-KV decode kernel when the head size has a compiled variant, and
the plain kernel otherwise; ``rt.options["attention"] = "plain"`` forces the
plain kernel (tests use it to compare the two).
"""

from __future__ import annotations

import torch

from . import core


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    out: torch.Tensor, ctx, tables: torch.Tensor, n_heads: int, scale: float,
                    window: int, rt, sink=None, keep_first: int = 0) -> None:
    """Attention of every row of the step over its request's pages.

    ``q`` holds the (already position-encoded) queries in its first
    ``n_heads * head_dim`` columns; keys and values of the step's own tokens
    are already in the pools.  ``sink`` (float32 [n_heads]): a logit per head
    whose exponential is added to the softmax's denominator.  ``keep_first``:
    behind a window, the keys at positions below it stay visible.  Values may
    have another size than keys (the value pool's last dimension)."""
    impl = rt.options.get("attention", "auto")
    if q.dtype == torch.bfloat16 and impl != "plain":
        from . import attention_fast

        if attention_fast.run(q, k_pool, v_pool, out, ctx, tables, n_heads, scale, window, rt, sink=sink,
                              keep_first=keep_first):
            return
    core.attention_plain(q, k_pool, v_pool, out, ctx.positions, ctx.row_entry, tables, n_heads,
                         scale, window, rt.err, sink=sink, keep_first=keep_first)


def latent_attention(q_abs: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, kv_rank: int, ctx,
                     tables: torch.Tensor, scale: float, window: int, rt) -> None:
    """Attention of every head of every row over its request's cached latents.

    ``q_abs`` [N, heads, kv_rank + rot_dim] holds each head's query in latent
    space followed by its rotated part; the pool [pages, 1, page_size,
    kv_rank + rot_dim] each token's latent followed by the shared rotated key;
    ``out`` [N, heads, kv_rank] receives the weighted sums of latents.  Rows and
    heads may lie in any order in memory (strides).  bfloat16 engines take the
    tensor-core kernel when the sizes have a variant, everything else the plain
    32-bit kernel; ``rt.options["attention"] = "plain"`` forces the latter."""
    impl = rt.options.get("attention", "auto")
    if q_abs.dtype == torch.bfloat16 and impl != "plain":
        from . import attention_latent

        if attention_latent.run(q_abs, pool, out, kv_rank, ctx, tables, scale, window, rt):
            return
    core.attention_latent_plain(q_abs, pool, out, kv_rank, ctx.positions, ctx.row_entry, tables, scale,
                                window, rt.err)
