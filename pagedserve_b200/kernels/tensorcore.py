"""The bfloat16 paths of the matrix product and of attention.

``linear``    out = act(a @ w.T + bias) with bfloat16 operands and float32 accumulation:
              at most 64 rows -> the weight-streaming kernel (csrc/gemm_skinny.cu), except 17 to 64
                                 rows with 4,096 or more output columns;
              more rows       -> the tcgen05 / TMA / TMEM kernel (csrc/gemm_tc.cu);
              shapes neither takes (K not a multiple of 8, unaligned rows) -> the CUDA-core kernel.
``attention`` causal attention over the paged cache for bfloat16 queries.
"""

from __future__ import annotations


def prefers_tc(ops, a, w) -> bool:
    """Whether the tcgen05 kernel takes this product.  The weight-streaming kernel brings the rows of ``a`` to
    every CTA (16 output columns): from 17 rows on and 4,096 columns up (a vocabulary, the wide projections of
    large models) that traffic costs more than the half-empty 128-row tiles of the tcgen05 kernel (64 rows x
    50,257 x 768: 46 vs 85 us; 64 x 4,800 x 1,600: 12 vs 37 us; 16 rows: the streaming kernel wins at every
    shape)."""
    if not ops.tc_ok(a, w):
        return False
    return (a.shape[0] > 16 and w.shape[0] >= 4096) or not ops.skinny_ok(a, w)


def linear(ops, a, w, bias, out, act=None, accumulate=False, status=None):
    if prefers_tc(ops, a, w):
        return ops.linear_tc(a, w, bias, out, act, accumulate, status=status)
    if ops.skinny_ok(a, w):
        return ops.linear_skinny(a, w, bias, out, act, accumulate)
    return ops.linear_simt(a, w, bias, out, act, accumulate)


def attention(ops, q, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale):
    """Short entries (fewer than ``ctx.LONG_ENTRY`` tokens: decode tokens, short portions) come first in the
    step's flat batch and go token by token through the split-key kernel; long portions go through the
    tensor-core prefill kernel in blocks of 64 queries."""
    short_tokens = ctx.num_short_tokens
    long_items = ctx.num_items - ctx.num_short_items
    if long_items and head_dim > 128:
        short_tokens, long_items = ctx.num_tokens, 0
    if short_tokens:
        # few (token, head) pairs: one thread-block cluster per pair merges its splits through shared memory
        # (batch 1: 231 vs 250 us per step); from a few dozen pairs on, co-scheduling whole clusters costs
        # more than the trip through global memory that it saves (batch 8: 354 vs 317 us)
        merge = "cluster" if short_tokens * n_heads * 8 <= 148 else "global"
        ops.paged_attention_decode(q[:short_tokens], out[:short_tokens], layer.k_pool, layer.v_pool,
                                   layer.page_stride, ctx.token_item[:short_tokens], ctx.positions[:short_tokens],
                                   layer.block_table, n_heads, n_kv_heads, head_dim, layer.page_size, window, scale,
                                   ctx.max_kv_len, status=ctx.status, q_start=ctx.q_start, kv_len=ctx.kv_len, merge=merge,
                                   token_row=ctx.token_slot[:short_tokens])
    if long_items:
        if ops.prefill_tc_ok(head_dim, layer.page_size, q, out, getattr(layer, "pool", None)):
            # blocks of 128 queries: never more than the count of 64-query blocks
            # Two threads per query row halve the chain of each 128-key tile but leave one CTA per SM: worth it
            # when all blocks are resident at once, or nearly so while some block runs over many tiles.
            blocks = -(-ctx.num_long_blocks // 2) * n_heads          # an upper bound of the 128-query blocks
            two = blocks <= 148 or (blocks <= 296 and ctx.max_kv_len >= 768)
            ops.prefill_attention_tc(q, out, layer.pool, layer.pool_layer, ctx.q_start, ctx.kv_len, layer.block_table,
                                     ctx.num_short_items, long_items, ctx.num_long_blocks, n_heads, n_kv_heads,
                                     head_dim, layer.page_size, window, scale, status=ctx.status,
                                     row_threads=2 if two else 1, item_row=ctx.item_slot)
        else:
            ops.prefill_attention(q, out, layer.k_pool, layer.v_pool, layer.page_stride, ctx.q_start, ctx.kv_len,
                                  layer.block_table, ctx.num_short_items, long_items, ctx.num_long_blocks, n_heads,
                                  n_kv_heads, head_dim, layer.page_size, window, scale, item_row=ctx.item_slot)
    return out
