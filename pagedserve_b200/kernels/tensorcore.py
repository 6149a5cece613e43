"""The bfloat16 paths of the matrix product and of attention.

``linear``    out = act(a @ w.T + bias) with bfloat16 operands and float32 accumulation:
              at most 64 rows -> the weight-streaming kernel (csrc/gemm_skinny.cu), except
                                 33 to 64 rows of a large matrix -> the few-rows tcgen05 kernel with the
                                 operands swapped and K split over a cluster (csrc/gemm_rows_tc.cu), and
                                 17 to 47 rows with 4,096 or more output columns -> the kernel below;
              more rows       -> the tcgen05 / TMA / TMEM kernel (csrc/gemm_tc.cu);
              shapes neither takes (K not a multiple of 8, unaligned rows) -> the CUDA-core kernel.
``attention`` causal attention over the paged cache for bfloat16 queries.
"""

from __future__ import annotations


def prefers_rows(ops, a, w) -> bool:
    """Whether the few-rows tcgen05 kernel takes this product.  Its cost hardly depends on the rows (about 5 us
    of latency, then 64 tokens ride along with the weights), the mma.sync kernel's grows with every 8 rows and
    with the matrix.  Measured on B200 (us, weight-streaming / few-rows tcgen05 / 128-row tcgen05):
    64 x 2,304 x 768: 6.6 / 7.5 / 8.1;  64 x 768 x 3,072: 12.5 / 7.7 / 18.2;  56 x 768 x 3,072: 7.7 / 7.7 / 18.1;
    48 x 2,304 x 768: 4.8 / 7.0 / 8.1;  64 x 4,096 x 1,024: 11.8 / 7.9 / 9.4;  64 x 1,024 x 4,096: 17.6 / 9.0 / 22.8;
    64 x 4,800 x 1,600: 25.1 / 12.0 / 12.1;  64 x 1,600 x 6,400: 23.0 / 12.1 / 33.1;  33 x 4,800 x 1,600: 13.0 /
    10.7 / 12.2;  64 x 50,257 x 768: 73.9 / 35.6 / 45.5;  33 x 50,257 x 768: 35.6 / 31.5 / 30.6.
    The rule depends on the shapes alone, so that the same step always runs the same kernels."""
    rows, columns, depth = a.shape[0], w.shape[0], a.shape[1]
    if not (32 < rows <= 64) or not ops.tc_ok(a, w):
        return False
    if columns >= 4096:
        return rows >= 48
    return rows > 56 or columns * depth >= 2_500_000


def prefers_tc(ops, a, w) -> bool:
    """Whether the tcgen05 kernel takes this product.  The weight-streaming kernel brings the rows of ``a`` to
    every CTA (16 output columns): from 17 rows on and 4,096 columns up (a vocabulary, the wide projections of
    large models) that traffic costs more than the half-empty 128-row tiles of the tcgen05 kernel (64 rows x
    50,257 x 768: 46 vs 85 us; 64 x 4,800 x 1,600: 12 vs 37 us; 16 rows: the streaming kernel wins at every
    shape)."""
    if not ops.tc_ok(a, w) or prefers_rows(ops, a, w):
        return False
    return (a.shape[0] > 16 and w.shape[0] >= 4096) or not ops.skinny_ok(a, w)


def linear(ops, a, w, bias, out, act=None, accumulate=False, status=None):
    if prefers_rows(ops, a, w):
        return ops.linear_rows_tc(a, w, bias, out, act, accumulate, status=status)
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
        # The splits of a (token, head) pair merge through global memory. (With at most one pair per SM the
        # kernel makes one CTA of six teams per pair instead and merges in shared memory: batch 8, 278 -> 259 us
        # per step. One thread-block cluster per pair, which the kernel also offers, lost to both: co-scheduling
        # whole clusters costs more than the trip through memory it saves, 354 vs 317 us at batch 8 when measured,
        # and 4,636 vs 4,734 tokens/s at batch 1 against the teams.)
        merge = "global"
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
