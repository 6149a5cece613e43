"""The bfloat16 paths of the matrix product and of attention.

``linear``    out = act(a @ w.T + bias) with bfloat16 operands and float32 accumulation:
              at most 64 rows -> the weight-streaming kernel (csrc/gemm_skinny.cu);
              more rows       -> the tcgen05 kernel (csrc/gemm_tc.cu) when it takes the shape,
                                 else the CUDA-core kernel.
``attention`` causal attention over the paged cache for bfloat16 queries.
"""

from __future__ import annotations

import torch


def linear(ops, a, w, bias, out, act=None, accumulate=False):
    if ops.skinny_ok(a, w):
        return ops.linear_skinny(a, w, bias, out, act, accumulate)
    return ops.linear_simt(a, w, bias, out, act, accumulate)


def attention(ops, q, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale):
    return ops.paged_attention_decode(q, out, layer.k_pool, layer.v_pool, layer.page_stride, ctx.token_item,
                                      ctx.positions, layer.block_table, n_heads, n_kv_heads, head_dim,
                                      layer.page_size, window, scale, ctx.max_kv_len, status=ctx.status)
