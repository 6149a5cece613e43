"""Time one kernel in isolation (CUDA events, after warm-up), for tuning and for ncu captures.

    python -m pagedserve_b200.kernels.microbench gemm --m 2048 --n 2304 --k 768 [--bn 0] [--impl tc|skinny|rows|simt]
    python -m pagedserve_b200.kernels.microbench attention --batch 64 --context 640 [--heads 12 --head-dim 64]

``gemm`` prints achieved TFLOP/s and the bytes-per-second of streaming the weight once;
``attention`` prints achieved GB/s over the K and V bytes of the contexts.  Inputs are rotated
over several buffers larger than L2 in total so that a repeat does not find its operands cached.
"""

from __future__ import annotations

import argparse
import math
import sys

import torch


def _time(fn, iters, warmup=3, graph=False):
    """Seconds per call.  ``graph``: the calls are captured into one CUDA graph and replayed, which takes
    the host's launch cost out of the figure (needed for kernels of a few microseconds)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            for i in range(iters):
                fn(i)
        captured.replay()
        torch.cuda.synchronize()
        start.record()
        for _ in range(5):
            captured.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / (5 * iters) * 1e-3
    start.record()
    for i in range(iters):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e-3


def bench_gemm(args):
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    M, N, K = args.m, args.n, args.k
    per_set = (M * K + N * K) * 2 + M * N * 4
    copies = max(2, min(64, int(160e6 // per_set) + 1))          # rotate operands past the 126 MB L2
    a = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    w = [(torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16) for _ in range(copies)]
    bias = torch.randn(N, device="cuda")
    out_dtype = torch.float32 if args.out == "float32" else torch.bfloat16
    out = torch.empty(M, N, dtype=out_dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = args.accumulate
    if args.norm:
        from types import SimpleNamespace

        from pagedserve_b200.parts.base import NormPrologue
        from pagedserve_b200.parts.norms import DeferredNorm

        prologue = NormPrologue(weight=torch.ones(K, device="cuda"), bias=torch.zeros(K, device="cuda"),
                                eps=1e-5, has_mean=True)
        norm = SimpleNamespace(fused_prologue=lambda: prologue)
        x32 = [t.float() for t in a]

    def run(i):
        j = i % copies
        if args.norm:
            ops.linear_skinny_fused(DeferredNorm(norm, x32[j]), w[j], bias, out, act=args.act, accumulate=acc)
        elif args.impl == "tc":
            ops.linear_tc(a[j], w[j], bias, out, act=args.act, accumulate=acc, status=status, bn=args.bn)
        elif args.impl == "skinny":
            ops.linear_skinny(a[j], w[j], bias, out, act=args.act, accumulate=acc)
        elif args.impl == "rows":
            ops.linear_rows_tc(a[j], w[j], bias, out, act=args.act, accumulate=acc, status=status, splits=args.splits)
        else:
            ops.linear_simt(a[j], w[j], bias, out, act=args.act, accumulate=acc)

    seconds = _time(run, args.iters, graph=args.graph)
    flops = 2.0 * M * N * K
    print(f"gemm {'skinny+norm' if args.norm else args.impl} M={M} N={N} K={K} bn={args.bn} out={args.out}"
          f"{' accumulate' if acc else ''}: {seconds * 1e6:.2f} us, "
          f"{flops / seconds / 1e12:.1f} TFLOP/s, weight stream {N * K * 2 / seconds / 1e9:.0f} GB/s, "
          f"status {int(status.item())}")


def bench_attention(args):
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    B, ctx, H, D, page = args.batch, args.context, args.heads, args.head_dim, args.page_size
    pages_per = -(-ctx // page)
    layers = max(1, min(48, int(200e6 // (B * pages_per * page * H * D * 4)) + 1))   # rotate layers past L2
    pool = torch.randn(B * pages_per + 1, layers, 2, H, page, D, device="cuda").to(torch.bfloat16)
    table = torch.randperm(B * pages_per, device="cuda").to(torch.int32).view(B, pages_per)
    q = torch.randn(B, H * D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    token_item = torch.arange(B, dtype=torch.int32, device="cuda")
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    stride = layers * 2 * H * page * D
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(i):
        layer = i % layers
        ops.paged_attention_decode(q, out, pool[:, layer, 0], pool[:, layer, 1], stride, token_item, positions, table,
                                   H, H, D, page, None, D ** -0.5, args.max_context or ctx, status=status)

    seconds = _time(run, args.iters, graph=args.graph)
    nbytes = B * ctx * H * D * 2 * 2
    print(f"decode attention B={B} ctx={ctx} heads={H} hd={D} page={page}: {seconds * 1e6:.2f} us, "
          f"{nbytes / seconds / 1e9:.0f} GB/s of K+V, status {int(status.item())}")


def main(argv=None):
    parser = argparse.ArgumentParser(prog="python -m pagedserve_b200.kernels.microbench")
    sub = parser.add_subparsers(dest="kind", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=2048)
    g.add_argument("--n", type=int, default=2304)
    g.add_argument("--k", type=int, default=768)
    g.add_argument("--bn", type=int, default=0)
    g.add_argument("--impl", default="tc", choices=("tc", "skinny", "rows", "simt"))
    g.add_argument("--splits", type=int, default=0, help="rows: CTAs per column tile (0: the kernel chooses)")
    g.add_argument("--act", default=None)
    g.add_argument("--out", default="bfloat16", choices=("bfloat16", "float32"))
    g.add_argument("--accumulate", action="store_true", help="add the product to what the output holds")
    g.add_argument("--norm", action="store_true",
                   help="the few-rows kernel with a LayerNorm of float32 rows fused in front")
    g.add_argument("--iters", type=int, default=50)
    g.add_argument("--graph", action="store_true", help="replay the calls as one CUDA graph")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=64)
    a.add_argument("--context", type=int, default=640)
    a.add_argument("--max-context", type=int, default=0)
    a.add_argument("--heads", type=int, default=12)
    a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--iters", type=int, default=50)
    a.add_argument("--graph", action="store_true", help="replay the calls as one CUDA graph")
    args = parser.parse_args(argv)
    if args.kind == "gemm":
        bench_gemm(args)
    else:
        bench_attention(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
