"""Each kernel alone against a plain float64 reference, at sizes other than the engine's."""

import math
import random

import pytest
import torch

import plain_gpt2

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops_for(dtype):
    from pagedserve_b200.kernels.ops import Ops

    return Ops(dtype)


def rel_err(got, want):
    want = want.double().cpu()
    return float((got.double().cpu() - want).abs().max() / max(1e-30, float(want.abs().max())))


# ------------------------------------------------------------------ embedding, norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 200, 768])
def test_embed(dtype, H):
    ops = ops_for(dtype)
    g = torch.Generator().manual_seed(1)
    wte = torch.randn(301, H, generator=g).to(dtype)
    wpe = torch.randn(77, H, generator=g).to(dtype)
    ids = torch.randint(0, 301, (53,), generator=g, dtype=torch.int32)
    pos = torch.randint(0, 77, (53,), generator=g, dtype=torch.int32)
    out = torch.empty(53, H, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(ids.to(DEV), pos.to(DEV), wte.to(DEV), wpe.to(DEV), out, status)
    want = wte.float()[ids.long()] + wpe.float()[pos.long()]
    assert torch.equal(out.cpu(), want) and int(status.item()) == 0
    ops.embed(ids.to(DEV), pos.to(DEV), wte.to(DEV), None, out, status)
    assert torch.equal(out.cpu(), wte.float()[ids.long()])
    bad = ids.clone(); bad[7] = 301
    ops.embed(bad.to(DEV), pos.to(DEV), wte.to(DEV), wpe.to(DEV), out, status)
    assert int(status.item()) == 1 and float(out[7].abs().max()) == 0.0      # flagged, not read out of range


@pytest.mark.parametrize("H", [16, 96, 200, 768, 1600, 2500])
@pytest.mark.parametrize("eps", [1e-5, 1e-6])
def test_layernorm(H, eps):
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(H)
    x = (torch.randn(37, H, generator=g) * 3 + 1.5)
    gamma, beta = torch.randn(H, generator=g), torch.randn(H, generator=g)
    want = plain_gpt2.layer_norm(x.double(), gamma.double(), beta.double(), eps)
    out32 = torch.empty(37, H, dtype=torch.float32, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out32)
    assert rel_err(out32, want) < 2e-6
    out16 = torch.empty(37, H, dtype=torch.bfloat16, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out16)
    assert rel_err(out16, want) < 5e-3
    rows = torch.tensor([36, 0, 5], dtype=torch.int32)
    picked = torch.empty(3, H, dtype=torch.float32, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, picked, rows=rows.to(DEV))
    assert torch.equal(picked.cpu(), out32.cpu()[rows.long()])
    rms = torch.empty(37, H, dtype=torch.float32, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), None, eps, rms, has_mean=False)
    want_rms = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * gamma.double()
    assert rel_err(rms, want_rms) < 2e-6


# ------------------------------------------------------------------ matrix products
def gemm_reference(a, w, bias, act, base):
    y = a.double() @ w.double().T
    if bias is not None:
        y = y + bias.double()
    if act == "gelu_tanh":
        y = plain_gpt2.activation(y, "gelu_new")
    elif act == "gelu_erf":
        y = plain_gpt2.activation(y, "gelu")
    if base is not None:
        y = y + base.double()
    return y


@pytest.mark.parametrize("M,N,K", [(1, 17, 8), (5, 130, 72), (70, 257, 100), (200, 96, 333)])
@pytest.mark.parametrize("act", [None, "gelu_tanh", "gelu_erf"])
def test_gemm_simt_float32(M, N, K, act):
    ops = ops_for(torch.float32)
    g = torch.Generator().manual_seed(M * N)
    a, w, bias = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(a.to(DEV), w.to(DEV), bias.to(DEV), out, act=act)
    assert rel_err(out, gemm_reference(a, w, bias, act, None)) < 3e-6
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_simt(a.to(DEV), w.to(DEV), None, stream, accumulate=True)
    assert rel_err(stream, gemm_reference(a, w, None, None, base)) < 3e-6
    # a row's result does not depend on the rows beside it
    alone = torch.empty(1, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(a[M - 1:].to(DEV), w.to(DEV), bias.to(DEV), alone, act=act)
    assert torch.equal(alone[0], out[M - 1])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 31, 40, 64])
@pytest.mark.parametrize("N,K", [(48, 64), (1003, 96), (300, 320), (2304, 768), (770, 3072), (33, 4104),
                                 (160, 6400), (768, 768)])
def test_gemm_skinny(M, N, K):
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    for act, out_dtype, tol in ((None, torch.float32, 2e-5), ("gelu_tanh", torch.bfloat16, 6e-3),
                                ("gelu_erf", torch.bfloat16, 6e-3)):
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.linear_skinny(a.to(DEV), w.to(DEV), bias.to(DEV), out, act=act)
        assert rel_err(out, gemm_reference(a, w, bias, act, None)) < tol, (act, out_dtype)
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_skinny(a.to(DEV), w.to(DEV), bias.to(DEV), stream, accumulate=True)
    assert rel_err(stream, gemm_reference(a, w, bias, None, base)) < 2e-5
    # against the CUDA-core product with the same bfloat16 inputs: float32 sums in another order
    simt = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fast = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(a.to(DEV), w.to(DEV), None, simt)
    ops.linear_skinny(a.to(DEV), w.to(DEV), None, fast)
    assert rel_err(fast, simt) < 1e-5


@pytest.mark.parametrize("M,N,K", [(65, 64, 64), (128, 256, 64), (130, 1003, 96), (300, 320, 328),
                                   (1024, 2304, 768), (257, 770, 3072), (2048, 96, 1600)])
@pytest.mark.parametrize("bn", [0, 64, 128, 192, 256])
def test_gemm_tcgen05(M, N, K, bn):
    """The tcgen05/TMA/TMEM product against the CUDA-core product on the same bfloat16 inputs (both
    accumulate in float32) and against float64: tails in M, N and K, every tile width, all epilogues."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + N + K + bn)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for act, out_dtype, tol in ((None, torch.float32, 2e-5), ("gelu_tanh", torch.bfloat16, 6e-3),
                                ("gelu_erf", torch.float32, 2e-5)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), out, act=act, status=status, bn=bn)
        assert rel_err(out, gemm_reference(a, w, bias, act, None)) < tol, (act, out_dtype)
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_tc(a.to(DEV), w.to(DEV), None, stream, accumulate=True, status=status, bn=bn)
    assert rel_err(stream, gemm_reference(a, w, None, None, base)) < 2e-5
    simt = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fast = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(a.to(DEV), w.to(DEV), None, simt)
    ops.linear_tc(a.to(DEV), w.to(DEV), None, fast, status=status, bn=bn)
    assert rel_err(fast, simt) < 1e-5
    # a row's result does not depend on the rows beside it
    rows = min(70, M)
    part = torch.empty(rows, N, dtype=torch.float32, device=DEV)
    ops.linear_tc(a[M - rows:].to(DEV), w.to(DEV), None, part, status=status, bn=bn)
    assert torch.equal(part, fast[M - rows:])
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,K", [(2048, 768, 768), (257, 770, 3072), (130, 1003, 96), (300, 96, 64)])
def test_gemm_tcgen05_96_wide(M, N, K):
    """Tiles of 96 columns exist for float32 outputs (three 32-column groups of the epilogue); a bfloat16
    output is refused at that width."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for act in (None, "gelu_erf"):
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), out, act=act, status=status, bn=96)
        assert rel_err(out, gemm_reference(a, w, bias, act, None)) < 2e-5
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), stream, accumulate=True, status=status, bn=96)
    assert rel_err(stream, gemm_reference(a, w, bias, None, base)) < 2e-5
    other = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), out, status=status, bn=96)
    ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), other, status=status, bn=128)
    assert torch.equal(out, other)                        # the tile width does not change a sum
    assert int(status.item()) == 0
    from pagedserve_b200.kernels.ops import KernelError
    with pytest.raises(KernelError):
        ops.linear_tc(a.to(DEV), w.to(DEV), bias.to(DEV), torch.empty(M, N, dtype=torch.bfloat16, device=DEV),
                      status=status, bn=96)


@pytest.mark.parametrize("M", [1, 8, 9, 16, 25, 32])
@pytest.mark.parametrize("N,K", [(288, 96), (2304, 768), (1000, 320), (768, 3072), (312, 104), (96, 328)])
def test_gemm_skinny_with_fused_norm_and_cache_write(M, N, K):
    """norm -> product in one kernel against norm kernel + product, with gathered rows, the RMS form, and
    the key/value columns of a packed projection landing in the right page slots."""
    from pagedserve_b200.parts.norms import DeferredNorm

    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = (torch.randn(M + 5, K, generator=g) * 2 + 0.7).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    rows = torch.randperm(M + 5, generator=g)[:M].to(torch.int32).to(DEV)

    class FakeNorm:
        def __init__(self, has_mean, has_bias):
            self.weight = (torch.randn(K, generator=g) * 0.1 + 1).to(DEV)
            self.bias = torch.randn(K, generator=g).to(DEV) if has_bias else None
            self.params = {"eps": 1e-5, "has_mean": has_mean}

        def forward(self, x, out=None, rows=None):
            count = rows.numel() if rows is not None else x.shape[0]
            out = torch.empty(count, K, dtype=torch.bfloat16, device=DEV)
            return ops.layernorm(x, self.weight, self.bias, 1e-5, out, rows=rows, has_mean=self.params["has_mean"])

        def fused_prologue(self):
            # any norm, whatever its class, that says how a product can compute it in its prologue is folded in
            from pagedserve_b200.parts.base import NormPrologue

            return NormPrologue(self.weight, self.bias, 1e-5, self.params["has_mean"])

    for has_mean, has_bias, use_rows in ((True, True, False), (False, False, True), (True, True, True)):
        norm = FakeNorm(has_mean, has_bias)
        deferred = DeferredNorm(norm, x if use_rows else x[:M], rows if use_rows else None)
        # bytes of normed rows and of the norm's scale and shift in shared memory
        staged = (8 if M <= 8 else 16 if M <= 16 else 32) * (K + 8) * 2 + 8 * K
        assert ops._fused_norm_ok(deferred, w) == (staged <= 96 * 1024)
        if staged > 160 * 1024:
            continue                                                            # beyond what the kernel takes
        fused = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops.linear_skinny_fused(deferred, w, bias, fused, act="gelu_tanh")
        separate = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops.linear_skinny(deferred.materialize(), w, bias, separate, act="gelu_tanh")
        # same bfloat16 roundings of the normed input up to float32 reassociation in the statistics
        assert rel_err(fused, separate) < 4e-3
        picked = x[rows.long()] if use_rows else x[:M]
        xd = picked.double().cpu()
        if has_mean:
            normed = plain_gpt2.layer_norm(xd, norm.weight.double().cpu(), norm.bias.double().cpu(), 1e-5)
        else:
            normed = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * norm.weight.double().cpu()
        assert rel_err(fused, gemm_reference(normed, w.cpu(), bias.cpu(), "gelu_tanh", None)) < 8e-3
    fits = (8 if M <= 8 else 16 if M <= 16 else 32) * (K + 8) * 2 + 8 * K <= 96 * 1024
    if N % 3 == 0 and (N // 3) % 16 == 0 and fits:
        # packed projection: q to the buffer, k and v into pages
        width = N // 3
        head_dim = 16 if width % 48 else 48
        kv_heads = width // head_dim
        page = 8
        lengths = [3 + 2 * i for i in range(M)]                 # every token is the last of its own request
        pages = [-(-n // page) for n in lengths]
        table = torch.full((M, max(pages)), -1, dtype=torch.int32)
        order = torch.randperm(sum(pages), generator=g)
        cursor = 0
        for i, count in enumerate(pages):
            table[i, :count] = order[cursor:cursor + count].to(torch.int32)
            cursor += count
        pool = torch.zeros(sum(pages), 1, 2, kv_heads, page, head_dim, dtype=torch.bfloat16, device=DEV)

        class Ctx:
            token_item = torch.arange(M, dtype=torch.int32, device=DEV)
            token_slot = token_item                       # this table is by item: a token's row is its item
            positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)

        class Layer:
            k_pool, v_pool = pool[:, 0, 0], pool[:, 0, 1]
            page_stride = 2 * kv_heads * page * head_dim
            page_size = page
            block_table = table.to(DEV)

        norm = FakeNorm(True, True)
        deferred = DeferredNorm(norm, x[:M])
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        assert ops.linear_qkv(deferred, w, bias, out, Ctx, Layer, width, width, head_dim, scatter=True)
        want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ops.linear_skinny(deferred.materialize(), w, bias, want)
        assert rel_err(out[:, :width], want[:, :width]) < 8e-3
        assert float(out[:, width:].abs().max()) == 0.0           # keys and values did not go to the buffer
        for i, n in enumerate(lengths):
            slot = pool[int(table[i, (n - 1) // page]), 0, :, :, (n - 1) % page, :].reshape(2, width)
            assert rel_err(slot[0], want[i, width:2 * width]) < 8e-3
            assert rel_err(slot[1], want[i, 2 * width:]) < 8e-3
        assert int((pool != 0).sum()) <= 2 * M * width             # nothing else was touched


@pytest.mark.parametrize("M", [17, 24, 25, 33, 41, 47, 49, 57])
@pytest.mark.parametrize("N,K", [(48, 8), (300, 328), (1003, 104), (2304, 768), (770, 3080), (160, 6400)])
def test_gemm_skinny_every_count_of_row_tiles(M, N, K):
    """Row counts that fall into each instance of the few-rows product (3 to 8 tiles of 8 rows), with widths
    that are no multiple of 32: against float64 and against the CUDA-core product on the same inputs."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(3 * M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    for act, out_dtype, tol in ((None, torch.float32, 2e-5), ("gelu_tanh", torch.bfloat16, 6e-3)):
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.linear_skinny(a, w, bias, out, act=act)
        assert rel_err(out, gemm_reference(a.cpu(), w.cpu(), bias.cpu(), act, None)) < tol, (act, out_dtype)
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_skinny(a, w, bias, stream, accumulate=True)
    assert rel_err(stream, gemm_reference(a.cpu(), w.cpu(), bias.cpu(), None, base)) < 2e-5
    simt = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fast = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(a, w, None, simt)
    ops.linear_skinny(a, w, None, fast)
    assert rel_err(fast, simt) < 1e-5


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("width,head_dim,K", [(96, 48, 96), (768, 64, 768), (160, 16, 264)])
def test_gemm_skinny_writes_the_cache(M, width, head_dim, K):
    """The packed q|k|v projection of 17 to 64 rows, too many for the norm to be folded in: queries to the
    buffer, keys and values into the pages."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + width + K)
    N = 3 * width
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    kv_heads = width // head_dim
    page = 8
    lengths = [3 + 2 * i for i in range(M)]                 # every token is the last of its own request
    pages = [-(-n // page) for n in lengths]
    table = torch.full((M, max(pages)), -1, dtype=torch.int32)
    order = torch.randperm(sum(pages), generator=g)
    cursor = 0
    for i, count in enumerate(pages):
        table[i, :count] = order[cursor:cursor + count].to(torch.int32)
        cursor += count
    pool = torch.zeros(sum(pages), 1, 2, kv_heads, page, head_dim, dtype=torch.bfloat16, device=DEV)

    class Ctx:
        token_item = torch.arange(M, dtype=torch.int32, device=DEV)
        token_slot = token_item                           # this table is by item: a token's row is its item
        positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)

    class Layer:
        k_pool, v_pool = pool[:, 0, 0], pool[:, 0, 1]
        page_stride = 2 * kv_heads * page * head_dim
        page_size = page
        block_table = table.to(DEV)

    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    assert ops.linear_qkv(a, w, bias, out, Ctx, Layer, width, width, head_dim, scatter=True)
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, bias, want)                              # the kernel that the dispatch picks for this shape
    assert torch.equal(out[:, :width], want[:, :width])       # the same kernel: the same sums in the same order
    assert float(out[:, width:].abs().max()) == 0.0           # keys and values did not go to the buffer
    for i, n in enumerate(lengths):
        slot = pool[int(table[i, (n - 1) // page]), 0, :, :, (n - 1) % page, :].reshape(2, width)
        assert torch.equal(slot[0], want[i, width:2 * width])
        assert torch.equal(slot[1], want[i, 2 * width:])
    assert int((pool != 0).sum()) <= 2 * M * width             # nothing else was touched


@pytest.mark.parametrize("M", [1, 16, 17, 33, 40, 48, 49, 64])
@pytest.mark.parametrize("N,K", [(128, 64), (48, 8), (300, 328), (1003, 104), (2304, 768), (768, 3072), (1600, 6400),
                                 (4800, 1600)])
@pytest.mark.parametrize("splits", [0, 1, 2, 8])
def test_gemm_rows_tcgen05(M, N, K, splits):
    """The few-rows tcgen05 product (weight rows on the 128-row side of the MMA, K split over the CTAs of a
    cluster) against float64 and the CUDA-core product: tails in N and K, every count of token rows, every
    split (some CTAs then have no k-block at all), all epilogues."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    da, dw, db = a.to(DEV), w.to(DEV), bias.to(DEV)
    for act, out_dtype, tol in ((None, torch.float32, 2e-5), ("gelu_tanh", torch.bfloat16, 6e-3),
                                ("gelu_erf", torch.float32, 2e-5)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops.linear_rows_tc(da, dw, db, out, act=act, status=status, splits=splits)
        assert rel_err(out, gemm_reference(a, w, bias, act, None)) < tol, (act, out_dtype)
    base = torch.randn(M, N, generator=g)
    stream = base.clone().to(DEV)
    ops.linear_rows_tc(da, dw, db, stream, accumulate=True, status=status, splits=splits)
    assert rel_err(stream, gemm_reference(a, w, bias, None, base)) < 2e-5
    simt = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fast = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_simt(da, dw, None, simt)
    ops.linear_rows_tc(da, dw, None, fast, status=status, splits=splits)
    assert rel_err(fast, simt) < 2e-5                      # two float32 sums of up to 6,400 terms in different orders
    # a row's result does not depend on the rows beside it, nor on how many there are
    for rows in (1, min(M, 20)):
        part = torch.empty(rows, N, dtype=torch.float32, device=DEV)
        ops.linear_rows_tc(da[M - rows:].contiguous(), dw, None, part, status=status, splits=splits)
        assert torch.equal(part, fast[M - rows:])
    assert int(status.item()) == 0


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("width,head_dim,K", [(96, 48, 96), (768, 64, 768), (160, 16, 264), (1600, 64, 1600)])
def test_gemm_rows_tcgen05_writes_the_cache(M, width, head_dim, K):
    """The packed q|k|v projection through the few-rows tcgen05 product: queries to the buffer, keys and values
    into the pages of each token's request, nothing else touched."""
    ops = ops_for(torch.bfloat16)
    g = torch.Generator().manual_seed(M + width + K)
    N = 3 * width
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    kv_heads = width // head_dim
    page = 8
    lengths = [3 + 2 * i for i in range(M)]                 # every token is the last of its own request
    pages = [-(-n // page) for n in lengths]
    rows_of = torch.randperm(M + 3, generator=g)[:M]        # the table is kept by slot: token i uses row rows_of[i]
    table = torch.full((M + 3, max(pages)), -1, dtype=torch.int32)
    order = torch.randperm(sum(pages), generator=g)
    cursor = 0
    for i, count in enumerate(pages):
        table[rows_of[i], :count] = order[cursor:cursor + count].to(torch.int32)
        cursor += count
    pool = torch.zeros(sum(pages), 1, 2, kv_heads, page, head_dim, dtype=torch.bfloat16, device=DEV)

    class Ctx:
        token_slot = rows_of.to(torch.int32).to(DEV)
        positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)

    class Layer:
        k_pool, v_pool = pool[:, 0, 0], pool[:, 0, 1]
        page_stride = 2 * kv_heads * page * head_dim
        page_size = page
        block_table = table.to(DEV)

    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear_rows_tc(a, w, bias, out, kv=(Ctx, Layer, width, width, head_dim))
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear_rows_tc(a, w, bias, want)
    assert torch.equal(out[:, :width], want[:, :width])       # the same kernel: the same sums in the same order
    assert float(out[:, width:].abs().max()) == 0.0           # keys and values did not go to the buffer
    for i, n in enumerate(lengths):
        slot = pool[int(table[rows_of[i], (n - 1) // page]), 0, :, :, (n - 1) % page, :].reshape(2, width)
        assert torch.equal(slot[0], want[i, width:2 * width])
        assert torch.equal(slot[1], want[i, 2 * width:])
    assert int((pool != 0).sum()) <= 2 * M * width             # nothing else was touched
    reference = gemm_reference(a.cpu(), w.cpu(), bias.cpu(), None, None)
    assert rel_err(want, reference) < 6e-3
    assert int(ops.status_flag(DEV).item()) == 0


def test_gemm_skinny_refuses_what_it_cannot_take():
    from pagedserve_b200.kernels.ops import KernelError

    ops = ops_for(torch.bfloat16)
    a = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="unsupported"):
        ops.linear_skinny(a, w, None, torch.empty(65, 32, dtype=torch.float32, device=DEV))
    a = torch.zeros(4, 36, dtype=torch.bfloat16, device=DEV)          # K not a multiple of 8
    w = torch.zeros(32, 36, dtype=torch.bfloat16, device=DEV)
    assert not ops.skinny_ok(a, w)
    out = torch.empty(4, 32, dtype=torch.float32, device=DEV)
    ops.linear(a, w, None, out)                                       # falls to the CUDA-core kernel
    assert float(out.abs().max()) == 0.0


# ------------------------------------------------------------------ paged cache + attention
class PagedCase:
    """Sequences with their own q, k, v; a fragmented page pool filled through kv_append."""

    def __init__(self, ops, dtype, lengths, n_heads, n_kv_heads, head_dim, page_size, seed, spike=None):
        g = torch.Generator().manual_seed(seed)
        self.ops, self.dtype = ops, dtype
        self.n_heads, self.n_kv_heads, self.head_dim, self.page_size = n_heads, n_kv_heads, head_dim, page_size
        self.lengths = lengths
        T = sum(lengths)
        self.q = torch.randn(T, n_heads * head_dim, generator=g).to(dtype)
        self.k = torch.randn(T, n_kv_heads * head_dim, generator=g).to(dtype)
        self.v = torch.randn(T, n_kv_heads * head_dim, generator=g).to(dtype)
        if spike is not None:
            # make one far key dominate the last query of sequence 0: a kernel that skips it shows
            far, head = spike
            last = lengths[0] - 1
            group = head // (n_heads // n_kv_heads)
            direction = torch.randn(head_dim, generator=g)
            direction = direction / direction.norm()
            self.q[last, head * head_dim:(head + 1) * head_dim] = (direction * 12).to(dtype)
            self.k[far, group * head_dim:(group + 1) * head_dim] = (direction * 12).to(dtype)
        max_pages = max(-(-length // page_size) for length in lengths)
        total_pages = sum(-(-length // page_size) for length in lengths) + 3
        order = list(range(total_pages))
        random.Random(seed).shuffle(order)                      # fragmented tables
        table = torch.full((len(lengths), max_pages + 2), -1, dtype=torch.int32)
        cursor = 0
        token_item, positions = [], []
        for item, length in enumerate(lengths):
            pages = -(-length // page_size)
            table[item, :pages] = torch.tensor(order[cursor:cursor + pages], dtype=torch.int32)
            cursor += pages
            token_item += [item] * length
            positions += list(range(length))
        self.table = table.to(DEV)
        self.token_item = torch.tensor(token_item, dtype=torch.int32, device=DEV)
        self.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
        # pool [pages, 1 layer, 2, kv heads, page, hd], poisoned so that a stale read shows
        self.pool = torch.full((total_pages, 1, 2, n_kv_heads, page_size, head_dim), float("nan"),
                               dtype=dtype, device=DEV)
        self.page_stride = 2 * n_kv_heads * page_size * head_dim
        self.k_pool, self.v_pool = self.pool[:, 0, 0], self.pool[:, 0, 1]
        ops.kv_append(self.k.to(DEV), self.v.to(DEV), self.token_item, self.positions, self.table, self.k_pool,
                      self.v_pool, self.page_stride, n_kv_heads, head_dim, page_size)

    def reference(self, window=None):
        rows = []
        start = 0
        rep = self.n_heads // self.n_kv_heads
        for length in self.lengths:
            sl = slice(start, start + length)
            q = self.q[sl].double().reshape(length, self.n_heads, self.head_dim)
            k = self.k[sl].double().reshape(length, self.n_kv_heads, self.head_dim).repeat_interleave(rep, 1)
            v = self.v[sl].double().reshape(length, self.n_kv_heads, self.head_dim).repeat_interleave(rep, 1)
            rows.append(plain_gpt2.causal_attention(q, k, v, window=window))
            start += length
        return torch.cat(rows)


def test_kv_append_places_every_row():
    ops = ops_for(torch.float32)
    case = PagedCase(ops, torch.float32, [5, 17, 40], 4, 2, 16, 8, seed=3)
    pool = case.pool.cpu()
    start = 0
    for item, length in enumerate(case.lengths):
        for p in range(length):
            page = int(case.table[item, p // 8])
            got_k = pool[page, 0, 0, :, p % 8, :].reshape(-1)
            got_v = pool[page, 0, 1, :, p % 8, :].reshape(-1)
            assert torch.equal(got_k, case.k[start + p]) and torch.equal(got_v, case.v[start + p])
        start += length
    assert int(torch.isnan(pool).sum()) > 0          # untouched slots stay untouched


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 4, 16, 16), (2, 2, 48, 8), (6, 2, 64, 16),
                                                          (3, 1, 128, 32), (2, 2, 256, 4)])
@pytest.mark.parametrize("window", [None, 19])
def test_attention_simt_float32(heads, kv_heads, head_dim, page, window):
    ops = ops_for(torch.float32)
    lengths = [1, 15, 16, 17, 31, 32, 33, 128, 200]
    case = PagedCase(ops, torch.float32, lengths, heads, kv_heads, head_dim, page, seed=head_dim + page)
    out = torch.empty(sum(lengths), heads * head_dim, dtype=torch.float32, device=DEV)
    ops.paged_attention_simt(case.q.to(DEV), out, case.k_pool, case.v_pool, case.page_stride, case.token_item,
                             case.positions, case.table, heads, kv_heads, head_dim, page, window,
                             head_dim ** -0.5)
    assert torch.isfinite(out).all()
    assert rel_err(out, case.reference(window)) < 3e-6


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 4, 16, 16), (2, 2, 48, 8), (12, 12, 64, 16),
                                                          (8, 2, 128, 32), (2, 1, 256, 64)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("target_ctas,merge", [(1, "global"), (1184, "global"), (10 ** 7, "global"),
                                               (1184, "cluster"), (10 ** 7, "cluster")])
def test_attention_decode_bfloat16(heads, kv_heads, head_dim, page, window, target_ctas, merge):
    """Contexts around page and chunk edges, fragmented tables, one split up to a split per chunk; the splits
    merged through global memory or inside a thread-block cluster."""
    ops = ops_for(torch.bfloat16)
    lengths = [1, 15, 16, 17, 31, 32, 33, 64, 65, 127, 128, 129, 512, 1024]
    case = PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=7 + head_dim)
    out = torch.empty(sum(lengths), heads * head_dim, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_decode(case.q.to(DEV), out, case.k_pool, case.v_pool, case.page_stride, case.token_item,
                               case.positions, case.table, heads, kv_heads, head_dim, page, window,
                               head_dim ** -0.5, max(lengths), target_ctas=target_ctas, merge=merge)
    assert torch.isfinite(out.float()).all()
    assert rel_err(out, case.reference(window)) < 8e-3
    assert int(ops._counters.abs().sum()) == 0 if ops._counters is not None else True


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 4, 16, 16), (12, 12, 64, 16), (8, 2, 128, 32),
                                                          (2, 2, 48, 8)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("target_ctas", [1, 400, 10 ** 7])
@pytest.mark.parametrize("merge", ["global", "cluster"])
def test_attention_decode_with_older_keys_fetched_early(heads, kv_heads, head_dim, page, window, target_ctas, merge):
    """Decode tokens and short portions at the end of long requests: with q_start / kv_len the kernel may
    fetch a chunk made of older keys only before it waits for the kernel in front of it. The newest keys are
    written by a kernel launched right before, so a chunk fetched too early would show stale (NaN) rows."""
    ops = ops_for(torch.bfloat16)
    lengths = [1, 16, 17, 128, 129, 300, 640, 1024]
    fresh = [1, 1, 3, 1, 2, 5, 1, 15]
    case = PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=11 + head_dim)
    rows, item_of, q_start = [], [], [0]
    start = 0
    for item, (length, new) in enumerate(zip(lengths, fresh)):
        rows += list(range(start + length - new, start + length))
        item_of += [item] * new
        q_start.append(q_start[-1] + new)
        start += length
    rows_dev = torch.tensor(rows, device=DEV)
    q = case.q.to(DEV)[rows_dev].contiguous()
    token_item = torch.tensor(item_of, dtype=torch.int32, device=DEV)
    positions = case.positions[rows_dev].contiguous()
    # poison the new keys, then write them again right before the attention launch
    k_new, v_new = case.k.to(DEV)[rows_dev].contiguous(), case.v.to(DEV)[rows_dev].contiguous()
    poison = torch.full_like(k_new, float("nan"))
    ops.kv_append(poison, poison, token_item, positions, case.table, case.k_pool, case.v_pool, case.page_stride,
                  kv_heads, head_dim, page)
    torch.cuda.synchronize()
    out = torch.empty(len(rows), heads * head_dim, dtype=torch.bfloat16, device=DEV)
    ops.kv_append(k_new, v_new, token_item, positions, case.table, case.k_pool, case.v_pool, case.page_stride,
                  kv_heads, head_dim, page)
    ops.paged_attention_decode(q, out, case.k_pool, case.v_pool, case.page_stride, token_item, positions,
                               case.table, heads, kv_heads, head_dim, page, window, head_dim ** -0.5, max(lengths),
                               target_ctas=target_ctas, merge=merge,
                               q_start=torch.tensor(q_start, dtype=torch.int32, device=DEV),
                               kv_len=torch.tensor(lengths, dtype=torch.int32, device=DEV))
    assert torch.isfinite(out.float()).all()
    assert rel_err(out, case.reference(window)[rows]) < 8e-3


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(12, 12, 64, 16), (4, 4, 16, 16), (6, 2, 48, 8),
                                                          (12, 4, 64, 64)])
@pytest.mark.parametrize("window", [None, 70, 700])
def test_attention_decode_few_pairs_one_cta_of_teams_each(heads, kv_heads, head_dim, page, window):
    """At most one (token, head) pair per SM and head sizes up to 64: the kernel runs one CTA of six teams per
    pair, each team on a chunk of its own, merged in shared memory. Contexts of one chunk, of exactly six, of
    seven (a second round for one team) and of twelve; windows that leave the first teams without keys; the
    newest keys written right before the launch, the older ones fetched before the wait."""
    ops = ops_for(torch.bfloat16)
    lengths = [1, 127, 128, 129, 640, 768, 769, 1024, 1500]
    fresh = [1, 1, 2, 1, 1, 1, 3, 1, 1]
    assert sum(fresh) * heads <= 148
    case = PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=23 + head_dim)
    rows, item_of, q_start = [], [], [0]
    start = 0
    for item, (length, new) in enumerate(zip(lengths, fresh)):
        rows += list(range(start + length - new, start + length))
        item_of += [item] * new
        q_start.append(q_start[-1] + new)
        start += length
    rows_dev = torch.tensor(rows, device=DEV)
    q = case.q.to(DEV)[rows_dev].contiguous()
    token_item = torch.tensor(item_of, dtype=torch.int32, device=DEV)
    positions = case.positions[rows_dev].contiguous()
    k_new, v_new = case.k.to(DEV)[rows_dev].contiguous(), case.v.to(DEV)[rows_dev].contiguous()
    poison = torch.full_like(k_new, float("nan"))
    reference = case.reference(window)[rows]
    results = []
    for target_ctas in (10 ** 7, 1):                       # a chunk per split (teams), one split (one team's walk)
        ops.kv_append(poison, poison, token_item, positions, case.table, case.k_pool, case.v_pool, case.page_stride,
                      kv_heads, head_dim, page)
        torch.cuda.synchronize()
        out = torch.full((len(rows), heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.kv_append(k_new, v_new, token_item, positions, case.table, case.k_pool, case.v_pool, case.page_stride,
                      kv_heads, head_dim, page)
        ops.paged_attention_decode(q, out, case.k_pool, case.v_pool, case.page_stride, token_item, positions,
                                   case.table, heads, kv_heads, head_dim, page, window, head_dim ** -0.5,
                                   max(lengths), target_ctas=target_ctas,
                                   q_start=torch.tensor(q_start, dtype=torch.int32, device=DEV),
                                   kv_len=torch.tensor(lengths, dtype=torch.int32, device=DEV))
        assert torch.isfinite(out.float()).all()
        assert rel_err(out, reference) < 8e-3
        results.append(out.float())
    # the two ways of cutting the keys agree far more closely with each other than with float64
    assert rel_err(results[0], results[1].double()) < 4e-3


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 4, 16, 16), (2, 2, 48, 8), (12, 12, 64, 16),
                                                          (8, 2, 128, 32), (3, 1, 96, 64), (2, 2, 80, 4)])
@pytest.mark.parametrize("window", [None, 70])
def test_prefill_attention_bfloat16(heads, kv_heads, head_dim, page, window):
    """Whole prompts and portions that continue a cached prompt, lengths around the 64-row and 64-key
    block edges, fragmented tables; items before ``first_item`` are left alone."""
    ops = ops_for(torch.bfloat16)
    lengths = [40, 16, 63, 64, 65, 127, 128, 129, 200, 1000]
    case = PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=3 + head_dim)
    reference = case.reference(window)
    # how many of each sequence's last tokens form the portion of this step (the rest is "cached")
    portions = [40, 16, 63, 17, 65, 64, 128, 100, 37, 1000]
    rows, q_start, kv_len, flat_ref = [], [0], [], []
    begin = 0
    for length, portion in zip(lengths, portions):
        index = torch.arange(begin + length - portion, begin + length)
        rows.append(index)
        q_start.append(q_start[-1] + portion)
        kv_len.append(length)
        begin += length
    rows = torch.cat(rows)
    q = case.q[rows].to(DEV)
    out = torch.full((rows.numel(), heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    first_item = 1                                             # item 0 belongs to "another kernel"
    blocks = sum(-(-p // 64) for p in portions[first_item:])
    ops.prefill_attention(q, out, case.k_pool, case.v_pool, case.page_stride,
                          torch.tensor(q_start, dtype=torch.int32, device=DEV),
                          torch.tensor(kv_len, dtype=torch.int32, device=DEV), case.table, first_item,
                          len(lengths) - first_item, blocks + 3, heads, kv_heads, head_dim, page, window,
                          head_dim ** -0.5)
    assert torch.isnan(out[:portions[0]].float()).all()        # untouched
    got = out[portions[0]:]
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, reference[rows[portions[0]:]]) < 8e-3


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(12, 12, 64, 16), (8, 2, 128, 32), (3, 1, 64, 8),
                                                          (2, 2, 128, 64)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("row_threads", [1, 2])
def test_prefill_attention_tcgen05(heads, kv_heads, head_dim, page, window, row_threads):
    """The tcgen05 kernel (S, P and O_j in TMEM) on whole prompts and on portions that continue a cached
    prompt, lengths around the 128-row and 128-key block edges, fragmented tables, a poisoned pool (NaN in
    every slot that was never written), items before ``first_item`` left alone; one thread per query row and
    two (which exchange the row's maximum and sum through shared memory)."""
    ops = ops_for(torch.bfloat16)
    lengths = [40, 16, 127, 128, 129, 255, 256, 257, 300, 1000]
    case = PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=5 + head_dim)
    reference = case.reference(window)
    portions = [40, 16, 127, 17, 129, 128, 256, 100, 37, 1000]
    rows, q_start, kv_len = [], [0], []
    begin = 0
    for length, portion in zip(lengths, portions):
        rows.append(torch.arange(begin + length - portion, begin + length))
        q_start.append(q_start[-1] + portion)
        kv_len.append(length)
        begin += length
    rows = torch.cat(rows)
    q = case.q[rows].to(DEV)
    out = torch.full((rows.numel(), heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    first_item = 1
    blocks = sum(-(-p // 128) for p in portions[first_item:])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.prefill_attention_tc(q, out, case.pool, 0, torch.tensor(q_start, dtype=torch.int32, device=DEV),
                             torch.tensor(kv_len, dtype=torch.int32, device=DEV), case.table, first_item,
                             len(lengths) - first_item, blocks + 2, heads, kv_heads, head_dim, page, window,
                             head_dim ** -0.5, status=status, row_threads=row_threads)
    assert int(status.item()) == 0
    assert torch.isnan(out[:portions[0]].float()).all()        # untouched
    got = out[portions[0]:]
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, reference[rows[portions[0]:]]) < 8e-3


@pytest.mark.parametrize("far", [0, 31, 32, 255, 256, 600])
def test_attention_finds_a_far_key(far):
    """One key among a thousand carries almost all the weight: the output must be its value."""
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        ops = ops_for(dtype)
        case = PagedCase(ops, dtype, [1000, 40], 4, 2, 64, 16, seed=far, spike=(far, 3))
        out = torch.empty(1040, 4 * 64, dtype=dtype, device=DEV)
        if dtype == torch.float32:
            ops.paged_attention_simt(case.q.to(DEV), out, case.k_pool, case.v_pool, case.page_stride,
                                     case.token_item, case.positions, case.table, 4, 2, 64, 16, None, 0.125)
        else:
            ops.paged_attention_decode(case.q.to(DEV), out, case.k_pool, case.v_pool, case.page_stride,
                                       case.token_item, case.positions, case.table, 4, 2, 64, 16, None, 0.125,
                                       1000, target_ctas=10 ** 7)
        want = case.reference()
        if dtype == torch.bfloat16:
            tensor_core = torch.empty_like(out)
            ops.prefill_attention(case.q.to(DEV), tensor_core, case.k_pool, case.v_pool, case.page_stride,
                                  torch.tensor([0, 1000, 1040], dtype=torch.int32, device=DEV),
                                  torch.tensor([1000, 40], dtype=torch.int32, device=DEV), case.table, 0, 2, 17,
                                  4, 2, 64, 16, None, 0.125)
            assert float((tensor_core[999, 192:256].double().cpu() - case.v[far, 64:128].double()).abs().max()) < 0.05
            assert rel_err(tensor_core, want) < tol
            fifth_gen = torch.empty_like(out)
            ops.prefill_attention_tc(case.q.to(DEV), fifth_gen, case.pool, 0,
                                     torch.tensor([0, 1000, 1040], dtype=torch.int32, device=DEV),
                                     torch.tensor([1000, 40], dtype=torch.int32, device=DEV), case.table, 0, 2, 9,
                                     4, 2, 64, 16, None, 0.125)
            assert float((fifth_gen[999, 192:256].double().cpu() - case.v[far, 64:128].double()).abs().max()) < 0.05
            assert rel_err(fifth_gen, want) < tol
        got_row = out[999, 3 * 64:4 * 64].double().cpu()
        value_row = case.v[far, 64:128].double()
        assert float((got_row - value_row).abs().max()) < 0.05          # the spike's value came through
        assert rel_err(out, want) < tol
