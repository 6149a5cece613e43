"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it (their process
handed the whole GPU to its own pool at start-up, or they call from outside Python and have no
allocator of ours).  ``ps_paged_attention_decode_noalloc`` serves them: the scratch of the
split-key attention kernel lives in a fixed array inside the library.  This test calls it twice in
a row, with different shapes so that the second call meets the first call's leftovers, and checks
each result against the ordinary entry point, which gets its scratch from the caller.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(ops, lengths, heads, kv_heads, head_dim, page, seed):
    from test_kernels_gpu import PagedCase

    return PagedCase(ops, torch.bfloat16, lengths, heads, kv_heads, head_dim, page, seed=seed)


def _call_noalloc(lib, case, out, split_tiles, n_splits, scale):
    message = ctypes.create_string_buffer(256)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q = case.q.to(DEV)
    rc = lib.ps_paged_attention_decode_noalloc(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_int(q.stride(0)), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(out.stride(0)), ctypes.c_void_p(case.k_pool.data_ptr()),
        ctypes.c_void_p(case.v_pool.data_ptr()), ctypes.c_longlong(case.page_stride),
        ctypes.c_void_p(case.token_item.data_ptr()), ctypes.c_void_p(case.positions.data_ptr()),
        ctypes.c_void_p(case.table.data_ptr()), ctypes.c_int(case.table.stride(0)), ctypes.c_int(q.shape[0]),
        ctypes.c_int(case.n_heads), ctypes.c_int(case.n_kv_heads), ctypes.c_int(case.head_dim),
        ctypes.c_int(case.page_size), ctypes.c_int(0), ctypes.c_float(scale), ctypes.c_int(split_tiles),
        ctypes.c_int(n_splits), stream, message, ctypes.c_int(256))
    torch.cuda.synchronize()
    return rc, message.value.decode()


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from pagedserve_b200.kernels.build import load
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    lib = load("bf16")
    assert hasattr(lib, "ps_paged_attention_decode_noalloc")
    shapes = [([200, 17, 70], 4, 2, 64, 16, 4, 2),           # (lengths, heads, kv, hd, page, split_tiles, n_splits)
              ([1, 33, 250], 3, 3, 48, 8, 4, 2)]                 # a split is a whole number of 128-key chunks
    for call, (lengths, heads, kv_heads, head_dim, page, split_tiles, n_splits) in enumerate(shapes):
        case = _case(ops, lengths, heads, kv_heads, head_dim, page, seed=90 + call)
        total = sum(lengths)
        scale = head_dim ** -0.5
        # the ordinary entry point with the same split rule, scratch handed in by the caller
        want = torch.empty(total, heads * head_dim, dtype=torch.bfloat16, device=DEV)
        counters = torch.zeros(total * heads, dtype=torch.int32, device=DEV)
        part_acc = torch.empty(total * heads * n_splits, head_dim, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(total * heads * n_splits, 2, dtype=torch.float32, device=DEV)
        q = case.q.to(DEV)
        rc = lib.ps_paged_attention_decode(
            ctypes.c_void_p(q.data_ptr()), ctypes.c_int(q.stride(0)), ctypes.c_void_p(want.data_ptr()),
            ctypes.c_int(want.stride(0)), ctypes.c_void_p(case.k_pool.data_ptr()),
            ctypes.c_void_p(case.v_pool.data_ptr()), ctypes.c_longlong(case.page_stride),
            ctypes.c_void_p(case.token_item.data_ptr()), ctypes.c_void_p(case.positions.data_ptr()),
            ctypes.c_void_p(case.table.data_ptr()), ctypes.c_int(case.table.stride(0)), ctypes.c_int(total),
            ctypes.c_int(heads), ctypes.c_int(kv_heads), ctypes.c_int(head_dim), ctypes.c_int(page),
            ctypes.c_int(0), ctypes.c_float(scale), ctypes.c_int(split_tiles), ctypes.c_int(n_splits),
            ctypes.c_void_p(part_acc.data_ptr()), ctypes.c_void_p(part_ml.data_ptr()),
            ctypes.c_void_p(counters.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc, message = _call_noalloc(lib, case, got, split_tiles, n_splits, scale)
        assert rc == 0, message
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        reference = case.reference()
        scale_ref = float(reference.abs().max())
        assert float((got.double().cpu() - reference).abs().max()) < 8e-3 * scale_ref       # as the kernel tests
        assert float((got.float() - want.float()).abs().max()) <= 8e-3 * scale_ref


def test_no_alloc_entry_point_refuses_sizes_beyond_its_scratch():
    from pagedserve_b200.kernels.build import load
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    lib = load("bf16")
    case = _case(ops, [700], 8, 8, 64, 16, seed=3)              # 700 tokens x 8 heads = 5600 rows > 4096
    out = torch.zeros(700, 8 * 64, dtype=torch.bfloat16, device=DEV)
    rc, message = _call_noalloc(lib, case, out, 4, 1, 0.125)
    assert rc == 4 and "exceeds the fixed scratch's limit" in message
    assert float(out.abs().max()) == 0.0                         # nothing ran
    small = _case(ops, [100], 8, 8, 64, 16, seed=4)              # 800 rows x 8 splits = 6400 partial states
    out = torch.zeros(100, 8 * 64, dtype=torch.bfloat16, device=DEV)
    rc, message = _call_noalloc(lib, small, out, 4, 8, 0.125)
    assert rc == 4 and "partial states" in message
