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


def _call_noalloc(lib, case, out, split_tiles, n_splits, scale, head_dim=None, q=None):
    message = ctypes.create_string_buffer(256)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q = case.q.to(DEV) if q is None else q
    rc = lib.ps_paged_attention_decode_noalloc(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_int(q.stride(0)), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(out.stride(0)), ctypes.c_void_p(case.k_pool.data_ptr()),
        ctypes.c_void_p(case.v_pool.data_ptr()), ctypes.c_longlong(case.page_stride),
        ctypes.c_void_p(case.token_item.data_ptr()), ctypes.c_void_p(case.positions.data_ptr()),
        ctypes.c_void_p(case.table.data_ptr()), ctypes.c_int(case.table.stride(0)), ctypes.c_int(q.shape[0]),
        ctypes.c_int(case.n_heads), ctypes.c_int(case.n_kv_heads), ctypes.c_int(head_dim or case.head_dim),
        ctypes.c_int(case.page_size), ctypes.c_int(0), ctypes.c_float(scale), ctypes.c_int(split_tiles),
        ctypes.c_int(n_splits), stream, message, ctypes.c_int(256))
    torch.cuda.synchronize()
    return rc, message.value.decode()


def _status(lib, clear=True):
    """The status word that the kernel leaves in the fixed array, read through its own C entry point."""
    value = ctypes.c_int(-1)
    rc = lib.ps_paged_attention_decode_noalloc_status(ctypes.byref(value), ctypes.c_int(1 if clear else 0),
                                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return value.value


def _ordinary(lib, case, split_tiles, n_splits, scale):
    """The ordinary entry point with the same split rule; the caller hands in the scratch."""
    total, heads, head_dim = case.q.shape[0], case.n_heads, case.head_dim
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
        ctypes.c_int(heads), ctypes.c_int(case.n_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(case.page_size),
        ctypes.c_int(0), ctypes.c_float(scale), ctypes.c_int(split_tiles), ctypes.c_int(n_splits),
        ctypes.c_void_p(part_acc.data_ptr()), ctypes.c_void_p(part_ml.data_ptr()),
        ctypes.c_void_p(counters.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    return want


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
        want = _ordinary(lib, case, split_tiles, n_splits, scale)
        got = torch.full_like(want, float("nan"))
        if call == 0:
            # the first call on a device looks the array's address up (and may load the module): not counted
            warm = torch.empty_like(want)
            assert _call_noalloc(lib, case, warm, split_tiles, n_splits, scale)[0] == 0
        # free device memory as the driver sees it: a cudaMalloc inside the entry point would show here,
        # whoever's allocator made it (torch's own counters would not see it)
        q = case.q.to(DEV)                      # the test's own allocations come before the measurement
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        before = torch.cuda.memory_allocated()
        rc, message = _call_noalloc(lib, case, got, split_tiles, n_splits, scale, q=q)
        assert rc == 0, message
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        assert _status(lib) == 0
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
    # a head size beyond the fixed array's rows is refused before anything runs
    rc, message = _call_noalloc(lib, small, out, 4, 1, 0.125, head_dim=272)
    assert rc == 4 and "head_dim 272 exceeds" in message


def test_no_alloc_entry_point_uses_its_last_slots_at_the_limits():
    """Exactly 4,096 partial states (the last slot of the fixed array is written and merged), then exactly
    4,096 (token, head) rows: both are accepted and right."""
    from pagedserve_b200.kernels.build import load
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    lib = load("bf16")
    for heads, split_tiles, n_splits in ((2, 4, 4), (8, 16, 1)):        # 512 x 2 x 4 partials; 512 x 8 rows
        case = _case(ops, [512], heads, heads, 64, 16, seed=7 + heads)
        assert 512 * heads * n_splits == 4096
        want = _ordinary(lib, case, split_tiles, n_splits, 0.125)
        got = torch.full_like(want, float("nan"))
        rc, message = _call_noalloc(lib, case, got, split_tiles, n_splits, 0.125)
        assert rc == 0, message
        assert _status(lib) == 0
        reference = case.reference()
        scale_ref = float(reference.abs().max())
        assert float((got.double().cpu() - reference).abs().max()) < 8e-3 * scale_ref
        assert float((got.float() - want.float()).abs().max()) <= 8e-3 * scale_ref


def test_no_alloc_entry_point_reports_a_grid_that_does_not_reach_the_newest_keys():
    """n_splits is the caller's to choose. One split of 128 keys for a context of 200 reaches positions 0-127
    only: the tokens beyond get no output, and the status word (3) says so until it is cleared."""
    from pagedserve_b200.kernels.build import load
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    lib = load("bf16")
    assert _status(lib) == 0
    case = _case(ops, [200], 2, 2, 64, 16, seed=11)
    out = torch.zeros(200, 2 * 64, dtype=torch.bfloat16, device=DEV)
    rc, message = _call_noalloc(lib, case, out, 4, 1, 0.125)
    assert rc == 0, message                                              # the host cannot know the positions
    assert _status(lib, clear=False) == 3
    assert float(out[128:].abs().max()) == 0.0                           # tokens the grid did not reach: untouched
    reference = case.reference()
    assert float((out[:128].double().cpu() - reference[:128]).abs().max()) < 8e-3 * float(reference.abs().max())
    assert _status(lib) == 3 and _status(lib) == 0                       # read and cleared
    # the same context with enough splits is fine, and the counters it shares were left clean
    rc, message = _call_noalloc(lib, case, out, 4, 2, 0.125)
    assert rc == 0 and _status(lib) == 0
    assert float((out.double().cpu() - reference).abs().max()) < 8e-3 * float(reference.abs().max())
