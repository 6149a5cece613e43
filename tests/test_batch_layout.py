"""The flat layout of a step (host arithmetic only): order, positions, wanted rows, padding."""

import numpy as np
import pytest

from pagedserve_b200.engine.batch import BatchLayout, StepContext, StepEntry, arrange_step, layout_order

LONG = StepContext.LONG_ENTRY
SCRATCH = 99


def random_step(rng, items, longest):
    """Entries with random counts (many single tokens, some portions), distinct slots, random cached lengths."""
    entries, slots, starts = [], [], []
    for index in range(items):
        kind = rng.integers(0, 3)
        count = 1 if kind == 0 else int(rng.integers(2, LONG)) if kind == 1 else int(rng.integers(LONG, longest + 1))
        tokens = rng.integers(0, 1000, size=count)
        want = sorted(set(int(place) for place in rng.integers(0, count, size=rng.integers(0, 3))))
        entries.append(StepEntry(f"r{index}", tokens, want))
        slots.append(index)
        starts.append(int(rng.integers(0, 500)))
    return entries, np.asarray(slots), np.asarray(starts)


def arrange(entries, slots, starts, **options):
    counts = np.asarray([len(entry.tokens) for entry in entries])
    order, num_short = layout_order(counts, LONG)
    tokens = np.concatenate([entries[source].tokens for source in order])
    batch = arrange_step(order, num_short, counts, tokens, slots[order], starts[order],
                         [entry.want for entry in entries], scratch_slot=SCRATCH, **options)
    return order, batch


def check_real_entries(entries, slots, starts, order, batch, item_of_source):
    for source, entry in enumerate(entries):
        item = item_of_source[source]
        first, last = int(batch.q_start[item]), int(batch.q_start[item + 1])
        count = len(entry.tokens)
        assert last - first == count
        assert np.array_equal(batch.token_ids[first:last], entry.tokens)
        assert np.array_equal(batch.positions[first:last], starts[source] + np.arange(count))
        assert np.all(batch.token_item[first:last] == item)
        assert batch.item_slot[item] == slots[source]
        assert batch.kv_len[item] == starts[source] + count
        assert (item < batch.num_short_items) == (count < LONG)
    # rows of logits in the caller's order
    expected = [int(batch.q_start[item_of_source[source]]) + place
                for source, entry in enumerate(entries) for place in entry.want]
    assert batch.logit_rows[:batch.real_rows].tolist() == expected
    assert batch.real_rows == len(expected)


def test_layout_order_keeps_the_callers_order_within_a_kind():
    order, num_short = layout_order(np.asarray([40, 1, 16, 15, 1, 100]), 16)
    assert order.tolist() == [1, 3, 4, 0, 2, 5]
    assert num_short == 3


@pytest.mark.parametrize("seed", range(20))
def test_unpadded_arrangement(seed):
    rng = np.random.default_rng(seed)
    entries, slots, starts = random_step(rng, int(rng.integers(1, 12)), 200)
    order, batch = arrange(entries, slots, starts)
    assert batch.num_items == len(entries)
    assert batch.num_tokens == sum(len(entry.tokens) for entry in entries)
    assert batch.num_rows == batch.real_rows
    item_of_source = np.empty(len(entries), dtype=np.int64)
    item_of_source[order] = np.arange(len(entries))
    check_real_entries(entries, slots, starts, order, batch, item_of_source)
    long_counts = np.diff(batch.q_start)[batch.num_short_items:]
    assert batch.num_long_blocks == int(sum(-(-count // 64) for count in long_counts))
    assert batch.num_short_tokens == int(batch.q_start[batch.num_short_items])


@pytest.mark.parametrize("seed", range(30))
def test_padded_arrangement(seed):
    rng = np.random.default_rng(100 + seed)
    entries, slots, starts = random_step(rng, int(rng.integers(1, 12)), 300)
    pad_short, pad_long = 16, 128
    order, batch = arrange(entries, slots, starts, pad=True, pad_short=pad_short, pad_long=pad_long)
    counts = np.diff(batch.q_start)
    short_tokens = batch.num_short_tokens
    long_tokens = batch.num_tokens - short_tokens
    assert short_tokens % pad_short == 0 and long_tokens % pad_long == 0
    assert batch.num_short_items % 8 == 0 and (batch.num_items - batch.num_short_items) % 4 == 0
    assert batch.num_rows % 8 == 0 and batch.num_rows - batch.real_rows < 8

    num_short_real = sum(len(entry.tokens) < LONG for entry in entries)
    num_long_real = len(entries) - num_short_real
    item_of_source = np.empty(len(entries), dtype=np.int64)
    item_of_source[order] = np.concatenate([np.arange(num_short_real),
                                            batch.num_short_items + np.arange(num_long_real)])
    check_real_entries(entries, slots, starts, order, batch, item_of_source)

    # everything else is padding: the scratch slot from position 0, at most one entry with tokens per kind
    real = set(item_of_source.tolist())
    padding = [item for item in range(batch.num_items) if item not in real]
    for kind in (range(0, batch.num_short_items), range(batch.num_short_items, batch.num_items)):
        with_tokens = [item for item in kind if item in padding and counts[item] > 0]
        assert len(with_tokens) <= 1
    for item in padding:
        assert batch.item_slot[item] == SCRATCH
        first, last = int(batch.q_start[item]), int(batch.q_start[item + 1])
        assert np.array_equal(batch.positions[first:last], np.arange(last - first))
        assert np.all(batch.token_ids[first:last] == 0)
        assert batch.kv_len[item] == last - first < max(pad_short, pad_long)
        if item < batch.num_short_items:
            assert last - first < LONG
    # padded rows repeat a real row; the bound on 64-query blocks covers every long item
    if batch.real_rows:
        assert np.all(batch.logit_rows[batch.real_rows:] == batch.logit_rows[0])
    assert batch.num_long_blocks >= int(sum(-(-count // 64) for count in counts[batch.num_short_items:]))


def test_padded_shape_depends_on_rounded_sizes_only():
    """Two steps whose sizes round to the same numbers get the same shape and the same block bound."""
    def shape(counts):
        entries = [StepEntry(index, np.zeros(count, dtype=np.int64), [count - 1]) for index, count in enumerate(counts)]
        slots = np.arange(len(counts))
        _, batch = arrange(entries, slots, np.zeros(len(counts), dtype=np.int64), pad=True)
        return (batch.num_tokens, batch.num_items, batch.num_rows, batch.num_short_items, batch.num_short_tokens,
                batch.num_long_blocks)

    assert shape([1, 1, 1, 100]) == shape([1, 1, 1, 1, 1, 120]) == shape([1, 2, 3, 64, 40])
    assert shape([1] * 16) == (16, 16, 16, 16, 16, 0)            # already a recurring shape: nothing is added
    assert shape([128]) == (128, 4, 8, 0, 0, 128 // 64 + 4)


def test_packed_sections_do_not_overlap_and_are_aligned():
    layout = BatchLayout(37, 5, 3, update_capacity=9)
    names = ["header", "item_slot", "q_start", "logit_rows", "updates", "token_ids", "positions", "token_item",
             "token_slot", "kv_len", "temperature", "seed"]
    sizes = [4, 5, 6, 3, 18, 37, 37, 37, 37, 5, 5, 10]
    spans = sorted((getattr(layout, name), getattr(layout, name) + size) for name, size in zip(names, sizes))
    for (start, end), (next_start, _) in zip(spans, spans[1:]):
        assert end <= next_start
    assert all(start % 4 == 0 for start, _ in spans)             # 16-byte sections: vector loads are legal
    assert spans[-1][1] <= layout.total
    # what the host uploads comes first and ends with the token ids, so that a step whose tokens the device
    # fed back uploads a prefix that stops after the corrections
    uploaded = ["header", "item_slot", "q_start", "logit_rows", "updates", "token_ids"]
    assert max(getattr(layout, name) for name in uploaded) == layout.token_ids < layout.uploaded
    assert min(getattr(layout, name) for name in names if name not in uploaded) >= layout.uploaded
    assert layout.updates < layout.token_ids and layout.counter == layout.header
    assert layout.words.tolist() == [37, 5, layout.header, layout.item_slot, layout.q_start, layout.updates, 9,
                                     layout.token_ids, layout.positions, layout.token_item, layout.token_slot,
                                     layout.kv_len, layout.temperature, layout.seed]


def test_step_entry_checks_and_normalises():
    entry = StepEntry("r", [5, 17, 3], (0, np.int32(2)))
    assert entry.tokens.dtype == np.int64 and entry.tokens.tolist() == [5, 17, 3]
    assert entry.want == [0, 2] and all(type(place) is int for place in entry.want)
    assert StepEntry("r", np.asarray([[1, 2], [3, 4]], dtype=np.uint16)).tokens.tolist() == [1, 2, 3, 4]
    assert StepEntry("r", np.int32(7)).tokens.tolist() == [7] and StepEntry("r", [7]).want == []
    kept = np.arange(4, dtype=np.int64)
    assert StepEntry("r", kept).tokens is kept                         # already in the kept form: no copy
    with pytest.raises(ValueError, match="at least one token"):
        StepEntry("r", [])
    for bad in ([1.0, 2.0], [True, False], ["a"]):
        with pytest.raises(ValueError, match="must be integers"):
            StepEntry("r", bad)
    for want in ([3], [-1], [0, 5]):
        with pytest.raises(ValueError, match="outside the entry"):
            StepEntry("r", [1, 2, 3], want)


# ------------------------------------------------------------------ the native builder against its specification
def _native():
    """The host-only entry points of the kernel library (compiled with nvcc, loaded without a GPU)."""
    import torch
    from pagedserve_b200.kernels.ops import Ops

    return Ops(torch.float32)


@pytest.mark.parametrize("pad", [False, True])
@pytest.mark.parametrize("seed", range(25))
def test_native_step_builder_equals_arrange_step(seed, pad):
    """``ps_step_shape`` / ``ps_step_fill`` (csrc/step_build.cu) lay a step out exactly as ``arrange_step`` does:
    the same shape, and the same slots, item starts, wanted rows and token ids in the staging buffer."""
    ops = _native()
    rng = np.random.default_rng(1000 + seed)
    entries, slots, starts = random_step(rng, int(rng.integers(1, 14)), 300)
    if seed % 5 == 0:                                                    # only decodes / only long portions
        keep = [i for i, entry in enumerate(entries) if (len(entry.tokens) < LONG) == (seed % 2 == 0)] or [0]
        entries, slots, starts = [entries[i] for i in keep], slots[keep], starts[keep]
    order, batch = arrange(entries, slots, starts, pad=pad, pad_short=16, pad_long=128)
    counts = np.asarray([len(entry.tokens) for entry in entries], dtype=np.int64)
    want_counts = np.asarray([len(entry.want) for entry in entries], dtype=np.int32)
    wants = np.asarray([place for entry in entries for place in entry.want], dtype=np.int32)
    tokens = np.concatenate([entry.tokens for entry in entries])
    slots64, starts64 = slots.astype(np.int64), starts.astype(np.int64)
    shape = ops.step_shape(counts, starts64, want_counts, LONG, pad, 16, 128)
    laid = np.diff(batch.q_start)
    assert shape == [batch.num_tokens, batch.num_items, batch.num_rows, batch.num_short_items, batch.num_short_tokens,
                     batch.num_long_blocks, batch.real_rows, int(laid.max()), int(batch.kv_len.max())]
    layout = BatchLayout(shape[0], shape[1], shape[2], update_capacity=5)
    staging = np.full(layout.total, -7, dtype=np.int32)
    assert ops.step_fill(counts, starts64, want_counts, tokens, slots64, wants, LONG, pad, 16, 128, SCRATCH, 1000,
                         staging.ctypes.data, layout) is None
    T, I, R = shape[:3]
    assert staging[layout.item_slot:layout.item_slot + I].tolist() == batch.item_slot.tolist()
    assert staging[layout.q_start:layout.q_start + I + 1].tolist() == batch.q_start.tolist()
    assert staging[layout.logit_rows:layout.logit_rows + R].tolist() == batch.logit_rows.tolist()
    assert staging[layout.token_ids:layout.token_ids + T].tolist() == batch.token_ids.tolist()
    untouched = np.ones(layout.total, dtype=bool)
    for offset, count in ((layout.item_slot, I), (layout.q_start, I + 1), (layout.logit_rows, R), (layout.token_ids, T)):
        untouched[offset:offset + count] = False
    assert (staging[untouched] == -7).all()                             # nothing else was written
    # a token outside the vocabulary is reported, not written
    tokens[len(tokens) // 2] = 1000
    assert ops.step_fill(counts, starts64, want_counts, tokens, slots64, wants, LONG, pad, 16, 128, SCRATCH, 1000,
                         staging.ctypes.data, layout) == 1000


def test_step_arena_hands_out_aligned_views_and_reuses_them():
    """The arena that a step's activations come from: views of a few chunks, 256-byte aligned, the same places
    again after ``reset`` and after ``release(mark)``, a new chunk when one is full, nothing shared between two
    tensors that are alive at the same time."""
    import torch

    from pagedserve_b200.kernels.ops import StepArena

    arena = StepArena()
    arena.CHUNK_BYTES = 4096                      # small chunks so that the test crosses their edges
    cpu = torch.device("cpu")
    a = arena.empty((3, 5), torch.float32, cpu)
    b = arena.empty((7,), torch.bfloat16, cpu)
    assert a.shape == (3, 5) and a.dtype == torch.float32 and b.shape == (7,) and b.dtype == torch.bfloat16
    assert a.data_ptr() % 256 == 0 and b.data_ptr() % 256 == 0
    assert b.data_ptr() >= a.data_ptr() + a.numel() * 4
    a.fill_(1.0)
    b.fill_(2.0)
    assert float(a.sum()) == 15.0                 # filling b did not touch a
    mark = arena.mark()
    c = arena.empty((900,), torch.float32, cpu)   # 3,600 bytes: does not fit behind a and b, goes to a new chunk
    d = arena.empty((10,), torch.int32, cpu)
    assert len(arena.chunks) == 2 and float(a.sum()) == 15.0
    arena.release(mark)
    c2 = arena.empty((900,), torch.float32, cpu)
    d2 = arena.empty((10,), torch.int32, cpu)
    assert c2.data_ptr() == c.data_ptr() and d2.data_ptr() == d.data_ptr() and len(arena.chunks) == 2
    big = arena.empty((5000,), torch.float32, cpu)          # larger than a chunk: a chunk of its own
    assert big.numel() == 5000 and len(arena.chunks) == 3
    arena.reset()
    again = arena.empty((3, 5), torch.float32, cpu)
    assert again.data_ptr() == a.data_ptr() and len(arena.chunks) == 3
    assert arena.empty((0, 8), torch.float32, cpu).numel() == 0
