"""What one step runs: a flat batch of (request, its next tokens).

The reference describes a step with ``IterationItem`` / ``IterationBatch``
(reference: src/model/iteration.py:10-74): per item a request id, phase, token
ids, position ids, flattened offsets and ``produces_output``.  Here an entry
carries only the request, its next tokens and the places whose logits are
wanted; positions follow from the request's cached length, and a "decode" is
simply an entry of one token.  The device side is one packed int32 buffer
(one host-to-device copy per step) of which the host fills only the part the
device cannot derive from the per-request state it keeps by slot.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are returned

    def __post_init__(self):
        tokens = np.asarray(self.tokens)
        if tokens.size and tokens.dtype.kind not in "iu":                  # signed or unsigned integers only
            raise ValueError("token ids must be integers")
        if tokens.dtype != np.int64 or tokens.ndim != 1:
            tokens = tokens.astype(np.int64, copy=False).reshape(-1)
        self.tokens = tokens                                               # kept as an array: prompts are long
        count = tokens.size
        if count == 0:
            # reference: src/model/iteration.py:23-24
            raise ValueError("a step entry must contain at least one token")
        want = self.want
        if type(want) is not list or any(type(place) is not int for place in want):
            want = self.want = [int(w) for w in want]
        for place in want:
            if not (0 <= place < count):
                raise ValueError(f"wanted place {place} is outside the entry's {count} tokens")


def layout_order(counts: np.ndarray, long_entry: int):
    """The order in which a step's entries are laid out: short entries (decode tokens, short portions)
    first, prompt portions of ``long_entry`` or more tokens after them, each kind in the caller's order.
    Returns (source index of each laid-out item, number of short items)."""
    is_long = np.asarray(counts) >= long_entry
    order = np.concatenate([np.flatnonzero(~is_long), np.flatnonzero(is_long)])
    return order, len(order) - int(is_long.sum())


def _round_up(value: int, step: int) -> int:
    return -(-value // step) * step


@dataclass
class Arrangement:
    """The flat batch of one step as host arrays (int64), before it is packed for the device."""

    token_ids: np.ndarray         # [T]
    positions: np.ndarray         # [T]
    token_item: np.ndarray        # [T]
    item_slot: np.ndarray         # [I]
    q_start: np.ndarray           # [I + 1]
    kv_len: np.ndarray            # [I]
    logit_rows: np.ndarray        # [R]
    num_short_items: int
    num_short_tokens: int
    num_long_blocks: int
    real_rows: int                # rows of logits that the caller asked for (the rest is padding)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_items(self) -> int:
        return len(self.item_slot)

    @property
    def num_rows(self) -> int:
        return len(self.logit_rows)


def arrange_step(order: np.ndarray, num_short_items: int, counts: np.ndarray, tokens: np.ndarray,
                 slots: np.ndarray, starts: np.ndarray, wants: Sequence[Sequence[int]], *,
                 pad: bool = False, pad_short: int = 16, pad_long: int = 128, scratch_slot: int = -1) -> Arrangement:
    """Lay a step out as one flat batch.

    ``order``/``num_short_items`` come from :func:`layout_order`; ``counts`` and ``wants`` are in the caller's
    order; ``tokens`` (all tokens), ``slots`` and ``starts`` (cached length of each request before the step) are
    in layout order.  With ``pad`` the batch is brought to a recurring shape: the short tokens to a multiple of
    ``pad_short`` and the long ones to a multiple of ``pad_long`` by one padding entry behind each kind (at
    positions 0.. of ``scratch_slot``), the items to multiples of 8 and 4 by empty entries of that slot, and
    the logits rows to a multiple of 8 by repeating the first row.
    """
    counts = np.asarray(counts, dtype=np.int64)
    real_items = len(order)
    laid_counts = counts[order]
    num_long_items = real_items - num_short_items
    short_tokens = int(laid_counts[:num_short_items].sum())
    long_tokens = int(laid_counts.sum()) - short_tokens
    real_rows = sum(len(want) for want in wants)
    num_rows = real_rows
    if pad:
        extra_short = _round_up(short_tokens, pad_short) - short_tokens
        extra_long = _round_up(long_tokens, pad_long) - long_tokens
        short_items = _round_up(num_short_items + (extra_short > 0), 8) if short_tokens else 0
        long_items = _round_up(num_long_items + (extra_long > 0), 4) if long_tokens else 0

        def with_padding(real, extra, total, fill):
            """``real`` values, then the padding entry's value if it exists, then ``fill`` up to ``total``."""
            head = [real, np.full(1, extra, dtype=np.int64)] if extra is not None else [real]
            used = sum(len(piece) for piece in head)
            return np.concatenate(head + [np.full(total - used, fill, dtype=np.int64)])

        pad_count = lambda extra: extra if extra else None
        laid_counts = np.concatenate([
            with_padding(laid_counts[:num_short_items], pad_count(extra_short), short_items, 0),
            with_padding(laid_counts[num_short_items:], pad_count(extra_long), long_items, 0)])
        slots = np.concatenate([with_padding(slots[:num_short_items], None, short_items, scratch_slot),
                                with_padding(slots[num_short_items:], None, long_items, scratch_slot)])
        starts = np.concatenate([with_padding(starts[:num_short_items], None, short_items, 0),
                                 with_padding(starts[num_short_items:], None, long_items, 0)])
        tokens = np.concatenate([tokens[:short_tokens], np.zeros(extra_short, dtype=np.int64),
                                 tokens[short_tokens:], np.zeros(extra_long, dtype=np.int64)])
        # where the real entries went
        new_index = np.concatenate([np.arange(num_short_items), short_items + np.arange(num_long_items)])
        num_short_items = short_items
        num_rows = _round_up(real_rows, 8)
    else:
        new_index = np.arange(real_items)
    num_items = len(laid_counts)
    num_tokens = len(tokens)

    first = np.zeros(num_items + 1, dtype=np.int64)
    np.cumsum(laid_counts, out=first[1:])                              # first token of each laid-out item
    item_of_token = np.repeat(np.arange(num_items, dtype=np.int64), laid_counts)
    positions = np.arange(num_tokens, dtype=np.int64) + (starts - first[:-1])[item_of_token]
    if pad:                                                            # a bound that depends on the padded shape alone
        num_long_blocks = int(laid_counts[num_short_items:].sum()) // 64 + (num_items - num_short_items)
    else:
        num_long_blocks = int((-(-laid_counts[num_short_items:] // 64)).sum())
    first_of_source = np.empty(real_items, dtype=np.int64)
    first_of_source[order] = first[new_index]
    rows = [int(first_of_source[source]) + place for source, want in enumerate(wants) for place in want]
    rows += [rows[0] if rows else 0] * (num_rows - real_rows)          # logits rows keep the caller's order
    return Arrangement(np.asarray(tokens, dtype=np.int64), positions, item_of_token, np.asarray(slots, dtype=np.int64),
                       first, starts + laid_counts, np.asarray(rows, dtype=np.int64), num_short_items,
                       int(first[num_short_items]), num_long_blocks, real_rows)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of the sections of a step's packed metadata buffer.

    The first part is what the host uploads: a header (``[0]`` steps the device has run since the upload,
    which selects the row of the token history; ``[1]`` 1 if the step's token ids are the ones the device
    sampled last; ``[2]`` number of corrections), the slot of each item, the first token of each item, the
    wanted rows, the corrections of the slot store as (offset, value) pairs, and the token ids.  The rest is
    written on the device by the step's first kernel from the slots' state: positions, the item and the
    block-table row of each token, each item's length after the step and its sampling parameters."""

    num_tokens: int
    num_items: int
    num_rows: int
    update_capacity: int = 0      # most corrections a step of this shape can carry
    header: int = 0
    item_slot: int = 0
    q_start: int = 0
    logit_rows: int = 0
    updates: int = 0              # (offset, value) pairs
    token_ids: int = 0
    uploaded: int = 0             # end of the part the host uploads
    positions: int = 0
    token_item: int = 0
    token_slot: int = 0
    kv_len: int = 0
    temperature: int = 0          # float32 bits, one per item
    seed: int = 0                 # 64-bit, two words per item
    total: int = 0

    HEADER_WORDS = 4
    COUNTER, FED, NUM_UPDATES = 0, 1, 2

    def __post_init__(self):
        cursor = 0
        for name, count in (("header", self.HEADER_WORDS), ("item_slot", self.num_items),
                            ("q_start", self.num_items + 1), ("logit_rows", max(self.num_rows, 1)),
                            ("updates", 2 * self.update_capacity), ("token_ids", self.num_tokens)):
            setattr(self, name, cursor)
            cursor += _pad4(count)
        self.uploaded = cursor
        for name, count in (("positions", self.num_tokens), ("token_item", self.num_tokens),
                            ("token_slot", self.num_tokens), ("kv_len", self.num_items),
                            ("temperature", self.num_items), ("seed", 2 * self.num_items)):
            setattr(self, name, cursor)
            cursor += _pad4(count)
        self.total = cursor
        # what the kernels that open and close a step are told of the layout
        self.words = np.asarray([self.num_tokens, self.num_items, self.header, self.item_slot, self.q_start,
                                 self.updates, self.update_capacity, self.token_ids, self.positions,
                                 self.token_item, self.token_slot, self.kv_len, self.temperature, self.seed],
                                dtype=np.int32)

    @property
    def counter(self) -> int:
        return self.header + self.COUNTER


class HostBatch:
    """Host-side (numpy) view of a step, for parts that need host logic and for tests: the same numbers that
    the step's first kernel derives on the device."""

    def __init__(self, token_ids, positions, token_item, item_slot, q_start, kv_len, logit_rows, requests):
        self.token_ids = token_ids
        self.positions = positions
        self.token_item = token_item
        self.item_slot = item_slot
        self.q_start = q_start
        self.kv_len = kv_len
        self.logit_rows = logit_rows
        self.requests = requests


class StepContext:
    """Everything a part may read during one step.

    Device tensors (int32): ``token_ids[T]``, ``positions[T]``, ``token_item[T]`` (index of the
    entry a token belongs to), ``token_slot[T]`` (slot of the token's request: the row of its block tables),
    ``item_slot[I]``, ``q_start[I+1]`` (first token of each entry), ``kv_len[I]`` (the request's length
    after this step), ``logit_rows[R]`` (flat token index of each wanted place), ``block_tables[g]``
    (``[slots + 1, max pages]`` per cache group, indexed by SLOT; -1 = no page).  Everything but
    ``token_ids`` (unless fed back), ``item_slot``, ``q_start`` and ``logit_rows`` is written by the step's
    first kernel (``ModelRunner.begin``), so it holds once that kernel has run.
    Items are laid out short entries first (``num_short_items`` items, ``num_short_tokens`` tokens), then
    the prompt portions of ``LONG_ENTRY`` or more tokens; ``logit_rows`` keeps the caller's order.
    ``status`` is a device int32 that kernels set non-zero on bad input (checked after the step).
    """

    LONG_ENTRY = 16          # entries of at least this many tokens count as prompt portions

    def __init__(self, layout: BatchLayout, device_buffer: torch.Tensor, host: HostBatch, cache, status,
                 max_q_len: int, max_kv_len: int, num_short_items: int = None, num_short_tokens: int = None,
                 num_long_blocks: int = 0, views: "DeviceViews" = None):
        self.layout = layout
        self._host = host            # a HostBatch, or a function that makes it when somebody asks
        self.cache = cache
        self.status = status
        self.num_tokens = layout.num_tokens
        self.num_items = layout.num_items
        self.num_logit_rows = layout.num_rows
        self.max_q_len = max_q_len
        self.max_kv_len = max_kv_len
        # short entries come first in the flat batch; long ones (prompt portions) after them
        self.num_short_items = layout.num_items if num_short_items is None else num_short_items
        self.num_short_tokens = layout.num_tokens if num_short_tokens is None else num_short_tokens
        self.num_long_blocks = num_long_blocks      # 64-query blocks of the long entries
        views = views if views is not None else DeviceViews(layout, device_buffer)
        self.views = views
        self.token_ids = views.token_ids
        self.positions = views.positions
        self.token_item = views.token_item
        self.token_slot = views.token_slot
        self.item_slot = views.item_slot
        self.q_start = views.q_start
        self.kv_len = views.kv_len
        self.logit_rows = views.logit_rows
        self.temperature = views.temperature
        self.seed = views.seed
        self.step_counter = views.step_counter
        self.block_tables = cache.slots.table_views
        self.decode_only = (layout.num_tokens == layout.num_items)

    @property
    def host(self) -> HostBatch:
        """The step as host arrays (computed on first use: only parts with host logic and tests ask)."""
        if callable(self._host):
            self._host = self._host()
        return self._host


class DeviceViews:
    """The sections of the packed device buffer as tensors; depends on the layout only, so the runner
    keeps one per step shape."""

    def __init__(self, layout: BatchLayout, device_buffer: torch.Tensor):
        T, I, R = layout.num_tokens, layout.num_items, layout.num_rows
        buf = device_buffer
        self.meta = buf
        self.token_ids = buf[layout.token_ids:layout.token_ids + T]
        self.positions = buf[layout.positions:layout.positions + T]
        self.token_item = buf[layout.token_item:layout.token_item + T]
        self.token_slot = buf[layout.token_slot:layout.token_slot + T]
        self.item_slot = buf[layout.item_slot:layout.item_slot + I]
        self.q_start = buf[layout.q_start:layout.q_start + I + 1]
        self.kv_len = buf[layout.kv_len:layout.kv_len + I]
        self.logit_rows = buf[layout.logit_rows:layout.logit_rows + R]
        self.temperature = buf[layout.temperature:layout.temperature + I].view(torch.float32)
        self.seed = buf[layout.seed:layout.seed + 2 * I].view(torch.int64)
        self.step_counter = buf[layout.counter:layout.counter + 1]
