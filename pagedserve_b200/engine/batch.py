"""What one step runs: a flat batch of (request, its next tokens).

The reference describes a step with ``IterationItem`` / ``IterationBatch``
(reference: src/model/iteration.py:10-74): per item a request id, phase, token
ids, position ids, flattened offsets and ``produces_output``.  Here an entry
carries only the request, its next tokens and the places whose logits are
wanted; positions follow from the request's cached length, and a "decode" is
simply an entry of one token.  The device side is one packed int32 buffer
(one host-to-device copy per step).
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
        if tokens.size and not np.issubdtype(tokens.dtype, np.integer):
            raise ValueError("token ids must be integers")
        self.tokens = tokens.astype(np.int64, copy=False).reshape(-1)      # kept as an array: prompts are long
        self.want = [int(w) for w in self.want]
        if self.tokens.size == 0:
            # reference: src/model/iteration.py:23-24
            raise ValueError("a step entry must contain at least one token")
        for place in self.want:
            if not (0 <= place < len(self.tokens)):
                raise ValueError(f"wanted place {place} is outside the entry's {len(self.tokens)} tokens")


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of the sections of the packed metadata buffer."""

    num_tokens: int
    num_items: int
    num_rows: int
    table_widths: Sequence[int]
    token_ids: int = 0
    positions: int = 0
    token_item: int = 0
    item_slot: int = 0
    q_start: int = 0
    kv_len: int = 0
    logit_rows: int = 0
    temperature: int = 0          # float32 bits, one per item
    seed: int = 0                 # 64-bit, two words per item
    counter: int = 0              # one word, uploaded as 0: decode steps the device has run since the upload
    tables: List[int] = field(default_factory=list)
    total: int = 0

    def __post_init__(self):
        cursor = 0
        for name, count in (("token_ids", self.num_tokens), ("positions", self.num_tokens),
                            ("token_item", self.num_tokens), ("item_slot", self.num_items),
                            ("q_start", self.num_items + 1), ("kv_len", self.num_items),
                            ("logit_rows", max(self.num_rows, 1)), ("temperature", self.num_items),
                            ("seed", 2 * self.num_items), ("counter", 1)):
            setattr(self, name, cursor)
            cursor += _pad4(count)
        self.tables = []
        for width in self.table_widths:
            self.tables.append(cursor)
            cursor += _pad4(self.num_items * width)
        self.total = cursor


class HostBatch:
    """Host-side (numpy) view of a step, for parts that need host logic and for tests.

    The arrays are views of the step's pinned staging buffer: they hold while the step runs and are
    overwritten a few steps later."""

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
    entry a token belongs to), ``item_slot[I]``, ``q_start[I+1]`` (first token of each entry),
    ``kv_len[I]`` (the request's length after this step), ``logit_rows[R]`` (flat token index of
    each wanted place), ``block_tables[g]`` (``[I, max pages]`` per cache group; -1 = no page).
    Items are laid out short entries first (``num_short_items`` items, ``num_short_tokens`` tokens), then
    the prompt portions of ``LONG_ENTRY`` or more tokens; ``logit_rows`` keeps the caller's order.
    ``status`` is a device int32 that kernels set non-zero on bad input (checked after the step).
    """

    LONG_ENTRY = 16          # entries of at least this many tokens count as prompt portions

    def __init__(self, layout: BatchLayout, device_buffer: torch.Tensor, host: HostBatch, cache, status,
                 max_q_len: int, max_kv_len: int, num_short_items: int = None, num_short_tokens: int = None,
                 num_long_blocks: int = 0, views: "DeviceViews" = None):
        self.layout = layout
        self.host = host
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
        self.token_ids = views.token_ids
        self.positions = views.positions
        self.token_item = views.token_item
        self.item_slot = views.item_slot
        self.q_start = views.q_start
        self.kv_len = views.kv_len
        self.logit_rows = views.logit_rows
        self.temperature = views.temperature
        self.seed = views.seed
        self.step_counter = views.step_counter
        self.block_tables = views.block_tables
        self.decode_only = (layout.num_tokens == layout.num_items)


class DeviceViews:
    """The sections of the packed device buffer as tensors; depends on the layout only, so the runner
    keeps one per step shape."""

    def __init__(self, layout: BatchLayout, device_buffer: torch.Tensor):
        T, I, R = layout.num_tokens, layout.num_items, layout.num_rows
        buf = device_buffer
        self.token_ids = buf[layout.token_ids:layout.token_ids + T]
        self.positions = buf[layout.positions:layout.positions + T]
        self.token_item = buf[layout.token_item:layout.token_item + T]
        self.item_slot = buf[layout.item_slot:layout.item_slot + I]
        self.q_start = buf[layout.q_start:layout.q_start + I + 1]
        self.kv_len = buf[layout.kv_len:layout.kv_len + I]
        self.logit_rows = buf[layout.logit_rows:layout.logit_rows + R]
        self.temperature = buf[layout.temperature:layout.temperature + I].view(torch.float32)
        self.seed = buf[layout.seed:layout.seed + 2 * I].view(torch.int64)
        self.step_counter = buf[layout.counter:layout.counter + 1]
        self.block_tables = [
            buf[offset:offset + I * width].view(I, width)
            for offset, width in zip(layout.tables, layout.table_widths)
        ]
