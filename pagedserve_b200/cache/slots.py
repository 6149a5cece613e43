"""The slot store: per-request state of fixed size that lives on the device.

Every live request holds a slot (:class:`pagedserve_b200.cache.manager.CacheManager`).  What the kernels need
to know about a request between steps is kept on the device, indexed by slot, in one int32 array:

=========  ============================================================================
section    per slot
=========  ============================================================================
len        tokens in the cache, i.e. the position of the request's next token
last       the token sampled last (the next input when a decode step feeds tokens back)
temp       sampling temperature (float32 bits)
seed       sampling seed (two words)
table g    the block table of cache group ``g``: ``width_g`` page ids, -1 = no page
=========  ============================================================================

(The reference keeps this on the host, ``RequestInfo`` at src/model/kv_manager.py:9-16, and rebuilds the device
copy of tables and lengths for every decode step, src/model/kv_manager.py:521-561.)

The host keeps a mirror of the array: what the device holds once every correction handed out so far has been
applied.  Writers call :meth:`set` / :meth:`set_many`; only words whose value really changes are queued.
A step drains the queue (:meth:`drain`) into its one upload as ``(offset, value)`` pairs, which the step's
first kernel applies.  A decode token that stays inside its last page therefore uploads no table entry at all,
and the upload of a step does not grow with the model's maximum context.

The device moves ``len`` on by itself at the start of every step (and ``last`` at its end); the runner tells
the mirror (:meth:`device_advanced`).  Where host and mirror disagree about a length, the runner queues a
correction, so the host's bookkeeping is the truth and the device copy heals itself: a request admitted into a
used slot, a step that was launched ahead and then dropped, a step that failed half-way.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

try:
    import torch
except ImportError:  # pragma: no cover
    torch = None


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class SlotStore:
    def __init__(self, max_slots: int, table_widths: Sequence[int], device=None):
        self.max_slots = max_slots
        rows = max_slots + 1                      # the last row is the scratch slot of padding entries
        self.rows = rows
        cursor = 0
        self.len = cursor
        cursor += _pad4(rows)
        self.last = cursor
        cursor += _pad4(rows)
        self.temp = cursor
        cursor += _pad4(rows)
        self.seed = cursor
        cursor += _pad4(2 * rows)
        self.table_widths = list(table_widths)
        self.tables: List[int] = []
        for width in self.table_widths:
            self.tables.append(cursor)
            cursor += _pad4(rows * width)
        self.size = cursor
        self.mirror = np.zeros(self.size, dtype=np.int32)
        for base, width in zip(self.tables, self.table_widths):
            self.mirror[base:base + rows * width] = -1
        self._pending: List[np.ndarray] = []      # offsets whose mirror value the device does not have yet
        self._pending_count = 0
        self.uploaded_words = 0                   # corrections handed out so far (a figure for tests and benchmarks)
        self.device = None
        self.store = None                         # the device array, once attached
        self.table_views = []                     # its block tables as [rows, width] tensors, one per group
        # {size, len, last, temp, seed, slots}: what the kernels are told of the layout
        self.layout_words = np.asarray([self.size, self.len, self.last, self.temp, self.seed, max_slots],
                                       dtype=np.int32)
        if device is not None:
            self.attach(device)

    def attach(self, device) -> None:
        """Create the device array from the mirror as it stands; nothing is left queued."""
        self.device = device
        self.store = torch.from_numpy(self.mirror.copy()).to(device)
        self.table_views = [self.store[base:base + self.rows * width].view(self.rows, width)
                            for base, width in zip(self.tables, self.table_widths)]
        self._pending = []
        self._pending_count = 0

    # ------------------------------------------------------------------ writers
    def set_many(self, offsets: np.ndarray, values: np.ndarray) -> int:
        """mirror[offsets] = values; queues the words that change. Returns how many did."""
        offsets = np.asarray(offsets, dtype=np.int64)
        values = np.asarray(values, dtype=np.int32)
        changed = self.mirror[offsets] != values
        if not changed.any():
            return 0
        offsets = offsets[changed]
        self.mirror[offsets] = values[changed] if values.ndim else values
        self._pending.append(offsets)
        self._pending_count += offsets.size
        return int(offsets.size)

    def set_table(self, group: int, slot: int, first_column: int, pages) -> int:
        pages = np.asarray(pages, dtype=np.int32).reshape(-1)
        if pages.size == 0:
            return 0
        base = self.tables[group] + slot * self.table_widths[group] + first_column
        return self.set_many(base + np.arange(pages.size, dtype=np.int64), pages)

    def clear_table(self, group: int, slot: int, first_column: int = 0) -> int:
        width = self.table_widths[group]
        if first_column >= width:
            return 0
        return self.set_table(group, slot, first_column, np.full(width - first_column, -1, dtype=np.int32))

    def set_lengths(self, slots: np.ndarray, lengths: np.ndarray) -> int:
        return self.set_many(self.len + np.asarray(slots, dtype=np.int64), lengths)

    def set_sampling(self, slots: np.ndarray, temperatures, seeds) -> int:
        slots = np.asarray(slots, dtype=np.int64)
        bits = np.asarray(temperatures, dtype=np.float32).view(np.int32)
        try:
            words = np.asarray(seeds, dtype=np.int64).view(np.int32)
        except OverflowError:                     # seeds of 2**63 and above
            words = np.array([int(seed) & 0xFFFFFFFFFFFFFFFF for seed in seeds], dtype=np.uint64).view(np.int32)
        changed = self.set_many(self.temp + slots, bits)
        seed_offsets = np.stack([self.seed + 2 * slots, self.seed + 2 * slots + 1], axis=1).reshape(-1)
        return changed + self.set_many(seed_offsets, words)

    def device_advanced(self, slots: np.ndarray, counts) -> None:
        """The device has moved (or is about to move) these slots' lengths on by ``counts`` itself."""
        self.mirror[self.len + np.asarray(slots, dtype=np.int64)] += np.asarray(counts, dtype=np.int32)

    def lengths_of(self, slots: np.ndarray) -> np.ndarray:
        return self.mirror[self.len + np.asarray(slots, dtype=np.int64)]

    # ------------------------------------------------------------------ the queue
    @property
    def pending(self) -> int:
        """An upper bound of the corrections waiting (an offset queued twice counts twice)."""
        return self._pending_count

    def drain(self) -> Tuple[np.ndarray, np.ndarray]:
        """(offsets, values) of every queued correction, each offset once, with its latest value."""
        if not self._pending:
            return _EMPTY, _EMPTY
        offsets = np.unique(np.concatenate(self._pending))
        self._pending = []
        self._pending_count = 0
        self.uploaded_words += 2 * offsets.size
        return offsets.astype(np.int32), self.mirror[offsets]

    def requeue(self, offsets: np.ndarray) -> None:
        """Corrections that were drained but never reached the device (a step prepared and then dropped)."""
        if len(offsets):
            self._pending.append(np.asarray(offsets, dtype=np.int64))
            self._pending_count += len(offsets)

    def take_all(self) -> np.ndarray:
        """The whole mirror, for a plain copy over the device array; the queue is then empty."""
        self._pending = []
        self._pending_count = 0
        self.uploaded_words += self.size
        return self.mirror


_EMPTY = np.zeros(0, dtype=np.int32)
