"""Cache manager: keys and values in pages, a block table per request, state slots.

What the reference does (src/model/kv_manager.py): one uniform pool
``[layers, blocks, heads, block, head_dim]`` for keys and one for values
(:77-86), a LIFO free list (:66, 115-127), a block-id list per request (:9-16),
pages given back when a request is freed (:425-442), ``"KV cache full"`` when
none is left (:116-117).

What is different here:

* Layers are put in **groups** by what they need of the cache (kv heads, head
  size, attention window).  Each group has its own pool, free list and block
  tables, so a group of windowed layers can give back the pages its window has
  passed while a group of full-attention layers keeps all of them.
* A page id addresses all cache layers of its group at once; the pool of a
  group is ``[pages, cache layers, 2 (k,v), kv heads, page size, head dim]``.
* Every live request also holds a **slot**: an index into fixed-size
  per-request state: on the device its length, last token, sampling
  parameters and block tables (:class:`pagedserve_b200.cache.slots.SlotStore`,
  kept up to date by corrections that travel with each step), and one state
  tensor per layer that declares a :class:`StateNeed`.  GPT-2 declares none;
  the slot mechanism is what a mixer with a state of fixed size uses instead
  of pages.
* The protocol is host-side and has two phases per step: ``extend`` makes sure
  pages exist for the step's new positions (all or nothing), the kernels write
  them, ``commit`` advances the length and releases pages behind a window.
  (The reference reserves one token at a time and tracks per-layer writes:
  src/model/kv_manager.py:149-224.)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

try:  # torch is only needed when pools live on a device
    import torch
except ImportError:  # pragma: no cover
    torch = None

from pagedserve_b200.cache.slots import SlotStore


class CacheError(RuntimeError):
    """A protocol violation: unknown request, double free, and the like."""


class CacheFull(CacheError):
    """No free page (or slot) is left.  reference: src/model/kv_manager.py:116-117"""


@dataclass(frozen=True)
class KVNeed:
    """What an attention-like mixer needs of the paged cache."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: all earlier keys; w: the last w keys


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size kept in the request's slot."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


class PageAllocator:
    """LIFO free list of page ids with ownership checks.

    The first page handed out is the highest id, and a page that was just
    released is the next to be handed out (reference: ``list.pop`` /
    ``append`` at src/model/kv_manager.py:115-127).
    """

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages))
        self._held = np.zeros(num_pages, dtype=bool)
        self.peak_used = 0

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise CacheFull("KV cache full")
        page = self._free.pop()
        if self._held[page]:
            raise CacheError(f"page {page} handed out twice")
        self._held[page] = True
        self.peak_used = max(self.peak_used, self.used_pages)
        return page

    def allocate_many(self, count: int) -> List[int]:
        """``count`` pages in the order that ``allocate`` would hand them out, or none at all."""
        if count > len(self._free):
            raise CacheFull("KV cache full")
        if count <= 0:
            return []
        pages = self._free[-count:][::-1]
        del self._free[-count:]
        taken = np.asarray(pages, dtype=np.int64)
        if self._held[taken].any():
            raise CacheError("a page was handed out twice")
        self._held[taken] = True
        self.peak_used = max(self.peak_used, self.used_pages)
        return pages

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page id {page} is outside the pool")
        if not self._held[page]:
            raise CacheError(f"page {page} freed twice")
        self._held[page] = False
        self._free.append(page)

    def reset_peak(self) -> None:
        self.peak_used = self.used_pages


class CacheGroup:
    """Layers with the same :class:`KVNeed`: one pool, one free list, one set of tables."""

    def __init__(self, need: KVNeed, cache_layers: Sequence[int], page_size: int, num_pages: int,
                 max_pages_per_request: int, dtype=None, device=None, scratch_pages: int = 0):
        self.need = need
        self.cache_layers = list(cache_layers)      # global cache-layer ids, in pool order
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages_per_request = max_pages_per_request
        self.allocator = PageAllocator(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}
        self.rows = None                            # [slots, max pages] int32 mirror of the tables, -1 = no page
        self.pool = None
        # pages behind the allocator's range that belong to no request (padding tokens of a step write there)
        self.scratch_pages = list(range(num_pages, num_pages + scratch_pages))
        if device is not None:
            shape = (num_pages + scratch_pages, len(self.cache_layers), 2, need.n_kv_heads, page_size,
                     need.head_dim)
            self.pool = torch.empty(shape, dtype=dtype, device=device)

    # strides in elements, used by the kernels
    @property
    def page_stride(self) -> int:
        return len(self.cache_layers) * 2 * self.need.n_kv_heads * self.page_size * self.need.head_dim

    def layer_views(self, cache_layer: int):
        """(k, v) views ``[pages, kv heads, page size, head dim]`` of one cache layer."""
        local = self.cache_layers.index(cache_layer)
        return self.pool[:, local, 0], self.pool[:, local, 1]

    @property
    def bytes_per_page(self) -> int:
        width = self.pool.element_size() if self.pool is not None else 0
        return self.page_stride * width

    def first_needed_position(self, length: int) -> int:
        """Lowest key position that a token at position >= ``length`` can still attend."""
        if self.need.window is None:
            return 0
        return max(0, length - self.need.window + 1)


class CacheManager:
    """Pages, block tables and slots for all live requests.

    ``kv_needs[i]`` is the need of cache layer ``i`` (``None`` for a layer that
    keeps nothing in pages); ``state_needs[i]`` likewise for slot state.
    """

    def __init__(self, kv_needs: Sequence[Optional[KVNeed]], state_needs: Sequence[Optional[StateNeed]],
                 page_size: int, num_pages: int, max_slots: int, max_model_len: int,
                 dtype=None, device=None, scratch_tokens: int = 0):
        if page_size <= 0 or (page_size & (page_size - 1)) or page_size > 64:
            raise CacheError("page_size must be a power of two, at most 64")
        if max_slots <= 0:
            raise CacheError("max_slots must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_model_len = max_model_len
        self.max_pages_per_request = -(-max_model_len // page_size)
        self.device = device
        self.dtype = dtype

        by_need: Dict[KVNeed, List[int]] = {}
        for layer, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(layer)
        # A scratch slot (index max_slots) with pages for ``scratch_tokens`` positions, outside the allocator and
        # the slot list: a step that pads its batch to a recurring shape sends the padding there.
        self.scratch_tokens = min(scratch_tokens, max_model_len)
        scratch_pages = -(-self.scratch_tokens // page_size)
        self.scratch_slot = max_slots
        self.groups: List[CacheGroup] = [
            CacheGroup(need, layers, page_size, num_pages, self.max_pages_per_request, dtype, device, scratch_pages)
            for need, layers in by_need.items()
        ]
        # the device copy of every slot's state: lengths, sampling parameters, block tables by slot
        self.slots = SlotStore(max_slots, [self.max_pages_per_request] * len(self.groups))
        for index, group in enumerate(self.groups):
            # the tables once more as one array by slot: what the slot store's tables must equal
            group.rows = np.full((max_slots + 1, self.max_pages_per_request), -1, dtype=np.int32)
            group.rows[max_slots, :scratch_pages] = group.scratch_pages
            self.slots.set_table(index, max_slots, 0, group.scratch_pages)
        if device is not None:
            self.slots.attach(device)
        self.group_of_layer: Dict[int, int] = {
            layer: index for index, group in enumerate(self.groups) for layer in group.cache_layers
        }

        # slots: fixed-size per-request state
        self._free_slots: List[int] = list(range(max_slots - 1, -1, -1))   # pop() gives slot 0 first
        self.slot_of: Dict[Hashable, int] = {}
        self.lengths = np.zeros(max_slots, dtype=np.int32)        # committed tokens per slot
        self.pending = np.zeros(max_slots, dtype=np.int32)        # tokens extended but not committed
        self.state: Dict[int, "torch.Tensor"] = {}
        self.state_needs = list(state_needs)
        if device is not None:
            for layer, need in enumerate(state_needs):
                if need is not None:
                    self.state[layer] = torch.zeros((max_slots + 1, *need.shape), dtype=getattr(torch, need.dtype),
                                                    device=device)

    # ------------------------------------------------------------------ queries
    def __contains__(self, request: Hashable) -> bool:
        return request in self.slot_of

    @property
    def live_requests(self) -> int:
        return len(self.slot_of)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def length(self, request: Hashable) -> int:
        return int(self.lengths[self._slot(request)])

    def _slot(self, request: Hashable) -> int:
        if request not in self.slot_of:
            raise CacheError(f"unknown request {request!r}")
        return self.slot_of[request]

    def pages_for_tokens(self, tokens: int) -> int:
        """Pages one group needs to hold ``tokens`` tokens of one request (no window credit)."""
        return -(-tokens // self.page_size)

    def free_pages(self) -> int:
        """Free pages of the tightest group."""
        if not self.groups:
            return 1 << 30
        return min(group.allocator.free_pages for group in self.groups)

    def total_pages(self) -> int:
        if not self.groups:
            return 1 << 30
        return min(group.num_pages for group in self.groups)

    # ------------------------------------------------------------------ protocol
    def admit(self, request: Hashable) -> int:
        """Give ``request`` a slot (length 0, state zeroed); returns the slot index."""
        if request in self.slot_of:
            raise CacheError(f"request {request!r} is already live")
        if not self._free_slots:
            raise CacheFull("no free request slot")
        slot = self._free_slots.pop()
        self.slot_of[request] = slot
        self.lengths[slot] = 0
        self.pending[slot] = 0
        for tensor in self.state.values():
            tensor[slot].zero_()
        for group in self.groups:
            group.tables[request] = []          # the slot's row is all -1 since its last owner was freed
        return slot

    def extend(self, request: Hashable, new_tokens: int) -> None:
        """Make sure pages exist for positions [length, length + new_tokens) in every group.

        All or nothing: if any group runs out, pages taken by this call are given
        back and :class:`CacheFull` is raised (reference rolls a failed chunk
        back the same way: src/model/kv_manager.py:267-274).
        """
        slot = self._slot(request)
        if new_tokens <= 0:
            raise CacheError("extend needs a positive token count")
        if self.pending[slot]:
            raise CacheError("the previous extension was not committed")   # reference: kv_manager.py:151-152
        end = int(self.lengths[slot]) + new_tokens
        if end > self.max_model_len:
            raise CacheError(f"request {request!r} would exceed the model's maximum length {self.max_model_len}")
        needed = -(-end // self.page_size)
        taken: List[Tuple[CacheGroup, List[int], int]] = []
        try:
            for index, group in enumerate(self.groups):
                table = group.tables[request]
                old_len = len(table)
                fresh: List[int] = []
                taken.append((index, group, fresh, old_len))
                if needed > old_len:
                    fresh.extend(group.allocator.allocate_many(needed - old_len))
                    self._set_rows(index, slot, old_len, fresh)
                    table.extend(fresh)
        except CacheFull:
            for index, group, fresh, old_len in taken:
                del group.tables[request][old_len:]
                self._set_rows(index, slot, old_len, [-1] * len(fresh), device=False)
                for page in reversed(fresh):
                    group.allocator.release(page)
            raise
        self.pending[slot] = new_tokens

    def _set_rows(self, group_index: int, slot: int, first_column: int, pages, device: bool = True) -> None:
        """Write page ids into a slot's table row: the host array and, queued, the device's.

        ``device=False`` leaves the device's copy as it is: entries that are taken back (a request freed, an
        extension undone) lie beyond every length a kernel is given, so nothing reads them, and a step's
        corrections stay bounded by the pages its own tokens start."""
        if len(pages):
            self.groups[group_index].rows[slot, first_column:first_column + len(pages)] = pages
            if device:
                self.slots.set_table(group_index, slot, first_column, pages)

    def extend_many(self, requests: Sequence[Hashable], counts: Sequence[int]) -> None:
        """``extend`` for several requests at once (each at most once), all or nothing.

        Most entries of a step are single decoded tokens that stay inside their last page: those are settled
        with whole-array operations, and only the requests that need a new page go through ``extend``."""
        try:
            slots = np.fromiter((self.slot_of[request] for request in requests), dtype=np.int64,
                                count=len(requests))
        except KeyError as missing:
            raise CacheError(f"unknown request {missing.args[0]!r}") from None
        counts = np.asarray(counts, dtype=np.int64)
        if counts.shape != slots.shape:
            raise CacheError("extend_many needs one count per request")
        if slots.size == 0:
            return
        if (counts <= 0).any():
            raise CacheError("extend needs a positive token count")
        if len(set(requests)) != len(requests):
            raise CacheError("a request can be extended only once at a time")
        if self.pending[slots].any():
            raise CacheError("the previous extension was not committed")
        starts = self.lengths[slots].astype(np.int64)
        ends = starts + counts
        if (ends > self.max_model_len).any():
            worst = requests[int(np.argmax(ends))]
            raise CacheError(f"request {worst!r} would exceed the model's maximum length {self.max_model_len}")
        # a table has a page for every committed position (released ones keep their place as -1)
        crossing = np.flatnonzero(-(-ends // self.page_size) > -(-starts // self.page_size))
        done: List[Hashable] = []
        try:
            for index in crossing.tolist():
                self.extend(requests[index], int(counts[index]))
                done.append(requests[index])
        except CacheFull:
            for request in reversed(done):          # last taken, first returned: the free list is as before
                self.rollback(request)
            raise
        self.pending[slots] = counts

    def commit_many(self, requests: Sequence[Hashable]) -> None:
        """``commit`` for several requests at once."""
        if any(group.need.window is not None for group in self.groups):
            for request in requests:                # pages that a window has passed are released one by one
                self.commit(request)
            return
        try:
            slots = np.fromiter((self.slot_of[request] for request in requests), dtype=np.int64,
                                count=len(requests))
        except KeyError as missing:
            raise CacheError(f"unknown request {missing.args[0]!r}") from None
        if slots.size == 0:
            return
        pending = self.pending[slots]
        if not pending.all():
            raise CacheError("nothing to commit")
        self.lengths[slots] += pending
        self.pending[slots] = 0

    def rollback(self, request: Hashable) -> None:
        """Undo an ``extend`` that was not committed (the step failed)."""
        slot = self._slot(request)
        if not self.pending[slot]:
            return
        keep = -(-int(self.lengths[slot]) // self.page_size)
        for index, group in enumerate(self.groups):
            table = group.tables[request]
            for page in reversed(table[keep:]):
                if page >= 0:
                    group.allocator.release(page)
            self._set_rows(index, slot, keep, [-1] * (len(table) - keep), device=False)
            del table[keep:]
        self.pending[slot] = 0

    def commit(self, request: Hashable) -> int:
        """The step wrote the extended positions: advance the length, release pages that
        every window of a group has passed.  Returns the new length."""
        slot = self._slot(request)
        if not self.pending[slot]:
            raise CacheError("nothing to commit")                          # reference: kv_manager.py:210-211
        self.lengths[slot] += self.pending[slot]
        self.pending[slot] = 0
        length = int(self.lengths[slot])
        for group_index, group in enumerate(self.groups):
            if group.need.window is None:
                continue
            first = group.first_needed_position(length)
            table = group.tables[request]
            for index in range(first // self.page_size):
                if table[index] >= 0:
                    group.allocator.release(table[index])
                    table[index] = -1
                    self._set_rows(group_index, slot, index, [-1])
        return length

    def free(self, request: Hashable) -> None:
        """Give back every page and the slot (reference: src/model/kv_manager.py:425-442)."""
        slot = self._slot(request)
        if self.pending[slot]:
            raise CacheError("cannot free a request with an uncommitted extension")
        for index, group in enumerate(self.groups):
            table = group.tables.pop(request)
            live = [page for page in table if page >= 0]
            if len(live) != len(set(live)):
                raise CacheError("request holds a page twice")
            for page in live:
                group.allocator.release(page)
            self._set_rows(index, slot, 0, [-1] * len(table), device=False)
        del self.slot_of[request]
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    # ------------------------------------------------------------------ tables for a step
    def table_row(self, group_index: int, request: Hashable, out: np.ndarray) -> None:
        """Write the request's block table (padded with -1) into ``out`` (int32 [max_pages])."""
        out[:] = self.groups[group_index].rows[self._slot(request)]

    def table_rows(self, group_index: int, slots: np.ndarray, out: np.ndarray) -> None:
        """The block tables of several slots at once into ``out`` (int32 [len(slots), max_pages])."""
        np.take(self.groups[group_index].rows, slots, axis=0, out=out)

    # ------------------------------------------------------------------ checks and figures
    def check_invariants(self) -> None:
        """No page lost, none held twice: free + held == pool, in every group."""
        for group in self.groups:
            held = [page for table in group.tables.values() for page in table if page >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is held by two requests")
            free = group.allocator._free
            if len(free) != len(set(free)):
                raise CacheError("a page is on the free list twice")
            if set(free) & set(held):
                raise CacheError("a page is both free and held")
            if len(free) + len(held) != group.num_pages:
                raise CacheError(f"pages lost: {group.num_pages - len(free) - len(held)}")
            for request, table in group.tables.items():
                row = group.rows[self.slot_of[request]]
                if row[:len(table)].tolist() != table or (row[len(table):] != -1).any():
                    raise CacheError(f"the table array of request {request!r} differs from its table")
        for index, group in enumerate(self.groups):
            base, width = self.slots.tables[index], self.slots.table_widths[index]
            mirrored = self.slots.mirror[base:base + group.rows.size].reshape(group.rows.shape)
            for request, table in group.tables.items():        # what a kernel may read: the live requests' entries
                slot = self.slot_of[request]
                if mirrored[slot, :len(table)].tolist() != table:
                    raise CacheError(f"the slot store's block table of request {request!r} differs from the host's")
            free_rows = [slot for slot in self._free_slots]
            if free_rows and (group.rows[free_rows] != -1).any():
                raise CacheError("a free slot still has pages in its table row")
        slots = list(self.slot_of.values())
        if len(slots) != len(set(slots)) or len(slots) + len(self._free_slots) != self.max_slots:
            raise CacheError("slot bookkeeping is inconsistent")

    def usage_summary(self) -> dict:
        """reference: src/model/kv_manager.py:134-147"""
        groups = []
        for group in self.groups:
            groups.append({
                "cache_layers": list(group.cache_layers),
                "window": group.need.window,
                "total_blocks": group.num_pages,
                "free_blocks": group.allocator.free_pages,
                "peak_allocated_blocks": group.allocator.peak_used,
                "peak_allocated_tokens": group.allocator.peak_used * self.page_size,
                "bytes_per_block": group.bytes_per_page,
                "peak_utilization_percent": 100.0 * group.allocator.peak_used / group.num_pages,
            })
        return {"block_size": self.page_size, "live_requests": self.live_requests,
                "free_slots": self.free_slots, "groups": groups}
