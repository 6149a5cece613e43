"""The step function: run a batch of (request, its next tokens) from the cache.

reference: ``PagedDecoderLM.forward_iteration`` (src/model/paged_decoder.py:509-619).
A step may hold whole prompts, portions of prompts cut anywhere and single
decoded tokens, each request at most once (reference: src/model/iteration.py:58-63).
It runs only the tokens it is given, as one flat batch, against the pages that
earlier steps left, and returns float32 logits at the wanted places, in the
order of the entries and of their ``want`` lists.
"""

from __future__ import annotations

from typing import Hashable, List, Sequence

import numpy as np
import torch

from pagedserve_b200.cache.manager import CacheFull, CacheManager
from pagedserve_b200.engine.batch import BatchLayout, HostBatch, StepContext, StepEntry


class StepError(ValueError):
    pass


class ModelRunner:
    """Owns the device metadata buffers and drives ``model.forward`` for one step."""

    STAGING_BUFFERS = 4

    def __init__(self, model, cache: CacheManager, device, max_step_tokens: int = 8192):
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size = model.spec.vocab_size
        self.max_model_len = model.spec.max_model_len
        self.table_widths = [group.max_pages_per_request for group in cache.groups]
        self._capacity = 0
        self._device_buffer = None
        self._staging = []
        self._staging_events = []
        self._turn = 0
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._grow(BatchLayout(max_step_tokens, min(max_step_tokens, cache.max_slots),
                               min(max_step_tokens, 4 * cache.max_slots), self.table_widths).total)
        self.steps = 0
        self.tokens_run = 0

    def _grow(self, needed: int) -> None:
        if needed <= self._capacity:
            return
        torch.cuda.synchronize(self.device)
        self._capacity = int(needed * 1.25) + 64
        self._device_buffer = torch.empty(self._capacity, dtype=torch.int32, device=self.device)
        self._staging = [torch.empty(self._capacity, dtype=torch.int32).pin_memory()
                         for _ in range(self.STAGING_BUFFERS)]
        self._staging_events = [None] * self.STAGING_BUFFERS

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Validate, take pages for the new positions, build and upload the metadata."""
        if not entries:
            raise StepError("a step cannot be empty")                 # reference: iteration.py:50-51
        cache = self.cache
        seen = set()
        for entry in entries:
            if entry.request in seen:
                raise StepError("a request can appear only once in a step")   # reference: iteration.py:62-63
            seen.add(entry.request)
            bad = [t for t in entry.tokens if not (0 <= t < self.vocab_size)]
            if bad:
                raise StepError(f"token id {bad[0]} is outside the vocabulary of {self.vocab_size}")

        admitted: List[Hashable] = []
        extended: List[Hashable] = []
        try:
            for entry in entries:
                if entry.request not in cache:
                    cache.admit(entry.request)
                    admitted.append(entry.request)
                start = cache.length(entry.request)
                if start + len(entry.tokens) > self.max_model_len:
                    # reference: src/model/paged_decoder.py:521-522
                    raise StepError(f"request {entry.request!r} would pass the model's maximum length "
                                    f"{self.max_model_len}")
                cache.extend(entry.request, len(entry.tokens))
                extended.append(entry.request)
        except Exception:
            for request in extended:
                cache.rollback(request)
            for request in admitted:
                cache.free(request)
            raise
        self._admitted_in_step = admitted

        T = sum(len(entry.tokens) for entry in entries)
        I = len(entries)
        R = sum(len(entry.want) for entry in entries)
        layout = BatchLayout(T, I, R, self.table_widths)
        self._grow(layout.total)
        turn = self._turn
        self._turn = (turn + 1) % self.STAGING_BUFFERS
        if self._staging_events[turn] is not None:
            self._staging_events[turn].synchronize()
        staging = self._staging[turn]
        host = staging.numpy()

        token_ids = host[layout.token_ids:layout.token_ids + T]
        positions = host[layout.positions:layout.positions + T]
        token_item = host[layout.token_item:layout.token_item + T]
        item_slot = host[layout.item_slot:layout.item_slot + I]
        q_start = host[layout.q_start:layout.q_start + I + 1]
        kv_len = host[layout.kv_len:layout.kv_len + I]
        logit_rows = host[layout.logit_rows:layout.logit_rows + R]
        cursor = 0
        row = 0
        max_q = 0
        max_kv = 0
        for index, entry in enumerate(entries):
            count = len(entry.tokens)
            start = cache.length(entry.request)
            token_ids[cursor:cursor + count] = entry.tokens
            positions[cursor:cursor + count] = np.arange(start, start + count, dtype=np.int32)
            token_item[cursor:cursor + count] = index
            item_slot[index] = cache.slot_of[entry.request]
            q_start[index] = cursor
            kv_len[index] = start + count
            for place in entry.want:
                logit_rows[row] = cursor + place
                row += 1
            max_q = max(max_q, count)
            max_kv = max(max_kv, start + count)
            cursor += count
        q_start[I] = cursor
        for group_index, (offset, width) in enumerate(zip(layout.tables, layout.table_widths)):
            table = host[offset:offset + I * width].reshape(I, width)
            for index, entry in enumerate(entries):
                cache.table_row(group_index, entry.request, table[index])

        self._device_buffer[:layout.total].copy_(staging[:layout.total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._staging_events[turn] = event
        host_batch = HostBatch(token_ids.copy(), positions.copy(), token_item.copy(), item_slot.copy(),
                               q_start.copy(), kv_len.copy(), logit_rows.copy(),
                               [entry.request for entry in entries])
        self.h2d_bytes = layout.total * 4
        return StepContext(layout, self._device_buffer, host_batch, cache, self._status, max_q, max_kv)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one step; returns float32 logits ``[R, V]`` (R may be 0)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        ctx = self.prepare(entries)
        try:
            logits = self.model.forward(ctx)
        except Exception:
            for entry in entries:
                self.cache.rollback(entry.request)
            for request in self._admitted_in_step:
                self.cache.free(request)
            raise
        for entry in entries:
            self.cache.commit(entry.request)
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        expected = sum(len(entry.want) for entry in entries)
        if logits.shape[0] != expected:
            # reference: src/scheduler/orca_scheduler.py:260-263, 281-286
            raise StepError(f"model returned {logits.shape[0]} logits rows, expected {expected}")
        return logits

    def finish(self, request: Hashable) -> None:
        """The request is done: its pages and its slot are given back."""
        self.cache.free(request)

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input (reads one int from the device)."""
        flag = int(self._status.item())
        if flag:
            self._status.zero_()
            raise StepError(f"a kernel reported bad input (status {flag})")
