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
from pagedserve_b200.engine.batch import (BatchLayout, DeviceViews, HostBatch, StepContext, StepEntry, arrange_step,
                                           layout_order)


class StepError(ValueError):
    pass


class _DecodeGraph:
    """A captured decode-only step of one batch size: static logits and the number of kernels."""

    def __init__(self, graph, logits, kernels):
        self.graph = graph
        self.logits = logits
        self.kernels = kernels

    def replay(self):
        self.graph.replay()


class _StagedStep:
    """A decode step prepared ahead of its tokens: its pages are taken, its buffer is filled.  ``launched``:
    it is already in the stream behind the step before it, whose kernel feeds the tokens back on the device;
    ``half`` is the half of the token history it writes, ``event`` marks its end and ``fed_tokens`` are the
    tokens it was given (what the step before it sampled)."""

    def __init__(self, requests, temperatures, seeds, ctx, turn):
        self.requests = requests
        self.temperatures = temperatures
        self.seeds = seeds
        self.ctx = ctx
        self.turn = turn
        self.launched = False
        self.half = 0
        self.event = None
        self.fed_tokens = None


class ModelRunner:
    """Owns the device metadata buffers and drives ``model.forward`` for one step."""

    STAGING_BUFFERS = 4

    MAX_DEVICE_STEPS = 1024          # most decode steps one ``decode`` call runs without the host
    # Destroying a captured graph returns its memory to the device, which stalls the stream for tens of
    # milliseconds: the limit is generous, and step shapes are bucketed so that few graphs are needed.
    MAX_GRAPHS = 512
    # A capture costs 6 to 14 ms (its allocations come fresh from the device even in the shared pool), an
    # eager mixed step about a millisecond of the host more than a replay: a shape is worth a graph once it has
    # come back a few times. Measured with 256 requests of random lengths (third pass): 42.1 k output tokens/s
    # when capturing at the second sighting, 44.4 k at the fourth, 44.3 k at the eighth, 36.4 k without graphs.
    MIXED_SHAPE_SIGHTINGS = 4
    # Mixed steps are padded to recurring shapes so that their graphs are found again: short tokens to a
    # multiple of PAD_SHORT, tokens of prompt portions to a multiple of PAD_LONG, entries and wanted rows to
    # multiples of 8 and 4. The padding tokens belong to the cache's scratch slot.
    PAD_SHORT = 16
    PAD_LONG = 128

    def __init__(self, model, cache: CacheManager, device, max_step_tokens: int = 8192,
                 enable_cuda_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size = model.spec.vocab_size
        self.max_model_len = model.spec.max_model_len
        self.slots = cache.slots              # per-request state on the device, corrected by each step's upload
        self._capacity = 0
        self._device_buffer = None
        self._staging = []
        self._staging_events = []
        self._turn = 0
        self.ops = model.env.ops
        if self.ops.arena is None:
            from pagedserve_b200.kernels.ops import StepArena

            self.ops.arena = StepArena()
        self._status = self.ops.status_flag(self.device)      # one flag for every kernel of the model's steps
        self._resync_pinned = None           # staging of a whole-store copy, made when one is first needed
        self._needs_resync = False
        self._grow(self._layout(max_step_tokens, min(max_step_tokens, cache.max_slots),
                                min(max_step_tokens, 4 * cache.max_slots)).total)
        self.steps = 0
        self.tokens_run = 0
        self.enable_cuda_graphs = enable_cuda_graphs and model.graph_safe
        # padding needs the scratch slot's pages and positions 0 .. PAD_LONG - 1 to exist in the model
        self._pad_mixed = (self.enable_cuda_graphs and cache.scratch_tokens >= self.PAD_LONG
                           and self.max_model_len >= 2 * self.PAD_LONG)
        # decode-only steps are padded too (1, 2, 4, 8, 16, 24, ... requests): one graph per bucket, not per count
        self._pad_decode = self.enable_cuda_graphs and cache.scratch_tokens >= 1
        self._graphs = {}                 # (batch size, kind) or step shape -> _DecodeGraph
        self._shape_seen = {}             # step shape -> times seen (a shape is captured when it comes back)
        self.graph_replays = 0
        self._sampled = torch.zeros(cache.max_slots, dtype=torch.int32, device=self.device)
        # the sampled tokens of a run of decode steps: page-locked host memory that the token feedback kernel
        # writes directly (no device-to-host copy after the step)
        # (its last word is the copy of the status flag that the same kernel leaves there)
        self._status_index = self.MAX_DEVICE_STEPS * cache.max_slots
        self._history = self.ops.mapped_host_buffer(self._status_index + 1)
        self._history.array[self._status_index] = 0
        self._shapes = {}                 # (T, I, R) -> (BatchLayout, DeviceViews)
        self._staged = None               # a decode step staged (and perhaps launched) ahead of its tokens
        self._step_events = [torch.cuda.Event(), torch.cuda.Event()]    # ends of the steps of the two halves
        self._capture_stream = None       # made at the first capture
        self._graph_pool = None
        self._ramp = np.arange(cache.max_slots + 2, dtype=np.int32)

    def _layout(self, T: int, I: int, R: int) -> BatchLayout:
        """The layout of a step shape.  Room for corrections: a page id per page the step's tokens can start,
        in every group, and per item a length and the sampling parameters; a step with more (many requests
        freed at once) copies the whole store instead."""
        page = self.cache.page_size
        capacity = len(self.cache.groups) * (-(-T // page) + I) + 4 * I + 8
        return BatchLayout(T, I, R, capacity)

    def _grow(self, needed: int) -> None:
        if needed <= self._capacity:
            return
        torch.cuda.synchronize(self.device)
        self._graphs = {}                 # captured graphs point into the old buffer
        self._shapes = {}
        self._capacity = int(needed * 1.25) + 64
        self._device_buffer = torch.empty(self._capacity, dtype=torch.int32, device=self.device)
        self._staging = [torch.empty(self._capacity, dtype=torch.int32).pin_memory()
                         for _ in range(self.STAGING_BUFFERS)]
        self._staging_numpy = [staging.numpy() for staging in self._staging]
        self._staging_ptr = [staging.data_ptr() for staging in self._staging]
        self._staging_events = [torch.cuda.Event() for _ in range(self.STAGING_BUFFERS)]
        for event in self._staging_events:
            event.record()

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry], pad: bool = False) -> StepContext:
        """Validate, take pages for the new positions, build and upload the metadata.  ``pad``: bring the
        batch to a recurring shape with padding tokens and empty entries (see PAD_SHORT)."""
        if not entries:
            raise StepError("a step cannot be empty")                 # reference: iteration.py:50-51
        self._drop_staged()
        cache = self.cache
        I = len(entries)
        requests = [entry.request for entry in entries]
        if len(set(requests)) != I:
            raise StepError("a request can appear only once in a step")       # reference: iteration.py:62-63
        counts = np.fromiter((len(entry.tokens) for entry in entries), dtype=np.int64, count=I)
        tokens = np.concatenate([entry.tokens for entry in entries]) if I > 1 else entries[0].tokens
        self._check_vocabulary(tokens)

        admitted: List[Hashable] = []
        slot_of = cache.slot_of
        try:
            for request in requests:
                if request not in slot_of:
                    cache.admit(request)
                    admitted.append(request)
            slots = np.fromiter((slot_of[request] for request in requests), dtype=np.int64, count=I)
            starts = cache.lengths[slots].astype(np.int64)             # cached length of each entry's request
            beyond = np.flatnonzero(starts + counts > self.max_model_len)
            if beyond.size:
                # reference: src/model/paged_decoder.py:521-522
                raise StepError(f"request {requests[int(beyond[0])]!r} would pass the model's maximum "
                                f"length {self.max_model_len}")
            cache.extend_many(requests, counts)                        # all or nothing
        except Exception:
            for request in admitted:
                cache.free(request)
            raise
        self._admitted_in_step = admitted
        # The flat batch (short entries first, prompt portions after them, padding) is laid out natively:
        # engine.batch.arrange_step is its specification and what ``ctx.host`` is computed with on demand.
        wants = [entry.want for entry in entries]
        want_counts = np.fromiter((len(want) for want in wants), dtype=np.int32, count=I)
        flat_wants = np.fromiter((place for want in wants for place in want), dtype=np.int32,
                                 count=int(want_counts.sum()))
        ops, LONG = self.ops, StepContext.LONG_ENTRY
        T, items, R, num_short_items, num_short_tokens, num_long_blocks, real_rows, max_q_len, max_kv_len = \
            ops.step_shape(counts, starts, want_counts, LONG, pad, self.PAD_SHORT, self.PAD_LONG)
        layout, views, staging, host = self._stage(T, items, R)
        bad = ops.step_fill(counts, starts, want_counts, tokens, slots, flat_wants, LONG, pad, self.PAD_SHORT,
                            self.PAD_LONG, cache.scratch_slot, self.vocab_size,
                            self._staging_ptr[self._staging_turn], layout)
        if bad is not None:                                # (checked above already: cannot happen)
            self._abandon(entries)
            raise StepError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        # where the device's idea of a request's length differs from the host's, a correction goes up
        self.slots.set_lengths(slots, starts)
        self._fill_corrections(layout, host, fed=0)
        self._upload(layout, staging)
        self.slots.device_advanced(slots, counts)

        def host_batch():
            order, short = layout_order(counts, LONG)
            batch = arrange_step(order, short, counts, np.concatenate([entries[source].tokens for source in order]),
                                 slots[order], starts[order], wants, pad=pad, pad_short=self.PAD_SHORT,
                                 pad_long=self.PAD_LONG, scratch_slot=cache.scratch_slot)
            as32 = lambda values: np.asarray(values, dtype=np.int32)
            return HostBatch(as32(batch.token_ids), as32(batch.positions), as32(batch.token_item),
                             as32(batch.item_slot), as32(batch.q_start), as32(batch.kv_len),
                             as32(batch.logit_rows), [requests[source] for source in order])

        ctx = StepContext(layout, self._device_buffer, host_batch, cache, self._status, max_q_len, max_kv_len,
                          num_short_items, num_short_tokens, num_long_blocks, views=views)
        ctx.real_logit_rows = real_rows
        return ctx

    def _fill(self, layout: BatchLayout, host: np.ndarray, item_slot, q_start, logit_rows, token_ids, fed: int):
        """Write the uploaded part of a step into its staging buffer; the queued corrections of the slot store
        go along (or, if there are more than the shape has room for, the whole store is copied first)."""
        I = layout.num_items
        host[layout.item_slot:layout.item_slot + I] = item_slot
        host[layout.q_start:layout.q_start + I + 1] = q_start
        host[layout.logit_rows:layout.logit_rows + len(logit_rows)] = logit_rows
        if token_ids is not None:
            host[layout.token_ids:layout.token_ids + layout.num_tokens] = token_ids
        self._fill_corrections(layout, host, fed)

    def _fill_corrections(self, layout: BatchLayout, host: np.ndarray, fed: int):
        """The header and the queued corrections of the slot store into the staging buffer (if more wait than
        the shape has room for, the whole store is copied first)."""
        if self._needs_resync or self.slots.pending > layout.update_capacity:
            self._resync()
        offsets, values = self.slots.drain()
        count = len(offsets)
        if count > layout.update_capacity:                # cannot happen: pending bounds the drained count
            raise StepError("more slot corrections than the step has room for")
        pairs = host[layout.updates:layout.updates + 2 * count].reshape(count, 2)
        pairs[:, 0] = offsets
        pairs[:, 1] = values
        header = host[layout.header:layout.header + layout.HEADER_WORDS]
        header[layout.COUNTER] = 0
        header[layout.FED] = fed
        header[layout.NUM_UPDATES] = count
        header[3] = 0
        self._drained = offsets

    def _resync(self) -> None:
        """Copy the whole slot store to the device: after a failed step (what the device applied is unknown),
        or when more corrections wait than a step carries. The lengths are the host's."""
        cache, slots = self.cache, self.slots
        slots.mirror[slots.len:slots.len + cache.max_slots] = cache.lengths
        words = slots.take_all()
        if self._resync_pinned is None:
            self._resync_pinned = torch.empty(slots.size, dtype=torch.int32).pin_memory()
        self._resync_pinned.numpy()[:] = words
        self.ops.copy_h2d(slots.store, self._resync_pinned.data_ptr(), slots.size * 4)
        torch.cuda.current_stream().synchronize()         # the pinned copy may be overwritten by the next one
        self._needs_resync = False

    def _stage(self, T: int, I: int, R: int):
        """The layout of a step shape, its device views, and the pinned staging buffer of this turn."""
        shape = self._shapes.get((T, I, R))
        if shape is None:
            layout = self._layout(T, I, R)
            self._grow(layout.total)
            if len(self._shapes) >= 1024:
                self._shapes.clear()
            shape = self._shapes[(T, I, R)] = (layout, DeviceViews(layout, self._device_buffer))
        layout, views = shape
        turn = self._turn
        self._turn = (turn + 1) % self.STAGING_BUFFERS
        self._staging_events[turn].synchronize()      # the copy that last read this buffer is done
        self._staging_turn = turn
        return layout, views, self._staging[turn], self._staging_numpy[turn]

    def _upload(self, layout: BatchLayout, staging: torch.Tensor, record: bool = True,
                with_tokens: bool = True) -> None:
        """The step's one host-to-device copy: header, slots, item starts, wanted rows and corrections, and
        the token ids unless the device has fed them back itself (``with_tokens=False``).  ``record=False``:
        the caller synchronises the stream before it returns, so the staging buffer needs no event."""
        if with_tokens:
            words = layout.token_ids + layout.num_tokens
        else:
            count = int(self._staging_numpy[self._staging_turn][layout.header + layout.NUM_UPDATES])
            words = layout.updates + 2 * count
        self.ops.copy_h2d(self._device_buffer, self._staging_ptr[self._staging_turn], words * 4)
        if record:
            self._staging_events[self._staging_turn].record()
        self.h2d_bytes = words * 4
        self._drained = None                               # the corrections are on their way

    def _prepare_single_tokens(self, requests, tokens, extra_tokens: int, sampling) -> StepContext:
        """``prepare`` for a step in which every request brings one token and wants its logits: the same
        buffer contents, filled with whole-array operations instead of a loop over entries.  ``extra_tokens``
        more positions per request get pages too (a run of several decode steps on the device);
        ``sampling`` = (temperatures, seeds) per request is uploaded with the batch.
        ``tokens=None`` stages everything but the token ids and uploads nothing (see ``_stage_ahead``)."""
        cache = self.cache
        I = len(requests)
        if I == 0:
            raise StepError("a step cannot be empty")
        slot_of = cache.slot_of
        try:
            slots = np.fromiter((slot_of[request] for request in requests), dtype=np.int64, count=I)
        except KeyError as missing:
            raise StepError(f"request {missing.args[0]!r} has no prompt in the cache") from None
        if I > 1 and np.unique(slots).size != I:
            raise StepError("a request can appear only once in a step")
        if tokens is not None:
            self._check_vocabulary(tokens)
        starts = cache.lengths[slots]
        if int(starts.max()) + 1 + extra_tokens > self.max_model_len:
            raise StepError(f"a request would pass the model's maximum length {self.max_model_len}")
        cache.extend_many(requests, np.full(I, 1 + extra_tokens, dtype=np.int64))      # all or nothing
        self._admitted_in_step = []

        # The step runs P >= I entries: the I requests, then entries of one token each at position 0 of the
        # cache's scratch slot (their results are dropped), so that batch sizes share captured graphs.
        P = self._decode_bucket(I)
        layout, views, staging, host = self._stage(P, P, P)
        slots_store = self.slots
        slots_store.set_lengths(slots, starts)
        if sampling is not None:
            slots_store.set_sampling(slots, sampling[0], sampling[1])
        ramp = self._ramp[:P + 1]
        item_slot, kv_len, positions = slots, starts + 1, starts
        token_ids = np.asarray(tokens, dtype=np.int32) if tokens is not None else np.zeros(I, dtype=np.int32)
        if P > I:
            item_slot = np.concatenate([slots, np.full(P - I, cache.scratch_slot, dtype=slots.dtype)])
            kv_len = np.concatenate([kv_len, np.ones(P - I, dtype=kv_len.dtype)])
            positions = np.concatenate([positions, np.zeros(P - I, dtype=positions.dtype)])
            token_ids = np.concatenate([token_ids, np.zeros(P - I, dtype=np.int32)])
        self._fill(layout, host, item_slot, ramp, ramp[:P], token_ids if tokens is not None else None,
                   fed=0 if tokens is not None else 1)
        if tokens is not None:
            self._upload(layout, staging, record=False)
            slots_store.device_advanced(slots, 1 + extra_tokens)
        host_batch = HostBatch(token_ids, positions.astype(np.int32), ramp[:P], item_slot.astype(np.int32), ramp,
                               kv_len.astype(np.int32), ramp[:P], list(requests))
        ctx = StepContext(layout, self._device_buffer, host_batch, cache, self._status, 1,
                          int(kv_len.max()), P, P, 0, views=views)
        ctx.slots = slots
        ctx.real_items = I
        ctx.drained = self._drained                        # corrections staged but not yet uploaded
        return ctx

    def _decode_bucket(self, count: int) -> int:
        """The number of entries a decode-only step of ``count`` requests runs with."""
        if not self._pad_decode:
            return count
        bucket = next((small for small in (1, 2, 4, 8) if count <= small), -(-count // 8) * 8)
        return bucket if bucket <= self.cache.max_slots else count      # buffers are sized for max_slots entries

    def _check_vocabulary(self, tokens: np.ndarray) -> None:
        low, high = int(tokens.min()), int(tokens.max())
        if low < 0 or high >= self.vocab_size:
            raise StepError(f"token id {low if low < 0 else high} is outside the vocabulary of "
                            f"{self.vocab_size}")

    # A decode step is followed, most of the time, by a decode step of the same requests.  While the device
    # runs step n the host therefore stages step n+1 (pages, positions, tables: everything but the token ids,
    # which step n has yet to produce).  Step n's last kernel feeds its tokens back on the device, so where the
    # step is a captured graph, step n+1 is also launched right behind it: its buffer goes up without the token
    # section and the graph is replayed before the host has seen step n's tokens.  The device then never waits
    # for the host between the two.  If the next call brings the same requests (and, for a launched step, the
    # tokens that step n sampled), the step is used: only its tokens are written and the buffer goes up, or it
    # is simply waited for.  If anything else is called first, the step is undone: its pages go back, and what
    # a launched step computes is ignored (everything later is ordered behind it in the stream).
    def _stage_ahead(self, requests, temperatures, seeds, launch_half=None):
        try:
            ctx = self._prepare_single_tokens(requests, None, 0, (temperatures, seeds))
        except (StepError, CacheFull):
            return None                       # no room or no length left: the real call will say so
        staged = _StagedStep(list(requests), list(temperatures), list(seeds), ctx, self._staging_turn)
        graph = self._graphs.get((ctx.num_items, "sample")) if launch_half is not None else None
        if graph is not None and not self.cache.state:
            # (a step that is launched and then dropped leaves its pages unread, but state of fixed size in
            # the slots would have been moved on by it: models with such state are never launched ahead)
            layout = ctx.layout
            # the step's tokens go to the half of the history that the step before it does not use
            self._staging_numpy[staged.turn][layout.counter] = launch_half
            self._upload(layout, self._staging[staged.turn], record=True, with_tokens=False)
            self.slots.device_advanced(ctx.slots, 1)
            ctx.drained = None
            graph.replay()
            self.graph_replays += 1
            staged.event = self._step_events[launch_half]
            staged.event.record()
            staged.half = launch_half
            staged.launched = True
        return staged

    def _drop_staged(self) -> None:
        staged, self._staged = self._staged, None
        if staged is not None:
            if staged.ctx.drained is not None:             # its corrections never went up: queue them again
                self.slots.requeue(staged.ctx.drained)
            for request in staged.requests:
                self.cache.rollback(request)

    def _abandon(self, entries) -> None:
        for entry in entries:
            self.cache.rollback(entry.request)
        for request in self._admitted_in_step:
            self.cache.free(request)
        self._needs_resync = True                           # how far the device got with the step is unknown

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one step; returns float32 logits ``[R, V]`` (R may be 0)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        decode_only = all(len(entry.tokens) == 1 and entry.want == [0] for entry in entries)
        ctx = self.prepare(entries, pad=self._pad_mixed and not decode_only)
        try:
            if decode_only and self.enable_cuda_graphs:
                logits = self._run_decode_graph(ctx, "logits").logits.clone()
            elif self.enable_cuda_graphs:
                logits = self._run_mixed_step(ctx).clone()     # out of the step arena (or the graph's buffer)
            else:
                logits = self._forward(ctx).clone()
        except Exception:
            self._abandon(entries)
            raise
        self.cache.commit_many([entry.request for entry in entries])
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        expected = sum(len(entry.want) for entry in entries)
        if logits.shape[0] != expected:
            # reference: src/scheduler/orca_scheduler.py:260-263, 281-286
            raise StepError(f"model returned {logits.shape[0]} logits rows, expected {expected}")
        return logits

    # ------------------------------------------------------------------ decode-only steps
    def decode(self, entries: Sequence[StepEntry], temperatures, seeds, steps: int = 1) -> np.ndarray:
        """``decode_tokens`` for entries of one token each."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries or any(len(entry.tokens) != 1 for entry in entries):
            raise StepError("decode takes exactly one token per request")
        return self.decode_tokens([entry.request for entry in entries],
                                  [int(entry.tokens[0]) for entry in entries], temperatures, seeds, steps)

    def decode_tokens(self, requests: Sequence[Hashable], tokens: Sequence[int], temperatures, seeds,
                      steps: int = 1, stage_next: bool = False) -> np.ndarray:
        """Run ``steps`` decode steps of a batch of single tokens without the host in between.

        ``tokens[i]`` is the one next token of ``requests[i]``, whose earlier tokens are in the cache.
        Each step samples on the device (greedy or temperature), feeds the token back as the next
        input and moves the request one position on.  Returns the sampled tokens ``[steps, B]``.
        The step is replayed as a CUDA graph (reference: decode-only fast path with CUDA graphs,
        src/model/paged_decoder.py:385-496) unless graphs are disabled.
        ``stage_next``: the caller expects to come back with the same requests for one more step; the host
        side of that step is prepared while the device runs this one.
        """
        tokens = np.asarray(tokens)
        if tokens.ndim != 1 or tokens.size != len(requests) or tokens.size == 0:
            raise StepError("decode takes exactly one token per request")
        if not np.issubdtype(tokens.dtype, np.integer):
            raise StepError("token ids must be integers")
        if not (1 <= steps <= self.MAX_DEVICE_STEPS):
            raise StepError(f"steps must be between 1 and {self.MAX_DEVICE_STEPS}")
        staged, self._staged = self._staged, None
        ahead = None                                        # this very step, if it was launched ahead
        if (staged is not None and steps == 1 and staged.requests == list(requests)
                and staged.temperatures == list(temperatures) and staged.seeds == list(seeds)
                and (not staged.launched or np.array_equal(staged.fed_tokens, tokens))):
            ctx = staged.ctx
            if staged.launched:
                ahead = staged
            else:
                self._check_vocabulary(tokens)
                layout = ctx.layout
                host = self._staging_numpy[staged.turn]
                host[layout.token_ids:layout.token_ids + tokens.size] = tokens
                host[layout.token_ids + tokens.size:layout.token_ids + layout.num_tokens] = 0
                host[layout.header + layout.FED] = 0
                ctx.host.token_ids[:tokens.size] = tokens
                self._staging_turn = staged.turn
                self._upload(layout, self._staging[staged.turn], record=False)
                self.slots.device_advanced(ctx.slots, 1)
                ctx.drained = None
        else:
            if staged is not None:
                self._staged = staged
                self._drop_staged()
            ctx = self._prepare_single_tokens(requests, tokens, steps - 1, (temperatures, seeds))
        B = ctx.num_items
        half, done = 0, None
        if ahead is not None:
            half, done = ahead.half, ahead.event
        else:
            try:
                if self.enable_cuda_graphs:
                    graph = self._run_decode_graph(ctx, "sample")
                    for _ in range(steps - 1):
                        graph.replay()
                        self.graph_replays += 1
                else:
                    # the positions move on the device: the bound that fixes the attention grid must cover
                    # the last step's context, not only the first one's
                    ctx.max_kv_len = min(self.max_model_len, ctx.max_kv_len + steps - 1)
                    for _ in range(steps):
                        self._forward_and_sample(ctx)
            except Exception:
                for request in requests:
                    self.cache.rollback(request)
                self._needs_resync = True
                raise
            if stage_next and steps == 1 and self.enable_cuda_graphs:
                done = self._step_events[0]
                done.record()
        # the step is on its way: what follows runs on the host while the device works
        self.cache.commit_many(requests)
        self.steps += steps
        self.tokens_run += steps * len(requests)
        if stage_next and steps == 1:
            self._staged = self._stage_ahead(requests, temperatures, seeds,
                                             launch_half=None if done is None else 1 - half)
        if done is not None:
            done.synchronize()                             # this step's tokens are in host memory now
        else:
            torch.cuda.current_stream().synchronize()
        if self._history.array[self._status_index]:
            self.check_status()
        # (B entries ran, the requests first; what the padding entries drew is dropped)
        result = self._history.array[half * B:(half + steps) * B].reshape(steps, B)[:, :len(requests)].copy()
        if self._staged is not None and self._staged.launched:
            self._staged.fed_tokens = result[0]
        return result

    def begin(self, ctx: StepContext) -> None:
        """The step's first kernel: apply the uploaded corrections to the slot store and derive the per-step
        arrays (positions, token -> item and slot, lengths after the step, sampling parameters) from it."""
        self.ops.step_begin(self.slots, ctx.layout, ctx.views.meta, self._status)

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        """The step's launches. Its intermediate tensors (and the logits it returns) come from the step arena
        and hold until the next call: whoever keeps the logits longer copies them."""
        self.ops.arena.reset()
        self.begin(ctx)
        return self.model.forward(ctx)

    def _forward_and_sample(self, ctx: StepContext) -> torch.Tensor:
        logits = self._forward(ctx)
        B = ctx.num_items
        sampled = self._sampled[:B]
        # the token drawn now will sit at position (input position + 1)
        self.ops.sample(logits, ctx.temperature, ctx.seed, ctx.positions, sampled, pos_offset=1)
        self.ops.step_end(self.slots, ctx.layout, ctx.views.meta, sampled, self._history, self.MAX_DEVICE_STEPS,
                          status=self._status, status_index=self._status_index)
        return logits

    def _run_mixed_step(self, ctx: StepContext) -> torch.Tensor:
        """A step with prompt portions.  Its ~100 launches cost the host about as much time as the device
        needs to run them, so a step shape that comes back (same counts of tokens, entries, wanted rows,
        short entries and query blocks: a steady chunked-prefill budget, a benchmark) is captured as a CUDA
        graph once it has been seen ``MIXED_SHAPE_SIGHTINGS`` times and replayed from then on."""
        bucket = -(-ctx.max_kv_len // 256) * 256
        ctx.max_kv_len = min(bucket, self.max_model_len)
        key = (ctx.num_tokens, ctx.num_items, ctx.num_logit_rows, ctx.num_short_items, ctx.num_short_tokens,
               ctx.num_long_blocks, ctx.max_kv_len, "mixed")
        rows = ctx.real_logit_rows                   # the rest are padding
        graph = self._graphs.get(key)
        if graph is not None:
            graph.replay()
            self.graph_replays += 1
            return graph.logits[:rows]
        seen = self._shape_seen.get(key, 0) + 1
        self._shape_seen[key] = seen
        logits = self._forward(ctx)[:rows]
        if seen < self.MIXED_SHAPE_SIGHTINGS:
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            return logits
        if len(self._graphs) >= self.MAX_GRAPHS:
            self._graphs.pop(next(iter(self._graphs)))
        launches_before = self.ops.launches
        captured, static_logits = self._capture(lambda: self._forward(ctx))
        self._graphs[key] = _DecodeGraph(captured, static_logits, self.ops.launches - launches_before)
        return logits

    def _capture(self, run):
        """Capture the launches of ``run()`` as a CUDA graph: on a side stream, into the pool that all graphs
        of this runner share. (``torch.cuda.graph`` would also synchronise the device, collect garbage and
        empty the allocator's cache, about 15 ms and a slow restart of every eager step after it.)"""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        side, main = self._capture_stream, torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool)
            try:
                result = run()
            finally:
                graph.capture_end()
        main.wait_stream(side)
        return graph, result

    def _run_decode_graph(self, ctx: StepContext, kind: str):
        """Run the decode-only step ``ctx`` once: eagerly the first time a batch size is seen
        (then capture it), by graph replay afterwards."""
        ctx.max_kv_len = self.max_model_len          # the graph's grid must cover any context
        key = (ctx.num_items, kind)
        graph = self._graphs.get(key)
        if graph is not None:
            graph.replay()
            self.graph_replays += 1
            return graph
        if len(self._graphs) >= self.MAX_GRAPHS:
            self._graphs.pop(next(iter(self._graphs)))
        # warm-up run (this is the step's real execution), then capture for the next time
        if kind == "sample":
            self._forward_and_sample(ctx)
        else:
            warm = self._forward(ctx)
        launches_before = self.ops.launches
        captured, logits = self._capture(
            lambda: self._forward_and_sample(ctx) if kind == "sample" else self._forward(ctx))
        graph = _DecodeGraph(captured, logits, self.ops.launches - launches_before)
        self._graphs[key] = graph
        if kind == "logits":
            logits.copy_(warm)                       # this call's result
        return graph

    def finish(self, request: Hashable) -> None:
        """The request is done: its pages and its slot are given back."""
        self._drop_staged()
        self.cache.free(request)

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input or a wait that ran out (reads one int from the device).
        Decode steps that sample on the device bring the flag along with their tokens and check it
        themselves; after other steps the caller decides when the read is worth a synchronisation."""
        flag = int(self._status.item())
        if flag:
            self._status.zero_()
            self._history.array[self._status_index] = 0
            self.ops.reset_after_fault()
            self._needs_resync = True
            raise StepError(f"a kernel reported bad input or gave up waiting (status {flag})")
