"""Continuous batching above the step function.

After the reference's ``ContinuousBatchScheduler`` (src/scheduler/orca_scheduler.py):
three states (waiting = still prefilling, active = decoding, finished; :63-67),
iteration-level scheduling, admission by a worst-case page reservation so that a
running request can never run out of pages (:119-122, 138-142, 229-232), FCFS
order by request id, greedy finish rule (:268-277).

Strategies
----------
``orca``     every selected waiting request runs its whole remaining prompt in one step
             (:128-146); selection stops at the first request that does not fit.
``sarathi``  decodes first, then prompt portions of ``prefill_chunk_size`` tokens
             (:148-169, 182-186).  The reference runs one prefill portion per step;
             ``max_prefills_per_step`` (default 1) lifts that to several.

Both are cut by ``max_num_batched_tokens``, the token budget of one step, which the
reference does not have: a portion is never larger than what is left of the budget.

When pages run out: a request is not admitted while its reservation would not fit; it
waits in the queue, and running requests are never preempted.  A request that could
never fit even in an empty pool is refused when it is added.  If work remains and
nothing can be scheduled, ``step`` raises (reference: :223-225).
"""

from __future__ import annotations

import math
import numbers
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from pagedserve_b200.config.engine_config import (
    ORCA_STRATEGY,
    SUPPORTED_SCHEDULING_STRATEGIES,
)
from pagedserve_b200.engine.batch import StepEntry


@dataclass
class RequestState:
    """reference: src/scheduler/orca_scheduler.py:19-28"""

    request_id: int
    prompt_token_ids: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    generated_token_ids: List[int] = field(default_factory=list)
    pending_token_id: Optional[int] = None
    reserved_blocks: int = 0
    prefill_cursor: int = 0


class Scheduler:
    def __init__(self, engine, max_num_seqs: int = 32, max_num_batched_tokens: int = 2048,
                 strategy: str = ORCA_STRATEGY, prefill_chunk_size: int = 16,
                 eos_token_id: Optional[int] = None, max_prefills_per_step: int = 1):
        if max_num_seqs <= 0:
            raise ValueError("max_num_seqs must be positive")              # reference: :43-44
        if strategy not in SUPPORTED_SCHEDULING_STRATEGIES:
            choices = ", ".join(SUPPORTED_SCHEDULING_STRATEGIES)
            raise ValueError(f"Unknown scheduling strategy '{strategy}'. Choose one of: {choices}")
        if prefill_chunk_size <= 0:
            raise ValueError("prefill_chunk_size must be positive")        # reference: :51-52
        if max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        self.engine = engine
        self.max_num_seqs = min(max_num_seqs, engine.cache.max_slots)
        self.max_num_batched_tokens = max_num_batched_tokens
        self.strategy = strategy
        self.prefill_chunk_size = prefill_chunk_size
        self.max_prefills_per_step = max_prefills_per_step
        self.eos_token_id = eos_token_id
        self.block_size = engine.cache.page_size
        self.total_blocks = engine.cache.total_pages()

        self.waiting = deque()                        # requests with prompt tokens still to run
        self.active: Dict[int, RequestState] = {}     # requests that decode
        self.finished: Dict[int, RequestState] = {}
        self.next_request_id = 0
        self.reserved_blocks = 0                      # pages promised to admitted requests
        self.steps = 0

    # ------------------------------------------------------------------ submit
    def add_token_request(self, prompt_token_ids: Sequence[int], max_new_tokens: int = 200,
                          temperature: float = 0.0, seed: int = 0) -> int:
        """reference: ``add_token_request`` (src/scheduler/orca_scheduler.py:85-117)"""
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if hasattr(prompt_token_ids, "tolist"):
            prompt_token_ids = prompt_token_ids.reshape(-1).tolist()
        prompt = list(prompt_token_ids)
        if not prompt:
            raise ValueError("The prompt is empty")
        # any integer type counts (a slice of a token array gives numpy integers), booleans do not
        if any(not isinstance(token, numbers.Integral) or isinstance(token, bool) for token in prompt):
            raise ValueError("Prompt token IDs must be integers")
        prompt = [int(token) for token in prompt]
        if min(prompt) < 0 or max(prompt) >= self.engine.vocab_size:
            raise ValueError("A prompt token is outside the model vocabulary")
        if len(prompt) + max_new_tokens > self.engine.max_model_len:
            raise ValueError("Prompt plus requested generation exceeds the model context limit")
        if temperature < 0:
            raise ValueError("temperature cannot be negative")
        request = RequestState(self.next_request_id, prompt, max_new_tokens, float(temperature), int(seed))
        if self._required_blocks(request) > self.total_blocks:
            raise ValueError("The request can never fit: it needs "
                             f"{self._required_blocks(request)} KV blocks, the pool has {self.total_blocks}")
        self.next_request_id += 1
        self.waiting.append(request)
        return request.request_id

    add_request = add_token_request

    def _required_blocks(self, request: RequestState) -> int:
        """Worst case pages of a request (reference: :119-122).  The last generated token is never run, so
        only prompt + max_new_tokens - 1 positions are ever cached: at exact multiples of the page size this
        reserves one page more than is used.  Kept, so that admission decisions equal the reference's."""
        return math.ceil((len(request.prompt_token_ids) + request.max_new_tokens) / self.block_size)

    # ------------------------------------------------------------------ decisions
    def select(self) -> List[Tuple[RequestState, int]]:
        """Decide this step: (request, number of its tokens to run), decodes as 1.

        Pure bookkeeping: touches neither the engine nor the reservations."""
        budget = self.max_num_batched_tokens
        selected: List[Tuple[RequestState, int]] = []
        newly_reserved = 0

        def fits(request: RequestState) -> bool:
            nonlocal newly_reserved
            if request.reserved_blocks > 0:
                return True
            need = self._required_blocks(request)
            if self.reserved_blocks + newly_reserved + need > self.total_blocks:
                return False
            newly_reserved += need
            return True

        if self.strategy == ORCA_STRATEGY:
            pool = sorted(list(self.active.values()) + list(self.waiting), key=lambda r: r.request_id)
            for request in pool:
                if len(selected) == self.max_num_seqs or budget == 0:
                    break
                if not fits(request):
                    break                                   # head of line (reference: :138-142)
                if request.pending_token_id is not None:
                    count = 1
                else:
                    count = min(len(request.prompt_token_ids) - request.prefill_cursor, budget)
                selected.append((request, count))
                budget -= count
            return selected

        # sarathi: decodes first, oldest first
        for request in sorted(self.active.values(), key=lambda r: r.request_id):
            if len(selected) == self.max_num_seqs or budget == 0:
                break
            selected.append((request, 1))
            budget -= 1
        prefills = 0
        for request in self.waiting:
            if len(selected) == self.max_num_seqs or budget == 0:
                break
            if self.max_prefills_per_step and prefills == self.max_prefills_per_step:
                break
            if not fits(request):
                break
            count = min(self.prefill_chunk_size, len(request.prompt_token_ids) - request.prefill_cursor, budget)
            selected.append((request, count))
            budget -= count
            prefills += 1
        return selected

    # ------------------------------------------------------------------ one iteration
    def step(self) -> Dict[int, int]:
        """Run one step; returns {request id: token emitted in this step}."""
        selected = self.select()
        if not selected:
            if self.waiting or self.active:
                raise RuntimeError("No request can be scheduled with the available KV memory")
            return {}
        new_requests = [request for request, _ in selected if request.reserved_blocks == 0]
        for request in new_requests:
            request.reserved_blocks = self._required_blocks(request)
            self.reserved_blocks += request.reserved_blocks

        decode_only = all(request.pending_token_id is not None for request, _ in selected)
        fused_decode = getattr(self.engine, "decode_tokens", None) if decode_only else None
        entries = []
        sampling = []        # requests whose next token is drawn in this step
        if fused_decode is not None:
            sampling = [request for request, _ in selected]
        else:
            for request, count in selected:
                if request.pending_token_id is not None:
                    tokens = [request.pending_token_id]
                    want = [0]
                else:
                    start = request.prefill_cursor
                    tokens = request.prompt_token_ids[start:start + count]
                    last = start + count == len(request.prompt_token_ids)
                    want = [count - 1] if last else []           # reference: :191
                if want:
                    sampling.append(request)
                entries.append(StepEntry(request.request_id, tokens, want))
        try:
            if fused_decode is not None:
                # every request brings one decoded token: forward and sampling run as one device step
                # the same batch comes back next step unless a request reaches its limit now (an end-of-
                # sequence token cannot be foreseen: then what was staged ahead is simply dropped)
                # (waiting requests cannot join while every sequence slot is taken)
                comes_back = (not self.waiting or len(sampling) >= self.max_num_seqs) and all(
                    len(request.generated_token_ids) + 1 < request.max_new_tokens for request in sampling)
                tokens = fused_decode(
                    [request.request_id for request in sampling],
                    [request.pending_token_id for request in sampling],
                    [request.temperature for request in sampling],
                    [request.seed for request in sampling],
                    1, comes_back,
                )[0].tolist()
            else:
                logits = self.engine.step(entries)
        except Exception:
            for request in new_requests:                      # reference: :243-247
                self.reserved_blocks -= request.reserved_blocks
                request.reserved_blocks = 0
            raise
        if fused_decode is None:
            if logits.shape[0] != len(sampling):
                raise RuntimeError("Model returned the wrong number of logits rows")   # reference: :260-263
            tokens = self.engine.sample(
                logits,
                [request.temperature for request in sampling],
                [request.seed for request in sampling],
                [len(request.prompt_token_ids) + len(request.generated_token_ids) for request in sampling],
            )
        emitted: Dict[int, int] = {}
        completed_prefill = set()
        produced = iter(tokens)
        for request, count in selected:
            if request.pending_token_id is None:
                request.prefill_cursor += count
                if request.prefill_cursor < len(request.prompt_token_ids):
                    continue
                completed_prefill.add(request.request_id)
            token = int(next(produced))
            request.generated_token_ids.append(token)
            request.pending_token_id = token
            emitted[request.request_id] = token
            done = len(request.generated_token_ids) >= request.max_new_tokens
            if self.eos_token_id is not None and token == self.eos_token_id:
                done = True
            if done:
                self.active.pop(request.request_id, None)
                self.engine.finish(request.request_id)
                self.reserved_blocks -= request.reserved_blocks
                request.reserved_blocks = 0
                self.finished[request.request_id] = request
            else:
                self.active[request.request_id] = request
        if completed_prefill:
            self.waiting = deque(r for r in self.waiting if r.request_id not in completed_prefill)
        self.steps += 1
        return emitted

    def abort(self, request_id: int) -> List[int]:
        """Take a request out before it is done: what it holds (pages, slot, reservation) is given back
        and it counts as finished with the tokens it has so far, which are returned.  Between steps only."""
        request = self.active.pop(request_id, None)
        if request is None:
            for candidate in self.waiting:
                if candidate.request_id == request_id:
                    request = candidate
                    break
            if request is None:
                raise KeyError(f"request {request_id} is not waiting or running")
            self.waiting.remove(request)
        if request.reserved_blocks:
            # admitted: it has run at least one step, so the cache knows it
            self.engine.finish(request.request_id)
            self.reserved_blocks -= request.reserved_blocks
            request.reserved_blocks = 0
        request.pending_token_id = None
        self.finished[request.request_id] = request
        return list(request.generated_token_ids)

    def run_until_complete(self) -> Dict[int, List[int]]:
        """reference: src/scheduler/orca_scheduler.py:297-303 (token ids instead of decoded text)"""
        while self.waiting or self.active:
            self.step()
        check = getattr(self.engine, "check_status", None)
        if check is not None:
            check()                   # a kernel that flagged something in a step without device sampling
        return {request_id: list(request.generated_token_ids) for request_id, request in self.finished.items()}

    run = run_until_complete
