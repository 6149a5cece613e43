"""Turn float32 logits rows into token ids on the device.

The reference samples with ``argmax`` only and then reads the ids on the host
(reference: src/scheduler/orca_scheduler.py:250).  ``temperature == 0`` keeps
that rule (lowest index on ties).  ``temperature > 0`` draws from
``softmax(logits / T)`` by the Gumbel-max rule with noise from a counter-based
generator keyed by (seed, position in the sequence, vocabulary index), so a
request's tokens do not depend on what else is in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch


@dataclass
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature cannot be negative")


class Sampler:
    def __init__(self, ops, device, max_rows: int = 1024):
        self.ops = ops
        self.device = torch.device(device)
        self._capacity = 0
        self._ensure(max_rows)

    def _ensure(self, rows: int) -> None:
        if rows <= self._capacity:
            return
        self._capacity = max(rows, 2 * self._capacity)
        n = self._capacity
        # one pinned staging area: temperature f32 | position i32 | seed i64, as raw int32 words
        self._host = torch.empty(4 * n, dtype=torch.int32).pin_memory()
        self._dev = torch.empty(4 * n, dtype=torch.int32, device=self.device)
        self._out = torch.empty(n, dtype=torch.int32, device=self.device)
        self._out_host = torch.empty(n, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], seeds: Sequence[int],
               positions: Sequence[int]) -> List[int]:
        """One token per logits row; reads the ids back to the host."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        if not (len(temperatures) == len(seeds) == len(positions) == rows):
            raise ValueError("sampling parameters must match the number of logits rows")
        self._ensure(rows)
        n = self._capacity
        host = self._host.numpy()
        greedy = all(t == 0 for t in temperatures)
        if greedy:
            self.ops.sample(logits, None, None, None, self._out[:rows])
        else:
            host[:rows].view(np.float32)[:] = np.asarray(temperatures, dtype=np.float32)
            host[n:n + rows] = np.asarray(positions, dtype=np.int32)
            host[2 * n:2 * n + 2 * rows].view(np.uint64)[:] = np.asarray(
                [int(s) & 0xFFFFFFFFFFFFFFFF for s in seeds], dtype=np.uint64)
            self._dev.copy_(self._host, non_blocking=True)
            temperature = self._dev[:rows].view(torch.float32)
            position = self._dev[n:n + rows]
            seed = self._dev[2 * n:2 * n + 2 * rows].view(torch.int64)
            self.ops.sample(logits, temperature, seed, position, self._out[:rows])
        self._out_host[:rows].copy_(self._out[:rows], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:rows].tolist()
