"""How many pages the cache pool gets when nobody says so.

reference: main.py:48-73 (``calculate_cuda_kv_cache_budget``): the pool may grow until the
device as a whole is ``memory_utilization`` full, and must leave ``safety_memory`` of what is
free now untouched; the smaller of the two is the budget.  The reference hands the whole
budget to its pool.  Here the pool is also capped by what the live requests can ever hold
(``max_num_seqs`` contexts of full length): pages beyond that could never be used.
"""

from __future__ import annotations

MIB = 1024 * 1024
DEFAULT_KV_MEMORY_UTILIZATION = 0.90      # reference: main.py:30
DEFAULT_KV_SAFETY_MB = 3072               # reference: main.py:31


def kv_cache_budget(free_memory: int, total_memory: int,
                    memory_utilization: float = DEFAULT_KV_MEMORY_UTILIZATION,
                    safety_memory: int = DEFAULT_KV_SAFETY_MB * MIB) -> int:
    """Bytes the cache pool may take, from the device's free and total memory."""
    if not 0 < memory_utilization <= 1:
        raise ValueError("KV-cache memory utilization must be in (0, 1]")
    if safety_memory < 0:
        raise ValueError("KV-cache safety memory cannot be negative")
    if not 0 < free_memory <= total_memory:
        raise ValueError("device memory information is invalid")
    in_use = total_memory - free_memory
    budget = min(int(total_memory * memory_utilization) - in_use, free_memory - safety_memory)
    if budget <= 0:
        raise RuntimeError("no device memory remains for the KV cache after the utilization target "
                           "and the safety margin")
    return budget


def pages_for_budget(budget_bytes: int, bytes_per_page: int, max_num_seqs: int, max_model_len: int,
                     block_size: int) -> int:
    """Pages of ``bytes_per_page`` within ``budget_bytes``, no more than the live requests can hold."""
    if bytes_per_page <= 0:
        return 1
    affordable = budget_bytes // bytes_per_page
    if affordable == 0:
        # reference: src/model/kv_manager.py:61-64
        raise ValueError(f"Memory budget is too small; one block requires {bytes_per_page} bytes")
    useful = max_num_seqs * (-(-max_model_len // block_size))
    return max(1, min(useful, affordable))
