"""Engine-level settings: everything that is not part of the model itself.

Counterpart of the arguments of the reference's ``build_scheduler``
(reference: main.py:136-150) with the backend switch and INT8 cache removed.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from pagedserve_b200.config.registry import ConfigError

SUPPORTED_DTYPES = ("float32", "bfloat16")
ORCA_STRATEGY = "orca"
SARATHI_STRATEGY = "sarathi"
SUPPORTED_SCHEDULING_STRATEGIES = (ORCA_STRATEGY, SARATHI_STRATEGY)


@dataclass
class EngineConfig:
    dtype: str = "float32"                      # reference default: main.py:299-304
    block_size: int = 16                        # tokens per KV page (reference: main.py:215)
    num_blocks: Optional[int] = None            # pages in the pool; None => from kv_cache_memory_mb
    kv_cache_memory_mb: Optional[int] = None    # reference: main.py:283-287
    kv_cache_memory_utilization: float = 0.90   # reference: main.py:288-293; used when neither is given
    kv_cache_safety_mb: int = 3072              # reference: main.py:294-298
    max_num_seqs: int = 32                      # live requests (reference --max-batch-size, main.py:151)
    max_num_batched_tokens: int = 2048          # token budget of one step
    strategy: str = ORCA_STRATEGY               # reference: main.py:265-270
    prefill_chunk_size: int = 16                # reference: main.py:271-276
    enable_cuda_graphs: bool = True             # reference: --disable-cuda-graphs, main.py:317-321
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype not in SUPPORTED_DTYPES:
            raise ConfigError(f"unknown dtype {self.dtype!r}; choose one of {SUPPORTED_DTYPES}")
        if self.block_size <= 0 or self.block_size > 64 or (self.block_size & (self.block_size - 1)):
            raise ConfigError("block_size must be a power of two between 1 and 64")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ConfigError("num_blocks must be positive")
        if self.kv_cache_memory_mb is not None and self.kv_cache_memory_mb <= 0:
            raise ConfigError("kv_cache_memory_mb must be positive")   # reference: main.py:209-210
        if not 0 < self.kv_cache_memory_utilization <= 1:
            raise ConfigError("kv_cache_memory_utilization must be in (0, 1]")   # reference: main.py:55-56
        if self.kv_cache_safety_mb < 0:
            raise ConfigError("kv_cache_safety_mb cannot be negative")           # reference: main.py:57-58
        if self.max_num_seqs <= 0:
            raise ConfigError("max_num_seqs must be positive")         # reference: main.py:183-184
        if self.max_num_batched_tokens <= 0:
            raise ConfigError("max_num_batched_tokens must be positive")
        if self.strategy not in SUPPORTED_SCHEDULING_STRATEGIES:
            raise ConfigError(
                f"unknown scheduling strategy {self.strategy!r}; choose one of "
                f"{SUPPORTED_SCHEDULING_STRATEGIES}"
            )
        if self.prefill_chunk_size <= 0:
            raise ConfigError("prefill_chunk_size must be positive")   # reference: orca_scheduler.py:51-52
