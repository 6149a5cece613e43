"""Command line and ``build_scheduler`` in the manner of the reference's main.py.

reference: main.py:136-254 (``build_scheduler``) and :257-342 (``main``).  Options
keep the reference's names and meanings where it has them (``--model``,
``--strategy``, ``--prefill-chunk-size``, ``--max-batch-size``,
``--kv-cache-memory-mb``, ``--kv-cache-memory-utilization``, ``--kv-cache-safety-mb``,
``--dtype``, ``--decode-attention-backend``, ``--kv-cache-dtype``, ``--disable-cuda-graphs``).  ``--model`` is a
folder with ``config.json`` and ``model.safetensors``, or the name of a size
(``tiny-a``, ``tiny-b``, ``gpt2-124m``, ``gpt2-345m``, ``gpt2-1.5b``) to be filled with
seeded random weights.  ``--decode-attention-backend`` names the implementation of
single-token attention as in the reference (main.py:305-310); this engine has one, its
own paged kernels (``cuda``), and says so when it is asked for ``torch`` or ``triton``.
``--kv-cache-dtype`` is ``model`` (main.py:311-316); ``int8`` is refused: quantised
caches are not built.  Prompts are token ids: there is no tokenizer in the engine.
"""

from __future__ import annotations

import argparse
import os
import sys
from typing import Optional

from pagedserve_b200.cache.budget import DEFAULT_KV_MEMORY_UTILIZATION, DEFAULT_KV_SAFETY_MB
from pagedserve_b200.config.engine_config import (
    EngineConfig,
    ORCA_STRATEGY,
    SUPPORTED_DTYPES,
    SUPPORTED_SCHEDULING_STRATEGIES,
)

# reference: main.py:27-28. "cuda" is this engine's only implementation; the reference's two names are accepted
# and answered with a note, so that its command lines keep working.
SUPPORTED_DECODE_ATTENTION_BACKENDS = ("cuda", "torch", "triton")
SUPPORTED_KV_CACHE_DTYPES = ("model", "int8")


def build_engine(model: str, seed: int = 0, **engine_options):
    from pagedserve_b200.config.gpt2 import NAMED_CONFIGS, named_config
    from pagedserve_b200.engine.engine import Engine

    config = EngineConfig(**engine_options)
    if os.path.isdir(model):
        return Engine.from_folder(model, config)
    if model in NAMED_CONFIGS:
        return Engine.random(named_config(model), seed, config)
    raise ValueError(f"--model must be a model folder or one of {sorted(NAMED_CONFIGS)}; got {model!r}")


def build_scheduler(model: str = "tiny-a", scheduling_strategy: str = ORCA_STRATEGY, prefill_chunk_size: int = 16,
                    max_batch_size: Optional[int] = None, kv_cache_memory_mb: Optional[int] = None,
                    kv_cache_memory_utilization: float = DEFAULT_KV_MEMORY_UTILIZATION,
                    kv_cache_safety_mb: int = DEFAULT_KV_SAFETY_MB,
                    execution_dtype: str = "float32", enable_cuda_graphs: bool = True, block_size: int = 16,
                    num_blocks: Optional[int] = None, max_num_batched_tokens: int = 2048, seed: int = 0,
                    eos_token_id: Optional[int] = None, decode_attention_backend: str = "cuda",
                    kv_cache_dtype: str = "model"):
    """reference: ``build_scheduler`` (main.py:136-254); returns a ready ``Scheduler``."""
    if decode_attention_backend not in SUPPORTED_DECODE_ATTENTION_BACKENDS:      # reference: main.py:152-157
        raise ValueError(f"Unknown decode attention backend '{decode_attention_backend}'. "
                         f"Choose one of: {', '.join(SUPPORTED_DECODE_ATTENTION_BACKENDS)}")
    if decode_attention_backend != "cuda":
        print(f"note: decode attention backend '{decode_attention_backend}' is the reference's; this engine runs "
              "its own paged CUDA kernels for every step", file=sys.stderr)
    if kv_cache_dtype not in SUPPORTED_KV_CACHE_DTYPES:                          # reference: main.py:165-167
        raise ValueError(f"Unknown KV cache dtype '{kv_cache_dtype}'. "
                         f"Choose one of: {', '.join(SUPPORTED_KV_CACHE_DTYPES)}")
    if kv_cache_dtype != "model":
        raise ValueError("KV cache dtype 'int8' is not built: the cache is kept in the execution dtype")
    if max_batch_size is None:
        max_batch_size = 32                                  # reference: main.py:181-182 (CUDA default)
    if max_batch_size <= 0:
        raise ValueError("max_batch_size must be positive")
    engine = build_engine(model, seed=seed, dtype=execution_dtype, block_size=block_size, num_blocks=num_blocks,
                          kv_cache_memory_mb=kv_cache_memory_mb,
                          kv_cache_memory_utilization=kv_cache_memory_utilization,
                          kv_cache_safety_mb=kv_cache_safety_mb, max_num_seqs=max_batch_size,
                          max_num_batched_tokens=max_num_batched_tokens, strategy=scheduling_strategy,
                          prefill_chunk_size=prefill_chunk_size, enable_cuda_graphs=enable_cuda_graphs)
    return engine.make_scheduler(eos_token_id=eos_token_id)


def _parse_ids(text: str):
    return [int(part) for part in text.replace(",", " ").split()]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Run the pagedserve_b200 inference engine")
    parser.add_argument("--model", default="tiny-a", help="model folder, or a named size with random weights")
    parser.add_argument("--strategy", choices=SUPPORTED_SCHEDULING_STRATEGIES, default=ORCA_STRATEGY,
                        help="request scheduling strategy")
    parser.add_argument("--prefill-chunk-size", type=int, default=16,
                        help="prompt tokens per Sarathi prefill chunk")
    parser.add_argument("--max-batch-size", type=int, help="maximum requests per iteration (default: 32)")
    parser.add_argument("--max-num-batched-tokens", type=int, default=2048, help="token budget of one step")
    parser.add_argument("--kv-cache-memory-mb", type=int, help="explicit KV-cache budget in MiB")
    parser.add_argument("--kv-cache-memory-utilization", type=float, default=DEFAULT_KV_MEMORY_UTILIZATION,
                        help="target total GPU memory utilization for automatic KV sizing")
    parser.add_argument("--kv-cache-safety-mb", type=int, default=DEFAULT_KV_SAFETY_MB,
                        help="device memory left free for activations and temporary buffers")
    parser.add_argument("--num-blocks", type=int, help="explicit number of KV pages")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per KV page")
    parser.add_argument("--dtype", choices=SUPPORTED_DTYPES, default="float32", help="execution dtype")
    parser.add_argument("--decode-attention-backend", choices=SUPPORTED_DECODE_ATTENTION_BACKENDS, default="cuda",
                        help="single-token decode attention implementation (this engine has one: cuda)")
    parser.add_argument("--kv-cache-dtype", choices=SUPPORTED_KV_CACHE_DTYPES, default="model",
                        help="KV storage dtype; int8 is not built and is refused")
    parser.add_argument("--disable-cuda-graphs", action="store_true",
                        help="disable steady-state decode CUDA-graph replay")
    parser.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    parser.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    parser.add_argument("--max-new-tokens", type=int, default=8)
    parser.add_argument("--prompt-ids", action="append",
                        help="a prompt as token ids, e.g. '5 17 3' (may be given several times)")
    parser.add_argument("--prompt-file", help="file with one prompt of token ids per line")
    args = parser.parse_args(argv)

    scheduler = build_scheduler(
        args.model, scheduling_strategy=args.strategy, prefill_chunk_size=args.prefill_chunk_size,
        max_batch_size=args.max_batch_size, kv_cache_memory_mb=args.kv_cache_memory_mb,
        kv_cache_memory_utilization=args.kv_cache_memory_utilization, kv_cache_safety_mb=args.kv_cache_safety_mb,
        execution_dtype=args.dtype, decode_attention_backend=args.decode_attention_backend,
        kv_cache_dtype=args.kv_cache_dtype, enable_cuda_graphs=not args.disable_cuda_graphs,
        block_size=args.block_size, num_blocks=args.num_blocks,
        max_num_batched_tokens=args.max_num_batched_tokens, seed=args.seed)
    prompts = [_parse_ids(text) for text in (args.prompt_ids or [])]
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as handle:
            prompts.extend(_parse_ids(line) for line in handle if line.strip())
    if not prompts:
        # the reference's demo submits two prompts with max_new_tokens=8 (main.py:337-342)
        vocab = scheduler.engine.vocab_size
        prompts = [[(7 * i + 3) % vocab for i in range(5)], [(11 * i + 1) % vocab for i in range(3)]]
    ids = [scheduler.add_token_request(prompt, max_new_tokens=args.max_new_tokens,
                                       temperature=args.temperature, seed=args.seed + index)
           for index, prompt in enumerate(prompts)]
    results = scheduler.run_until_complete()
    for request_id in ids:
        print(f"request {request_id}: {results[request_id]!r}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
