"""The engine: a model, its cache, the step function and the sampler on one GPU.

Python entry point in the manner of the reference's ``build_scheduler``
(reference: main.py:136-254), but from a model folder (``config.json`` +
``model.safetensors``) or a configuration and a seed instead of a model name.
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from pagedserve_b200.cache.budget import MIB, kv_cache_budget, pages_for_budget
from pagedserve_b200.cache.manager import CacheManager
from pagedserve_b200.config.engine_config import EngineConfig
from pagedserve_b200.config.registry import ModelConfig, load_config_dict, resolve_architecture
from pagedserve_b200.engine.step import ModelRunner
from pagedserve_b200.kernels.ops import Ops
from pagedserve_b200.models.model import Model
from pagedserve_b200.parts.base import PartEnv
from pagedserve_b200.sampling.sampler import Sampler

_TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class Engine:
    def __init__(self, model_config: ModelConfig, engine_config: EngineConfig, folder: Optional[str] = None,
                 tensors: Optional[Dict[str, torch.Tensor]] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("pagedserve_b200 needs a CUDA device: there is no CPU path")
        self.model_config = model_config
        self.config = engine_config
        self.device = torch.device(engine_config.device)
        torch.cuda.set_device(self.device)
        self.dtype = _TORCH_DTYPE[engine_config.dtype]
        _, _, builder = resolve_architecture(model_config.to_dict())
        self.spec = builder(model_config)
        self.ops = Ops(self.dtype)
        env = PartEnv(ops=self.ops, dtype=self.dtype, device=self.device)
        self.model = Model(self.spec, env)
        if folder is not None:
            self.model.load_folder(folder)
        elif tensors is not None:
            self.model.load_tensors(tensors)
        else:
            raise ValueError("an engine needs a model folder or tensors")
        self.cache = self._make_cache()
        self.runner = ModelRunner(self.model, self.cache, self.device,
                                  max_step_tokens=engine_config.max_num_batched_tokens,
                                  enable_cuda_graphs=engine_config.enable_cuda_graphs)
        self.sampler = Sampler(self.ops, self.device, max_rows=max(64, engine_config.max_num_seqs))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, engine_config: Optional[EngineConfig] = None, **overrides) -> "Engine":
        """``folder`` holds config.json and model.safetensors; the model class follows config.json."""
        engine_config = engine_config or EngineConfig(**overrides)
        values = load_config_dict(folder)
        _, config_class, _ = resolve_architecture(values)
        return cls(config_class.from_dict(values), engine_config, folder=folder)

    @classmethod
    def random(cls, model_config: ModelConfig, seed: int, engine_config: Optional[EngineConfig] = None,
               **overrides) -> "Engine":
        """A model of ``model_config`` with seeded random weights (nothing is written to disk)."""
        from pagedserve_b200.weights.random_init import random_tensors

        engine_config = engine_config or EngineConfig(**overrides)
        return cls(model_config, engine_config, tensors=random_tensors(model_config, seed))

    def _make_cache(self) -> CacheManager:
        cfg = self.config
        kv_needs = self.model.kv_needs()
        state_needs = self.model.state_needs()
        width = torch.empty(0, dtype=self.dtype).element_size()
        # bytes one page costs summed over the groups (each group has its own pool of equal page count)
        by_need: Dict[object, int] = {}
        for need in kv_needs:
            if need is not None:
                by_need[need] = by_need.get(need, 0) + 1
        bytes_per_page = sum(2 * count * need.n_kv_heads * need.head_dim * cfg.block_size * width
                             for need, count in by_need.items())
        self.bytes_per_block = bytes_per_page
        if cfg.num_blocks is not None:
            num_pages = cfg.num_blocks
        elif cfg.kv_cache_memory_mb is not None:
            # reference: src/model/kv_manager.py:55-64
            num_pages = (cfg.kv_cache_memory_mb * MIB) // max(bytes_per_page, 1)
            if num_pages == 0:
                raise ValueError(f"Memory budget is too small; one block requires {bytes_per_page} bytes")
        else:
            # reference: main.py:186-200 (budget from the device's free and total memory)
            free, total = torch.cuda.mem_get_info(self.device)
            budget = kv_cache_budget(free, total, cfg.kv_cache_memory_utilization, cfg.kv_cache_safety_mb * MIB)
            num_pages = pages_for_budget(budget, bytes_per_page, cfg.max_num_seqs, self.spec.max_model_len,
                                         cfg.block_size)
        return CacheManager(kv_needs, state_needs, cfg.block_size, int(num_pages), cfg.max_num_seqs,
                            self.spec.max_model_len, dtype=self.dtype, device=self.device,
                            scratch_tokens=ModelRunner.PAD_LONG)

    # ------------------------------------------------------------------ the calls a user makes
    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    @property
    def max_model_len(self) -> int:
        return self.spec.max_model_len

    def step(self, entries: Sequence) -> torch.Tensor:
        """Run (request, tokens, want) entries as one batch; float32 logits at the wanted places."""
        return self.runner.step(entries)

    def decode(self, entries: Sequence, temperatures, seeds, steps: int = 1):
        """Run ``steps`` decode steps of single-token entries on the device (sampling included);
        returns the sampled tokens as an int32 array ``[steps, batch]``."""
        return self.runner.decode(entries, temperatures, seeds, steps)

    def decode_tokens(self, requests: Sequence[Hashable], tokens: Sequence[int], temperatures, seeds,
                      steps: int = 1, stage_next: bool = False):
        """``decode`` with the requests and their next tokens as two sequences (no entry objects);
        ``stage_next`` announces one more step of the same requests."""
        return self.runner.decode_tokens(requests, tokens, temperatures, seeds, steps, stage_next)

    def finish(self, request: Hashable) -> None:
        self.runner.finish(request)

    def check_status(self) -> None:
        """Raise if a kernel of an earlier step flagged bad input or gave up a wait (synchronises)."""
        self.runner.check_status()

    def sample(self, logits, temperatures, seeds, positions) -> List[int]:
        return self.sampler.sample(logits, temperatures, seeds, positions)

    def make_scheduler(self, **kwargs):
        from pagedserve_b200.engine.scheduler import Scheduler

        cfg = self.config
        defaults = dict(max_num_seqs=cfg.max_num_seqs, max_num_batched_tokens=cfg.max_num_batched_tokens,
                        strategy=cfg.strategy, prefill_chunk_size=cfg.prefill_chunk_size)
        defaults.update(kwargs)
        return Scheduler(self, **defaults)


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16,
             temperature: float = 0.0, seed: int = 0, **scheduler_options) -> List[List[int]]:
    """Token ids in, token ids out: run ``prompts`` to completion with continuous batching."""
    scheduler = engine.make_scheduler(**scheduler_options)
    ids = [scheduler.add_token_request(prompt, max_new_tokens=max_new_tokens, temperature=temperature,
                                       seed=seed + index)
           for index, prompt in enumerate(prompts)]
    results = scheduler.run_until_complete()
    return [results[request_id] for request_id in ids]
