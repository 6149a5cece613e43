"""Random-weights mode: write a model folder from a configuration and a seed.

The reference gets random weights from ``PagedDecoderLM(config)`` under
``torch.manual_seed`` (reference: main.py:115, benchmark.py:107).  Here the
tensors are produced in the checkpoint's own names and layouts so that the
same folder feeds the loader, a plain implementation and the reference model.

Every part says how each of its tensors is drawn (``init`` of its ParamSpec
companion, see ``Model.init_plan``): ``normal(std)``, ``ones_plus_normal(std)``.
Values are rounded to bfloat16 before they are stored, whatever the storage
dtype, so that a bfloat16 run and a float32 run start from the same numbers.
"""

from __future__ import annotations

import json
import os
from typing import Dict

import torch

from pagedserve_b200.config.registry import ModelConfig, resolve_architecture
from pagedserve_b200.weights.safetensors_io import write_safetensors

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(config: ModelConfig, seed: int, storage_dtype: str = "bfloat16") -> Dict[str, torch.Tensor]:
    """Seed-deterministic tensors in checkpoint names/layouts for ``config``."""
    from pagedserve_b200.models.model import init_plan

    if storage_dtype not in _STORAGE:
        raise ValueError(f"storage dtype must be one of {sorted(_STORAGE)}")
    _, _, builder = resolve_architecture(config.to_dict())
    spec = builder(config)
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    tensors: Dict[str, torch.Tensor] = {}
    for param, (kind, scale) in init_plan(spec):
        if kind == "skip":
            continue
        if param.role == "index":
            raise ValueError("random integer tables are not defined")
        noise = torch.randn(param.shape, generator=generator, dtype=torch.float32) * scale
        if kind == "ones_plus_normal":
            noise = noise + 1.0
        elif kind != "normal":
            raise ValueError(f"unknown init kind {kind!r}")
        stored_name = spec.checkpoint_name(param.name) if spec.checkpoint_name else param.name
        tensors[stored_name] = noise.to(torch.bfloat16).to(_STORAGE[storage_dtype])
    return tensors


def write_random_model(folder: str, config: ModelConfig, seed: int, storage_dtype: str = "bfloat16") -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``folder``; return it."""
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(config, seed, storage_dtype)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_dict(), handle, indent=1)
    write_safetensors(
        os.path.join(folder, "model.safetensors"), tensors,
        metadata={"format": "pt", "seed": str(seed)},
    )
    return folder
