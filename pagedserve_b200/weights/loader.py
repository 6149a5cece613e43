"""Load a model's tensors by name and report every mismatch in one error.

Each part of a model declares the tensors it needs as :class:`ParamSpec`
entries (name in the checkpoint, shape as stored, role, optional transform).
``load_weights`` matches them against a safetensors file, applies the
transforms (the GPT-2 "Conv1D" ``[in, out]`` matrices are transposed once into
``[out, in]``, K-major for the GEMM's B operand; reference:
src/model/gpt2.py:14-17) and casts by role:

=========  =====================================================
role       kept as
=========  =====================================================
matmul     the engine's compute dtype (bfloat16 or float32)
table      the engine's compute dtype (embedding tables)
vector     float32 (norm scale/shift, biases: they feed 32-bit math)
keep32     float32 when stored in 32-bit, else the compute dtype
index      int32 (integer tables)
=========  =====================================================
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

from pagedserve_b200.weights.safetensors_io import read_safetensors

ROLES = ("matmul", "table", "vector", "keep32", "index")


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; lists all of them."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), not_tied=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.not_tied = list(not_tied)        # (name, name it is tied to): stored copies that differ


@dataclass(frozen=True)
class ParamSpec:
    name: str                         # canonical checkpoint name
    shape: Tuple[int, ...]            # shape as stored in the file
    role: str = "matmul"
    transpose: bool = False           # store [in,out] -> keep [out,in]
    optional: bool = False            # may be absent (e.g. a tied head)
    same_as: Optional[str] = None     # canonical name of the tensor this one is tied to: a stored copy must
                                      # equal it (reference: src/model/gpt2.py:42, 77-78 ties or copies the head)

    def __post_init__(self):
        if self.role not in ROLES:
            raise ValueError(f"unknown role {self.role!r}")


def _target_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if role == "index":
        return torch.int32
    if role == "vector":
        return torch.float32
    if role == "keep32":
        return torch.float32 if stored in (torch.float32, torch.float64) else compute
    return compute


def place_tensors(
    specs: Sequence[ParamSpec],
    stored: Dict[str, torch.Tensor],
    compute_dtype: torch.dtype,
    device,
    normalise_name: Optional[Callable[[str], Optional[str]]] = None,
    source: str = "<tensors>",
) -> Dict[str, torch.Tensor]:
    """Match ``stored`` against ``specs``; return {canonical name: device tensor}.

    ``normalise_name`` maps a name found in the file to its canonical name, or
    to ``None`` for tensors that are to be ignored (non-parameter buffers).
    """
    canonical: Dict[str, torch.Tensor] = {}
    origin: Dict[str, str] = {}
    for name, tensor in stored.items():
        mapped = normalise_name(name) if normalise_name is not None else name
        if mapped is None:
            continue
        if mapped in canonical:
            raise WeightError(f"{source}: tensors {origin[mapped]!r} and {name!r} name the same parameter")
        canonical[mapped] = tensor
        origin[mapped] = name

    wanted = {spec.name: spec for spec in specs}
    missing = [spec.name for spec in specs if spec.name not in canonical and not spec.optional]
    unexpected = sorted(origin[name] for name in canonical if name not in wanted)
    wrong_shape = []
    wrong_dtype = []
    for name, spec in wanted.items():
        tensor = canonical.get(name)
        if tensor is None:
            continue
        if tuple(tensor.shape) != tuple(spec.shape):
            wrong_shape.append((origin[name], tuple(spec.shape), tuple(tensor.shape)))
        if spec.role == "index":
            if tensor.dtype.is_floating_point:
                wrong_dtype.append((origin[name], "integer", str(tensor.dtype)))
        elif not tensor.dtype.is_floating_point:
            wrong_dtype.append((origin[name], "floating point", str(tensor.dtype)))
    not_tied = []
    for name, spec in wanted.items():
        tensor, twin = canonical.get(name), canonical.get(spec.same_as) if spec.same_as else None
        if tensor is None or twin is None or tensor.shape != twin.shape:
            continue                          # absent, or already reported above
        if not torch.equal(tensor.to(torch.float32), twin.to(torch.float32)):
            not_tied.append((origin[name], origin[spec.same_as]))
    if missing or unexpected or wrong_shape or wrong_dtype or not_tied:
        lines = [f"{source}: the tensors do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, expected, got in wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(expected)}, got {list(got)}")
        for name, expected, got in wrong_dtype:
            lines.append(f"  wrong dtype: {name}: expected {expected}, got {got}")
        for name, twin in not_tied:
            lines.append(f"  not tied: {name} differs from {twin}, to which the configuration ties it")
        raise WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype, not_tied)

    placed: Dict[str, torch.Tensor] = {}
    for name, spec in wanted.items():
        tensor = canonical.get(name)
        if tensor is None or (spec.same_as and spec.same_as in canonical):
            continue                          # absent, or an equal copy of a tensor that is placed anyway
        if spec.transpose:
            tensor = tensor.transpose(0, 1)
        target = _target_dtype(spec.role, tensor.dtype, compute_dtype)
        placed[name] = tensor.to(device=device, dtype=target).contiguous()
    return placed


def load_weights(
    folder: str,
    specs: Sequence[ParamSpec],
    compute_dtype: torch.dtype,
    device,
    normalise_name: Optional[Callable[[str], Optional[str]]] = None,
) -> Dict[str, torch.Tensor]:
    path = os.path.join(folder, "model.safetensors")
    if not os.path.isfile(path):
        raise WeightError(f"no model.safetensors in {folder!r}")
    stored = read_safetensors(path)
    return place_tensors(specs, stored, compute_dtype, device, normalise_name, source=path)
