"""Weights: safetensors reading/writing, by-name loading, seeded random models."""

from pagedserve_b200.weights.safetensors_io import read_safetensors, write_safetensors  # noqa: F401
from pagedserve_b200.weights.loader import (  # noqa: F401
    ParamSpec,
    WeightError,
    load_weights,
)
from pagedserve_b200.weights.random_init import write_random_model  # noqa: F401
