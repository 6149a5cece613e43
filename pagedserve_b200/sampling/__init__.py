"""Sampling: greedy and temperature (Gumbel-max with a counter-based generator)."""

from pagedserve_b200.sampling.sampler import Sampler, SamplingParams  # noqa: F401
