"""Kernel libraries: nvcc build driver and ctypes wrappers."""

from pagedserve_b200.kernels.build import BuildError, build_all, load  # noqa: F401
from pagedserve_b200.kernels.ops import KernelError, Ops  # noqa: F401
