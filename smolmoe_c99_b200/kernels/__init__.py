"""The CUDA kernel library (sm_100a): build, load and Python faces."""
from .build import KernelBuildError, build, load
from .ops import KernelError, Ops, PAGE_SIZE, get_ops

__all__ = ["KernelBuildError", "KernelError", "Ops", "PAGE_SIZE", "build", "get_ops", "load"]
