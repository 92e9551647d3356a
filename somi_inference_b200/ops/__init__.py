"""Kernel table: the ctypes wrappers over the sm_100a library built from `csrc/`."""

from .build import BuildError, build
from .cuda import CudaOps, KernelError, cuda_ops

__all__ = ["BuildError", "build", "CudaOps", "KernelError", "cuda_ops"]
