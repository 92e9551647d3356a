"""Kernel table: the ctypes wrappers over the sm_100a library built from `csrc/`."""

from .build import BuildError, build, build_library
from .cuda import CudaOps, KernelError, cuda_ops

__all__ = ["BuildError", "build", "build_library", "CudaOps", "KernelError", "cuda_ops"]
