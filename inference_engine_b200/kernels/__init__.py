from .build import BuildError, build_core, build_library
from .cuda_ops import CudaOps, KernelError, get_ops

__all__ = ["BuildError", "CudaOps", "KernelError", "build_core", "build_library", "get_ops"]
