from .ops import AttentionGeometry, CudaOps, KernelError, load_library

__all__ = ["AttentionGeometry", "CudaOps", "KernelError", "load_library"]
