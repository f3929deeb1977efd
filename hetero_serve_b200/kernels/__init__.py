from .ops import AttentionGeometry, AttentionPlan, CudaOps, KernelError, load_library

__all__ = ["AttentionGeometry", "AttentionPlan", "CudaOps", "KernelError", "load_library"]
