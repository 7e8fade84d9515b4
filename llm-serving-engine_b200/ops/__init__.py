from .cuda_ops import CudaOps, get_ops

__all__ = ["CudaOps", "get_ops"]
