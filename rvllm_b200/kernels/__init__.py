"""The hand-written sm_100a kernels and their Python bindings."""
from .build import build, library_path

_OPS = None


def cuda_ops():
    """The process-wide CUDA kernel set; raises `KernelError` when there is no CUDA
    device or the native library cannot be built or loaded."""
    global _OPS
    if _OPS is None:
        from .bindings import CudaOps
        _OPS = CudaOps()
    return _OPS
