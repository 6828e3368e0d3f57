"""B200-native (sm_100a) KV-cache hot path: append of RoPE'd K/V rows, GQA flash-decode
attention over the resident cache, prefix-KV snapshot / restore and truncation of rejected
speculative tokens, behind the C ABI declared in ``include/itak_cuda_compute.h``.

This package is the Python-side mirror of the backend seam (``CudaCompute`` stands where the
reference's ``CpuCompute`` stands).  There is no CPU path: every data-path call runs CUDA
kernels from the in-tree shared library and raises when that library or a device is missing.
"""
from .backend import (  # noqa: F401
    CudaCompute,
    CudaComputeError,
    DeviceSnapshot,
    KvDtype,
    PositionCache,
)
from . import _lib  # noqa: F401

__all__ = ["CudaCompute", "CudaComputeError", "DeviceSnapshot", "KvDtype", "PositionCache"]
