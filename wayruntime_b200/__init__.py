"""wayruntime_b200 — B200 (sm_100a) attention hot path for wayruntime.

The product is ``lib/libwr_cuda.so`` (CUDA kernels behind the C-ABI declared
in ``include/wr_cuda.h``).  This package only loads it and mirrors the calls
for Python callers; there is no CPU path, and loading fails loudly when the
library is missing.
"""
from .binding import (  # noqa: F401
    Batch,
    Exchange,
    Context,
    DeviceModel,
    KVCache,
    WrCudaError,
    MEM_DEVICE,
    MEM_HOST,
    F16,
    F32,
    APPEND_ROPE,
    TRIPLE_PAD,
    device_check,
    load_library,
    status_name,
)

__all__ = [
    "Batch", "Context", "DeviceModel", "Exchange", "KVCache", "WrCudaError", "MEM_DEVICE", "MEM_HOST", "F16", "F32",
    "APPEND_ROPE", "TRIPLE_PAD", "device_check", "load_library", "status_name",
]
