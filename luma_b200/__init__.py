"""Host-side mirror of luma's `luma-flash-attn` crate over the sm_100a attention library.

Layers, named after the reference's modules (luma-flash-attn/src/api/):
  ffi   — ctypes declarations of the C ABI (ffi.rs)
  low   — device-buffer API with argument validation (low.rs)
  high  — tensor-level entry points flash_attn_func / flash_attn_varlen_func /
          flash_attn_with_kvcache (high.rs)
  error — FlashAttnError hierarchy (error.rs)
  dist  — head-sharded attention + output all-gather (luma-dist Comm::all_gather)
  functional — the Math / Flash dispatcher of luma-nn (functional/attention.rs); Math is the
          reference's portable tensor-op path, chosen only when the caller names it — Flash
          never falls back to it

There is no CPU implementation behind any of these: importing `ffi` without a built
libflash_attn.so raises, and every compute call needs a CUDA device.
"""
from .error import (  # noqa: F401
    FlashAttnError, NullPtr, InvalidShape, InvalidHeadSize, InvalidStartPos, BufferTooSmall,
    CudaError, Unsupported, Unknown,
)

__all__ = [
    "FlashAttnError", "NullPtr", "InvalidShape", "InvalidHeadSize", "InvalidStartPos",
    "BufferTooSmall", "CudaError", "Unsupported", "Unknown",
]
