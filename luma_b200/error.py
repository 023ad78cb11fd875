"""Typed errors of the attention op; mirrors luma-flash-attn/src/error.rs:7-75.

`from_status` maps a C status code to the error class and attaches the library's thread-local
message, exactly as FlashAttnError::from_status does (error.rs:38-51).
"""
from __future__ import annotations


class FlashAttnError(Exception):
    """Base class; str() reproduces the reference's Display strings (error.rs:9-31)."""

    prefix = "flash_attn: error"

    def __init__(self, detail: str = ""):
        self.detail = detail
        super().__init__(f"{self.prefix} ({detail})")


class NullPtr(FlashAttnError):
    prefix = "flash_attn: null pointer parameter"


class InvalidShape(FlashAttnError):
    prefix = "flash_attn: invalid shape parameter"


class InvalidHeadSize(FlashAttnError):
    prefix = "flash_attn: unsupported head_size"


class InvalidStartPos(FlashAttnError):
    prefix = "flash_attn: invalid start_pos"


class BufferTooSmall(FlashAttnError):
    prefix = "flash_attn: buffer too small"


class CudaError(FlashAttnError):
    prefix = "flash_attn: CUDA error"


class Unsupported(FlashAttnError):
    prefix = "flash_attn: unsupported"


class Unknown(FlashAttnError):
    def __init__(self, code: int):
        self.code = code
        Exception.__init__(self, f"flash_attn: unknown error code {code}")
        self.detail = str(code)


FLASH_ATTN_OK = 0
FLASH_ATTN_ERR_NULL_PTR = 1
FLASH_ATTN_ERR_INVALID_SHAPE = 2
FLASH_ATTN_ERR_INVALID_HEAD_SIZE = 3
FLASH_ATTN_ERR_INVALID_START_POS = 4
FLASH_ATTN_ERR_CUDA = 5

_BY_STATUS = {
    FLASH_ATTN_ERR_NULL_PTR: NullPtr,
    FLASH_ATTN_ERR_INVALID_SHAPE: InvalidShape,
    FLASH_ATTN_ERR_INVALID_HEAD_SIZE: InvalidHeadSize,
    FLASH_ATTN_ERR_INVALID_START_POS: InvalidStartPos,
    FLASH_ATTN_ERR_CUDA: CudaError,
}


def from_status(status: int, last_error: str) -> None:
    """Raises the error for a non-zero status; returns None on FLASH_ATTN_OK."""
    if status == FLASH_ATTN_OK:
        return None
    cls = _BY_STATUS.get(status)
    if cls is None:
        raise Unknown(status)
    raise cls(last_error)
