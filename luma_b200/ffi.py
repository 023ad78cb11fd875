"""ctypes declarations of libflash_attn's C ABI; mirrors luma-flash-attn/src/api/ffi.rs:6-193.

The library is loaded from luma_b200/lib/libflash_attn.so (built by luma_b200/build.py). A missing
library is an ImportError: there is no fallback implementation.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p
from pathlib import Path

import os

# the in-tree build; LUMA_B200_LIB names another build of the same library (e.g. one made with other -D flags)
LIB_PATH = Path(os.environ.get("LUMA_B200_LIB") or (Path(__file__).resolve().parent / "lib" / "libflash_attn.so"))

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m luma_b200.build` "
        "(needs nvcc; the attention op has no CPU or PyTorch fallback)"
    )

lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_LOCAL)

DTYPE_SUFFIX = ("f32", "f16", "bf16")

_BATCH_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p,
               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
_BATCH_LSE_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
_VARLEN_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
_KVCACHE_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]

#: every symbol include/flash_attn.h declares
EXPORTED_SYMBOLS = (
    [f"flash_attn_{s}" for s in DTYPE_SUFFIX]
    + [f"flash_attn_varlen_{s}" for s in DTYPE_SUFFIX]
    + [f"flash_attn_with_kvcache_{s}" for s in DTYPE_SUFFIX]
    + ["flash_attn_last_error"]
    + [f"flash_attn_{s}_lse" for s in DTYPE_SUFFIX]
    + ["flash_attn_decode_bf16_noalloc", "flash_attn_f16_allgather", "flash_attn_bf16_allgather",
       "flash_attn_f16_allgather_lse", "flash_attn_bf16_allgather_lse",
       "flash_attn_f16_allgather_multicast", "flash_attn_bf16_allgather_multicast",
       "flash_attn_with_kvcache_f16_allgather", "flash_attn_with_kvcache_bf16_allgather",
       "flash_attn_kvcache_append", "flash_attn_varlen_f16_total", "flash_attn_varlen_bf16_total",
       "flash_attn_release_workspaces", "flash_attn_debug_launch_rank", "flash_attn_host_steps"]
    + [f"flash_attn_host_{s}" for s in DTYPE_SUFFIX]
    + [f"luma_softmax_{s}" for s in DTYPE_SUFFIX]   # include/luma_nn_kernels.h
    + ["flash_attn_debug_block_slots", "flash_attn_version", "flash_attn_device_status", "flash_attn_debug_read", "flash_attn_last_path",
       "flash_attn_last_launches", "flash_attn_set_option"]
    # include/luma_dist_comm.h
    + ["luma_comm_unique_id", "luma_comm_from_rank", "luma_comm_from_devices", "luma_comm_rank", "luma_comm_world_size",
       "luma_comm_device", "luma_comm_all_gather", "luma_comm_barrier", "luma_comm_destroy", "luma_ipc_export",
       "luma_ipc_open", "luma_ipc_close", "luma_peer_copy", "luma_comm_last_error"]
)

for _s in DTYPE_SUFFIX:
    getattr(lib, f"luma_softmax_{_s}").argtypes = [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_void_p]
    getattr(lib, f"luma_softmax_{_s}").restype = c_int

_VARLEN_TOTAL_ARGS = _VARLEN_ARGS[:-1] + [c_int, c_int, c_void_p]
for _s in ("f16", "bf16"):
    getattr(lib, f"flash_attn_varlen_{_s}_total").argtypes = _VARLEN_TOTAL_ARGS
    getattr(lib, f"flash_attn_varlen_{_s}_total").restype = c_int

for _s in DTYPE_SUFFIX:
    getattr(lib, f"flash_attn_{_s}").argtypes = _BATCH_ARGS
    getattr(lib, f"flash_attn_{_s}").restype = c_int
    getattr(lib, f"flash_attn_{_s}_lse").argtypes = _BATCH_LSE_ARGS
    getattr(lib, f"flash_attn_{_s}_lse").restype = c_int
    getattr(lib, f"flash_attn_varlen_{_s}").argtypes = _VARLEN_ARGS
    getattr(lib, f"flash_attn_varlen_{_s}").restype = c_int
    getattr(lib, f"flash_attn_with_kvcache_{_s}").argtypes = _KVCACHE_ARGS
    getattr(lib, f"flash_attn_with_kvcache_{_s}").restype = c_int

lib.flash_attn_decode_bf16_noalloc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
lib.flash_attn_decode_bf16_noalloc.restype = c_int
for _s in ("f16", "bf16"):
    getattr(lib, f"flash_attn_{_s}_allgather").argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                          c_float, c_void_p]
    getattr(lib, f"flash_attn_{_s}_allgather").restype = c_int
    getattr(lib, f"flash_attn_{_s}_allgather_lse").argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                              c_float, c_void_p]
    getattr(lib, f"flash_attn_{_s}_allgather_lse").restype = c_int
    getattr(lib, f"flash_attn_{_s}_allgather_multicast").argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                                    c_void_p]
    getattr(lib, f"flash_attn_{_s}_allgather_multicast").restype = c_int
    getattr(lib, f"flash_attn_with_kvcache_{_s}_allgather").argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                                       c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                                       c_int, c_int, c_float, c_void_p]
    getattr(lib, f"flash_attn_with_kvcache_{_s}_allgather").restype = c_int
lib.flash_attn_debug_launch_rank.argtypes = [c_int, c_int, c_int]
lib.flash_attn_debug_launch_rank.restype = c_int
_HOST_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
for _s in DTYPE_SUFFIX:
    getattr(lib, f"flash_attn_host_{_s}").argtypes = _HOST_ARGS
    getattr(lib, f"flash_attn_host_{_s}").restype = c_int
lib.flash_attn_host_steps.argtypes = [c_int, c_int, c_int, c_void_p, c_int]
lib.flash_attn_host_steps.restype = c_int
lib.flash_attn_release_workspaces.argtypes = []
lib.flash_attn_release_workspaces.restype = c_int
lib.luma_comm_unique_id.argtypes = [c_void_p]
lib.luma_comm_from_rank.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int]
lib.luma_comm_from_devices.argtypes = [c_void_p, c_int, c_void_p]
lib.luma_comm_rank.argtypes = [c_void_p]
lib.luma_comm_world_size.argtypes = [c_void_p]
lib.luma_comm_device.argtypes = [c_void_p]
lib.luma_comm_all_gather.argtypes = [c_void_p, c_void_p, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p]
lib.luma_comm_barrier.argtypes = [c_void_p, c_void_p]
lib.luma_comm_destroy.argtypes = [c_void_p]
lib.luma_ipc_export.argtypes = [c_void_p, c_void_p, c_void_p]
lib.luma_ipc_open.argtypes = [c_void_p, ctypes.c_longlong, c_void_p]
lib.luma_ipc_close.argtypes = [c_void_p]
lib.luma_peer_copy.argtypes = [c_void_p, c_void_p, ctypes.c_longlong, c_void_p]
lib.luma_comm_last_error.argtypes = []
lib.luma_comm_last_error.restype = c_char_p
lib.flash_attn_kvcache_append.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
lib.flash_attn_kvcache_append.restype = c_int
lib.flash_attn_last_error.argtypes = []
lib.flash_attn_last_error.restype = c_char_p
lib.flash_attn_version.argtypes = []
lib.flash_attn_version.restype = c_char_p
lib.flash_attn_device_status.argtypes = []
lib.flash_attn_device_status.restype = c_int
lib.flash_attn_debug_read.argtypes = [c_void_p, c_int]
lib.flash_attn_debug_read.restype = c_int
lib.flash_attn_last_path.argtypes = []
lib.flash_attn_last_path.restype = c_char_p
lib.flash_attn_last_launches.argtypes = []
lib.flash_attn_last_launches.restype = c_int
lib.flash_attn_set_option.argtypes = [c_char_p, c_int]
lib.flash_attn_set_option.restype = c_int
lib.flash_attn_debug_block_slots.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
lib.flash_attn_debug_block_slots.restype = c_int


def last_error() -> str:
    """flash_attn_last_error() as str; NULL is treated as "" like error.rs:66-75."""
    p = lib.flash_attn_last_error()
    return "" if p is None else p.decode("utf-8", "replace")


def last_path() -> str:
    p = lib.flash_attn_last_path()
    return "" if p is None else p.decode()


def device_status() -> int:
    """Synchronises, then reads and clears the device status word (0 = healthy)."""
    return int(lib.flash_attn_device_status())


def _options_from_environment() -> None:
    """LUMA_B200_OPTIONS="name=value,name=value" sets the library's integer knobs at import
    (flash_attn_set_option), e.g. to run a test suite with another kernel variant."""
    import os
    for item in os.environ.get("LUMA_B200_OPTIONS", "").split(","):
        name, sep, value = item.partition("=")
        if sep and name.strip():
            if lib.flash_attn_set_option(name.strip().encode(), int(value)) != 0:
                raise KeyError(f"LUMA_B200_OPTIONS: unknown option {name.strip()!r}")


_options_from_environment()


def last_launches() -> int:
    return int(lib.flash_attn_last_launches())


def set_option(name: str, value: int) -> None:
    if lib.flash_attn_set_option(name.encode(), int(value)) != 0:
        raise KeyError(name)
