"""numpy front end of oracle/liboracle.so (test infrastructure, not a product path).

Wraps the C++ restatement in attention_oracle.cpp:
  sdpa_math_f32   — luma-cpu's math-path attention in f32 (luma-tensor/src/ops/nn/attention.rs:11-45)
  attn_f64_*      — the f64 loop of the reference's GPU tests (luma-flash-attn/tests/low.rs:45-117,
                    tests/high.rs:29-86) for the batched / varlen / paged-cache entry points
  block_slots     — host walk of the block table (luma-flash-attn/kernels/common.cuh:89-108)
  XorShift        — the tests' xorshift64* generator (tests/low.rs:363-384, tests/high.rs:13-24)
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_uint64, c_void_p
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
LIB_PATH = _DIR / "liboracle.so"


def reference_root():
    """Where the reference tree is mounted, if anywhere: the environment variable LUMA_REF_ROOT, else
    a sibling `reference` directory of this repository's parent."""
    env = os.environ.get("LUMA_REF_ROOT")
    cand = Path(env) if env else _DIR.parent.parent / "reference"
    return cand if (cand / "luma-flash-attn" / "kernels").is_dir() else None


def build() -> Path:
    """Compiles liboracle.so and, where the reference tree is mounted, the reference's own CUDA
    kernels into oracle/_ref. A reference tree that is present but does not build is an error."""
    subprocess.run(["make", "-C", str(_DIR), "-s"], check=True)
    ref = reference_root()
    if ref is not None:
        subprocess.run(["make", "-C", str(_DIR), "-s", "ref", f"REF_ROOT={ref}"], check=True)
    return LIB_PATH


def _load():
    if not LIB_PATH.exists():
        build()
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.oracle_sdpa_math_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_double, c_int, c_int, c_int]
    lib.oracle_sdpa_math_f32.restype = c_int
    lib.oracle_block_slots.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.oracle_block_slots.restype = c_int
    lib.oracle_attn_f64.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_double,
                                    c_void_p, c_int, c_int, c_void_p, c_int, c_int]
    lib.oracle_attn_f64.restype = c_int
    lib.oracle_xorshift_fill_f32.argtypes = [POINTER(c_uint64), c_void_p, c_int64]
    lib.oracle_xorshift_fill_f32.restype = None
    lib.oracle_xorshift_fill_f64.argtypes = [POINTER(c_uint64), c_void_p, c_int64]
    lib.oracle_xorshift_fill_f64.restype = None
    lib.oracle_hardware_threads.argtypes = []
    lib.oracle_hardware_threads.restype = c_int
    return lib


_lib = _load()


def hardware_threads() -> int:
    """luma-cpu's rule: RAYON_NUM_THREADS, else every core (luma-cpu/src/kernels/matmul.rs:13-15)."""
    env = os.environ.get("RAYON_NUM_THREADS")
    if env and env.isdigit() and int(env) > 0:
        return int(env)
    return int(_lib.oracle_hardware_threads())


def _p(a):
    return None if a is None else a.ctypes.data


def sdpa_math_f32(q, k, v, scale=None, causal=True, start_pos=0, nthreads=None, return_lse=False):
    """q (B, Lq, Hq, D), k/v (B, Lk, Hkv, D) float32 -> (B, Lq, Hq, D) float32 [, lse (B, Hq, Lq)]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, Lq, Hq, D = q.shape
    _, Lk, Hkv, _ = k.shape
    if scale is None:
        scale = 1.0 / np.sqrt(float(D))
    o = np.empty_like(q)
    lse = np.empty((B, Hq, Lq), dtype=np.float32) if return_lse else None
    rc = _lib.oracle_sdpa_math_f32(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Lq, Lk, Hq, Hkv, D,
                                   float(scale), int(bool(causal)), int(start_pos),
                                   int(nthreads or hardware_threads()))
    if rc != 0:
        raise ValueError("oracle_sdpa_math_f32: bad arguments")
    return (o, lse) if return_lse else o


def softmax_last_dim_f32(x):
    """Row softmax over the last dimension with luma-cpu's online softmax, f32 (any leading shape)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    rows = x.size // n if n else 0
    out = np.empty_like(x)
    _lib.oracle_softmax_last_dim_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int]
    _lib.oracle_softmax_last_dim_f32.restype = ctypes.c_int
    if _lib.oracle_softmax_last_dim_f32(_p(x), _p(out), rows, n) != 0:
        raise ValueError("oracle_softmax_last_dim_f32: bad arguments")
    return out


def _attn_f64(q, k, v, q_start, q_len, kv_start, kv_len, pos_off, Hq, Hkv, D, scale,
              block_tables=None, max_blocks=0, block_size=0, mask=None, mask_stride=0,
              nthreads=None, return_lse=False):
    q = np.ascontiguousarray(q, dtype=np.float64)
    k = np.ascontiguousarray(k, dtype=np.float64)
    v = np.ascontiguousarray(v, dtype=np.float64)
    o = np.zeros_like(q)
    lse = np.empty(q.size // D, dtype=np.float64) if return_lse else None
    arrs = [np.ascontiguousarray(a, dtype=np.int32) for a in (q_start, q_len, kv_start, kv_len, pos_off)]
    bt = None if block_tables is None else np.ascontiguousarray(block_tables, dtype=np.int32)
    mk = None if mask is None else np.ascontiguousarray(mask, dtype=np.uint8)
    rc = _lib.oracle_attn_f64(_p(q), _p(k), _p(v), _p(o), _p(lse), len(arrs[0]),
                              *[_p(a) for a in arrs], Hq, Hkv, D, float(scale),
                              _p(bt), int(max_blocks), int(block_size), _p(mk), int(mask_stride),
                              int(nthreads or hardware_threads()))
    if rc != 0:
        raise ValueError("oracle_attn_f64: bad arguments")
    return (o, lse) if return_lse else o


def attn_f64_batch(q, k, v, scale=None, start_pos=0, mask=None, return_lse=False):
    """Batched reference with start_pos and optional (B, Skv) padding mask (tests/low.rs:45-117).
    With return_lse the lse comes back as (B, Hq, Sq)."""
    B, Sq, Hq, D = q.shape
    _, Skv, Hkv, _ = k.shape
    if scale is None:
        scale = 1.0 / np.sqrt(float(D))
    idx = np.arange(B, dtype=np.int32)
    res = _attn_f64(q, k, v, idx * Sq, np.full(B, Sq), idx * Skv, np.full(B, Skv), np.full(B, start_pos),
                    Hq, Hkv, D, scale, mask=mask, mask_stride=Skv, return_lse=return_lse)
    if return_lse:
        o, lse = res
        return o.reshape(q.shape), lse.reshape(B, Sq, Hq).transpose(0, 2, 1).copy()
    return res.reshape(q.shape)


def attn_f64_varlen(q, k, v, cu_q, cu_k, scale=None, block_table=None):
    """Packed varlen reference, bottom-right causal; k/v contiguous (total_kv, Hkv, D) or a paged
    cache (num_blocks, block_size, Hkv, D) with block_table (num_seqs, max_blocks)."""
    total_q, Hq, D = q.shape
    cu_q = np.asarray(cu_q, dtype=np.int64)
    cu_k = np.asarray(cu_k, dtype=np.int64)
    ql, kl = np.diff(cu_q), np.diff(cu_k)
    if scale is None:
        scale = 1.0 / np.sqrt(float(D))
    if block_table is not None:
        nb, bs, Hkv, _ = k.shape
        bt = np.asarray(block_table, dtype=np.int32)
        return _attn_f64(q, k, v, cu_q[:-1], ql, np.zeros_like(ql), kl, kl - ql, Hq, Hkv, D, scale,
                         block_tables=bt, max_blocks=bt.shape[1], block_size=bs).reshape(q.shape)
    Hkv = k.shape[1]
    return _attn_f64(q, k, v, cu_q[:-1], ql, cu_k[:-1], kl, kl - ql, Hq, Hkv, D, scale).reshape(q.shape)


def attn_f64_kvcache(q, k_cache, v_cache, cache_seqlens, block_table, scale=None):
    """Paged-cache reference: q (B, Sq, Hq, D); row i sits at cache_seqlens[s] - Sq + i."""
    B, Sq, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    lens = np.asarray(cache_seqlens, dtype=np.int32)
    bt = np.asarray(block_table, dtype=np.int32)
    if scale is None:
        scale = 1.0 / np.sqrt(float(D))
    idx = np.arange(B, dtype=np.int32)
    return _attn_f64(q, k_cache, v_cache, idx * Sq, np.full(B, Sq), np.zeros(B), lens, lens - Sq,
                     Hq, Hkv, D, scale, block_tables=bt, max_blocks=bt.shape[1], block_size=bs).reshape(q.shape)


def block_slots(block_table, lens, block_size):
    """Host walk of the block table: concatenated physical token slots of every sequence."""
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    out = np.empty(int(lens.sum()), dtype=np.int32)
    rc = _lib.oracle_block_slots(_p(bt), _p(lens), bt.shape[0], bt.shape[1], int(block_size), _p(out))
    if rc != 0:
        raise ValueError("oracle_block_slots: bad arguments")
    return out


class XorShift:
    """xorshift64* stream; one instance continues across tensors like tests/low.rs:148-152."""

    def __init__(self, seed: int):
        self.state = c_uint64(int(seed) | 1)

    def f32(self, n: int) -> np.ndarray:
        out = np.empty(int(n), dtype=np.float32)
        _lib.oracle_xorshift_fill_f32(ctypes.byref(self.state), _p(out), int(n))
        return out

    def f64(self, n: int) -> np.ndarray:
        out = np.empty(int(n), dtype=np.float64)
        _lib.oracle_xorshift_fill_f64(ctypes.byref(self.state), _p(out), int(n))
        return out


def data_f64(n: int, seed: int) -> np.ndarray:
    """tests/high.rs:13-24 `data(n, seed)`."""
    return XorShift(seed).f64(n)
