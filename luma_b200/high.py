"""Tensor-level entry points; mirrors luma-flash-attn/src/api/high.rs.

Same names, argument meaning and error behaviour as the reference's public functions
(high.rs:38-52, 82-109, 135-149): causal only, f32/f16/bf16 only, forward only. Tensors are torch
CUDA tensors standing in for luma's Tensor<Cuda, Float>; non-contiguous inputs are made
contiguous first (high.rs:217-219) and the output is a fresh, uninitialised allocation
(high.rs:240) that the kernels fully overwrite.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import error as E
from . import ffi, low


def _check_float(t: torch.Tensor, what: str) -> None:
    if t.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise E.Unsupported(f"{what}: dtype {t.dtype} (only f32/f16/bf16)")
    if not t.is_cuda:
        raise E.Unsupported(f"{what}: tensors must live on a CUDA device")


def flash_attn_func(q, k, v, softmax_scale: Optional[float] = None, causal: bool = True,
                    start_pos: int = 0, return_lse: bool = False):
    """Batched attention. q (B, Sq, Hq, d); k, v (B, Skv, Hkv, d) -> (B, Sq, Hq, d).

    Query token i sits at global position start_pos + i (high.rs:15-52). `return_lse` is this
    library's addition: also returns the fp32 log-sum-exp (B, Hq, Sq).
    """
    if not causal:
        raise E.Unsupported("flash_attn_func: non-causal is not supported yet (kernels are causal-only)")
    _check_float(q, "flash_attn_func")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise E.InvalidShape("flash_attn_func: q/k/v must be rank 4")
    b, sq, hq, d = q.shape
    bk, skv, hkv, dk = k.shape
    if tuple(v.shape) != tuple(k.shape) or bk != b or dk != d:
        raise E.InvalidShape(f"flash_attn_func: incompatible shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise E.Unsupported("flash_attn_func: q/k/v dtypes differ")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(d)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device) if return_lse else None
    low.flash_attn(q, k, v, o, b, sq, skv, hq, hkv, d, int(start_pos), scale, None, None, lse)
    return (o, lse) if return_lse else o


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                           softmax_scale: Optional[float] = None, causal: bool = True,
                           block_table=None):
    """Packed variable-length attention (high.rs:54-109). q (total_q, Hq, d); k, v
    (total_kv, Hkv, d) or, with `block_table` (batch, max_blocks), a paged cache
    (num_blocks, block_size, Hkv, d)."""
    if not causal:
        raise E.Unsupported("flash_attn_varlen_func: non-causal is not supported yet (kernels are causal-only)")
    _check_float(q, "flash_attn_varlen_func")
    if q.dim() != 3:
        raise E.InvalidShape("flash_attn_varlen_func: q must be (total_q, heads, head_size)")
    total_q, hq, d = q.shape
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise E.Unsupported("flash_attn_varlen_func: cu_seqlens must be i32")
    num_seqs = cu_seqlens_q.numel() - 1
    if block_table is not None:
        if k.dim() != 4:
            raise E.InvalidShape("flash_attn_varlen_func: paged k/v must be (num_blocks, block_size, heads, head_size)")
        if block_table.dtype != torch.int32:
            raise E.Unsupported("flash_attn_varlen_func: block_table must be i32")
        block_size, hkv = k.shape[1], k.shape[2]
        block_table = block_table.contiguous()
    else:
        if k.dim() != 3:
            raise E.InvalidShape("flash_attn_varlen_func: k/v must be (total_kv, heads, head_size)")
        block_size, hkv = 1, k.shape[1]  # high.rs:327
    if k.shape[-1] != d or tuple(v.shape) != tuple(k.shape):
        raise E.InvalidShape("flash_attn_varlen_func: incompatible q/k/v shapes")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(d)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q)
    low.flash_attn_varlen(q, k, v, o, cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous(), num_seqs,
                          int(max_seqlen_q), int(max_seqlen_k), hq, hkv, d, scale, block_table, block_size)
    return o


def flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens, block_table,
                            softmax_scale: Optional[float] = None):
    """Attention over a paged KV cache (high.rs:111-149). q (B, Sq, Hq, d); caches
    (num_blocks, block_size, Hkv, d); cache_seqlens (B,) i32 including the q tokens; block_table
    (B, max_blocks) i32. Sq == 1 decodes, Sq > 1 is chunked prefill (bottom-right causal)."""
    _check_float(q, "flash_attn_with_kvcache")
    if q.dim() != 4 or k_cache.dim() != 4 or v_cache.dim() != 4:
        raise E.InvalidShape("flash_attn_with_kvcache: q and caches must be rank 4")
    b, sq, hq, d = q.shape
    nb, block_size, hkv, dk = k_cache.shape
    if dk != d or tuple(v_cache.shape) != tuple(k_cache.shape):
        raise E.InvalidShape("flash_attn_with_kvcache: incompatible q/cache shapes")
    if cache_seqlens.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise E.Unsupported("flash_attn_with_kvcache: cache_seqlens/block_table must be i32")  # high.rs:525-531
    if block_table.dim() != 2 or block_table.shape[0] != b or cache_seqlens.numel() != b:
        raise E.InvalidShape("flash_attn_with_kvcache: block_table must be (batch, max_blocks), cache_seqlens (batch,)")
    max_blocks = block_table.shape[1]
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(d)
    q, k_cache, v_cache = q.contiguous(), k_cache.contiguous(), v_cache.contiguous()
    o = torch.empty_like(q)
    low.flash_attn_with_kvcache(q, k_cache, v_cache, o, block_table.contiguous(), cache_seqlens.contiguous(),
                                b, sq, hq, hkv, d, block_size, max_blocks, scale)
    return o


def host_steps(b: int, sq: int, chunk_rows: int = 0):
    """The (batch element, first row, end row) steps `flash_attn_func_host` cuts a call into."""
    import numpy as np
    n = ffi.lib.flash_attn_host_steps(b, sq, int(chunk_rows), None, 0)
    buf = np.zeros((max(n, 1), 3), dtype=np.int32)
    ffi.lib.flash_attn_host_steps(b, sq, int(chunk_rows), buf.ctypes.data, n)
    return [tuple(int(x) for x in row) for row in buf[:n]]


def flash_attn_func_host(q, k, v, out=None, softmax_scale: Optional[float] = None, causal: bool = True,
                         start_pos: int = 0, device=None, chunk_rows: Optional[int] = None):
    """Batched attention for HOST tensors (this library's addition; luma has no counterpart).

    q (B, Sq, Hq, d), k, v (B, Skv, Hkv, d) in (preferably pinned) host memory -> `out` (B, Sq, Hq, d)
    in host memory (allocated pinned when None). The library's `flash_attn_host_<T>` does the work: it
    is cut into steps of one batch element and `chunk_rows` query rows (a chunked prefill: the rows of
    a chunk see the keys up to their own position, so a chunk needs only the K/V rows up to its end,
    which travel with it) and the steps are pipelined over three streams: while one chunk is in the
    kernel, the next chunk's q rows and K/V rows are on their way to the device and the previous
    chunk's result on its way back, which keeps both directions of the host link busy instead of using
    them in turn. The caller's current stream waits for the last copy; `out` is complete when that
    stream has caught up.
    """
    if not causal:
        raise E.Unsupported("flash_attn_func_host: non-causal is not supported yet (kernels are causal-only)")
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise E.Unsupported("flash_attn_func_host: q/k/v must be host tensors (use flash_attn_func for device tensors)")
    if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise E.Unsupported(f"flash_attn_func_host: dtype {q.dtype} (only f32/f16/bf16)")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise E.InvalidShape("flash_attn_func_host: q/k/v must be rank 4")
    b, sq, hq, d = q.shape
    bk, skv, hkv, dk = k.shape
    if tuple(v.shape) != tuple(k.shape) or bk != b or dk != d:
        raise E.InvalidShape(f"flash_attn_func_host: incompatible shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise E.Unsupported("flash_attn_func_host: q/k/v dtypes differ")
    if start_pos < 0:
        raise E.InvalidStartPos(f"start_pos={start_pos}")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(d)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    elif out.is_cuda or tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
        raise E.InvalidShape("flash_attn_func_host: out must be a contiguous host tensor shaped and typed like q")
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = torch.cuda.current_stream(index).cuda_stream
    low.flash_attn_host(q, k, v, out, b, sq, skv, hq, hkv, d, int(start_pos), scale, index, int(chunk_rows or 0), stream)
    return out
