"""Device-buffer API; mirrors luma-flash-attn/src/api/low.rs.

Buffers are torch CUDA tensors used purely as typed device memory (the role cudarc's
CudaSlice<T> plays in the reference): `numel()` is the slice length, `data_ptr()` the pointer.
Dims are explicit i32 arguments and the layout is assumed dense, exactly as in low.rs. `stream`
is a torch.cuda.Stream or None (the tensor's current stream).
"""
from __future__ import annotations

import torch

from . import error as E
from . import ffi

_SUFFIX = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}


def _suffix(t: torch.Tensor) -> str:
    """FlashDtype dispatch (low.rs:14-134): f32 / f16 / bf16 only."""
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise E.Unsupported(f"dtype {t.dtype} (only f32/f16/bf16)") from None


def _stream_ptr(stream, ref: torch.Tensor) -> int:
    if stream is None:
        stream = torch.cuda.current_stream(ref.device)
    return int(stream.cuda_stream)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check_len(name: str, actual: int, need: int) -> None:
    """low.rs:409-416"""
    if actual >= need:
        return
    raise E.BufferTooSmall(f"{name}: need at least {need} elements, got {actual}")


def _validate(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size,
              start_pos, attn_mask) -> None:
    """low.rs:360-407 — same order, same error classes."""
    if batch <= 0 or q_seq_len <= 0 or kv_seq_len <= 0 or q_num_heads <= 0 or kv_num_heads <= 0:
        raise E.InvalidShape(
            f"batch={batch} q_seq_len={q_seq_len} kv_seq_len={kv_seq_len} "
            f"q_num_heads={q_num_heads} kv_num_heads={kv_num_heads} must be positive")
    if q_num_heads % kv_num_heads != 0:
        raise E.InvalidShape(
            f"q_num_heads={q_num_heads} must be a multiple of kv_num_heads={kv_num_heads} (GQA)")
    if start_pos < 0:
        raise E.InvalidStartPos(f"start_pos={start_pos}")
    if head_size not in (32, 64, 128):
        raise E.InvalidHeadSize(f"head_size={head_size} (only 32/64/128)")
    q_need = batch * q_seq_len * q_num_heads * head_size
    kv_need = batch * kv_seq_len * kv_num_heads * head_size
    _check_len("q", q.numel(), q_need)
    _check_len("k", k.numel(), kv_need)
    _check_len("v", v.numel(), kv_need)
    _check_len("o", o.numel(), q_need)
    if attn_mask is not None:
        _check_len("attn_mask", attn_mask.numel(), batch * kv_seq_len)


def flash_attn(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size,
               start_pos, scale, attn_mask=None, stream=None, lse=None) -> None:
    """Batched causal attention on device buffers (low.rs:146-197).

    q/o are (batch, q_seq_len, q_num_heads, head_size), k/v (batch, kv_seq_len, kv_num_heads,
    head_size), attn_mask (batch, kv_seq_len) uint8. `lse` (optional f32 buffer of
    batch*q_num_heads*q_seq_len) is this library's additive output.
    """
    _validate(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size,
              start_pos, attn_mask)
    sfx = _suffix(q)
    if lse is not None:
        _check_len("lse", lse.numel(), batch * q_num_heads * q_seq_len)
        code = getattr(ffi.lib, f"flash_attn_{sfx}_lse")(
            _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), batch, q_seq_len, kv_seq_len,
            q_num_heads, kv_num_heads, head_size, start_pos, scale, _ptr(attn_mask),
            _stream_ptr(stream, q))
    else:
        code = getattr(ffi.lib, f"flash_attn_{sfx}")(
            _ptr(q), _ptr(k), _ptr(v), _ptr(o), batch, q_seq_len, kv_seq_len, q_num_heads,
            kv_num_heads, head_size, start_pos, scale, _ptr(attn_mask), _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def flash_attn_f32(*args, **kwargs) -> None:
    """Historical alias kept by the reference (low.rs:199-218)."""
    flash_attn(*args, **kwargs)


def flash_attn_varlen(q, k, v, o, cu_seqlens_q, cu_seqlens_k, num_seqs, max_seqlen_q, max_seqlen_k,
                      q_heads, kv_heads, head_size, scale, block_tables=None, block_size=1,
                      stream=None, total_q=None, total_k=None) -> None:
    """Packed variable-length attention (low.rs:231-295). With `block_tables` the K/V are a paged
    cache and max_blocks is inferred as block_tables.numel() // num_seqs (low.rs:266-269).
    The call goes through the reference's symbol. When the caller gives the row counts of the packed
    buffers (`total_q`, and `total_k` unless paged) and the storage is 16-bit, they go along through
    the additive `flash_attn_varlen_<T>_total` entry point and bound the tensor maps as well; the
    results are bit-identical either way."""
    sfx = _suffix(q)
    k_paged = 1 if block_tables is not None else 0
    max_blocks = (block_tables.numel() // num_seqs) if (block_tables is not None and num_seqs > 0) else 0
    if sfx in ("f16", "bf16") and total_q is not None and (k_paged or total_k is not None):
        if total_k is None:
            total_k = 0
        code = getattr(ffi.lib, f"flash_attn_varlen_{sfx}_total")(
            _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(cu_seqlens_q), _ptr(cu_seqlens_k),
            _ptr(block_tables), num_seqs, max_seqlen_q, max_seqlen_k, q_heads, kv_heads, head_size,
            block_size, max_blocks, k_paged, scale, int(total_q), int(total_k), _stream_ptr(stream, q))
    else:
        code = getattr(ffi.lib, f"flash_attn_varlen_{sfx}")(
            _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(cu_seqlens_q), _ptr(cu_seqlens_k),
            _ptr(block_tables), num_seqs, max_seqlen_q, max_seqlen_k, q_heads, kv_heads, head_size,
            block_size, max_blocks, k_paged, scale, _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def flash_attn_with_kvcache(q, k_cache, v_cache, o, block_tables, context_lens, num_seqs, q_seq_len,
                            q_heads, kv_heads, head_size, block_size, max_blocks, scale,
                            stream=None) -> None:
    """Attention over a paged KV cache (low.rs:305-357): q_seq_len == 1 decodes, > 1 prefills."""
    if q_seq_len <= 0:
        raise E.InvalidShape(f"q_seq_len={q_seq_len} must be > 0")
    q_need = num_seqs * q_seq_len * q_heads * head_size
    _check_len("q", q.numel(), q_need)
    _check_len("o", o.numel(), q_need)
    sfx = _suffix(q)
    code = getattr(ffi.lib, f"flash_attn_with_kvcache_{sfx}")(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(o), _ptr(block_tables), _ptr(context_lens),
        num_seqs, q_seq_len, q_heads, kv_heads, head_size, block_size, max_blocks, scale,
        _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def debug_block_slots(block_tables, context_lens, offsets, num_seqs, block_size, max_blocks,
                      out_slots, stream=None) -> None:
    """Device-side block_slot() of every cached token, for the bit-exact page-index check."""
    code = ffi.lib.flash_attn_debug_block_slots(
        _ptr(block_tables), _ptr(context_lens), _ptr(offsets), num_seqs, block_size, max_blocks,
        _ptr(out_slots), _stream_ptr(stream, block_tables))
    E.from_status(code, ffi.last_error())


def flash_attn_allgather(q, k, v, o_peer_ptrs, q_heads_total, q_head_offset, batch, q_seq_len, kv_seq_len,
                         q_num_heads, kv_num_heads, head_size, start_pos, scale, stream=None, lse=None,
                         lse_peer_ptrs=None) -> None:
    """Head-sharded prefill whose epilogue stores this rank's heads into the full output buffer of
    every GPU of the group (`o_peer_ptrs`: device pointers, own buffer included). With
    `lse_peer_ptrs` the log-sum-exp is gathered the same way into every GPU's (batch, q_heads_total,
    q_seq_len) f32 tensor. Additive; the reference runs attention and luma-dist's all_gather as two
    separate steps."""
    import ctypes
    sfx = _suffix(q)
    if sfx == "f32":
        raise E.Unsupported("flash_attn_allgather: f16/bf16 only")
    q_need = batch * q_seq_len * q_num_heads * head_size
    kv_need = batch * kv_seq_len * kv_num_heads * head_size
    _check_len("q", q.numel(), q_need)
    _check_len("k", k.numel(), kv_need)
    _check_len("v", v.numel(), kv_need)
    n = len(o_peer_ptrs)
    arr = (ctypes.c_void_p * n)(*[int(p) for p in o_peer_ptrs])
    if lse_peer_ptrs is not None:
        if len(lse_peer_ptrs) != n:
            raise E.InvalidShape("flash_attn_allgather: lse_peer_ptrs must have one entry per output buffer")
        larr = (ctypes.c_void_p * n)(*[int(p) for p in lse_peer_ptrs])
        code = getattr(ffi.lib, f"flash_attn_{sfx}_allgather_lse")(
            _ptr(q), _ptr(k), _ptr(v), ctypes.cast(arr, ctypes.c_void_p), ctypes.cast(larr, ctypes.c_void_p), n,
            q_heads_total, q_head_offset, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos,
            scale, _stream_ptr(stream, q))
    else:
        code = getattr(ffi.lib, f"flash_attn_{sfx}_allgather")(
            _ptr(q), _ptr(k), _ptr(v), ctypes.cast(arr, ctypes.c_void_p), n, q_heads_total, q_head_offset, _ptr(lse),
            batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def flash_attn_allgather_multicast(q, k, v, o_multicast_ptr, q_heads_total, q_head_offset, batch, q_seq_len, kv_seq_len,
                                   q_num_heads, kv_num_heads, head_size, start_pos, scale, stream=None, lse=None) -> None:
    """The fused all-gather through an NVSwitch multicast address of the group's output tensors: one
    multimem.st per 16 bytes reaches every GPU's copy. Additive."""
    sfx = _suffix(q)
    if sfx == "f32":
        raise E.Unsupported("flash_attn_allgather_multicast: f16/bf16 only")
    _check_len("q", q.numel(), batch * q_seq_len * q_num_heads * head_size)
    _check_len("k", k.numel(), batch * kv_seq_len * kv_num_heads * head_size)
    _check_len("v", v.numel(), batch * kv_seq_len * kv_num_heads * head_size)
    code = getattr(ffi.lib, f"flash_attn_{sfx}_allgather_multicast")(
        _ptr(q), _ptr(k), _ptr(v), int(o_multicast_ptr), q_heads_total, q_head_offset, _ptr(lse), batch, q_seq_len, kv_seq_len,
        q_num_heads, kv_num_heads, head_size, start_pos, scale, _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def flash_attn_with_kvcache_allgather(q, k_cache, v_cache, o_peer_ptrs, q_heads_total, q_head_offset, block_tables,
                                      context_lens, num_seqs, q_heads, kv_heads, head_size, block_size, max_blocks,
                                      scale, stream=None) -> None:
    """Head-sharded single-token paged decode whose merge kernel stores this rank's heads into the
    (num_seqs, 1, q_heads_total, head_size) output of every GPU of the group. Additive."""
    import ctypes
    sfx = _suffix(q)
    if sfx == "f32":
        raise E.Unsupported("flash_attn_with_kvcache_allgather: f16/bf16 only")
    _check_len("q", q.numel(), num_seqs * q_heads * head_size)
    n = len(o_peer_ptrs)
    arr = (ctypes.c_void_p * n)(*[int(p) for p in o_peer_ptrs])
    code = getattr(ffi.lib, f"flash_attn_with_kvcache_{sfx}_allgather")(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), ctypes.cast(arr, ctypes.c_void_p), n, q_heads_total, q_head_offset,
        _ptr(block_tables), _ptr(context_lens), num_seqs, q_heads, kv_heads, head_size, block_size, max_blocks, scale,
        _stream_ptr(stream, q))
    E.from_status(code, ffi.last_error())


def kvcache_append(k_new, v_new, k_cache, v_cache, block_tables, context_lens, num_seqs, n_new, kv_heads,
                   head_size, block_size, max_blocks, stream=None) -> None:
    """Writes the K/V rows of the n_new newest tokens of every sequence into their pages
    (`context_lens` = lengths after the append). Additive: the reference leaves this to the caller
    (luma-flash-attn/src/api/high.rs:123-125)."""
    need = num_seqs * n_new * kv_heads * head_size
    _check_len("k_new", k_new.numel(), need)
    _check_len("v_new", v_new.numel(), need)
    code = ffi.lib.flash_attn_kvcache_append(
        _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(context_lens),
        num_seqs, n_new, kv_heads, head_size, k_new.element_size(), block_size, max_blocks,
        _stream_ptr(stream, k_new))
    E.from_status(code, ffi.last_error())


def softmax_last_dim(x, out=None, stream=None):
    """Softmax over the last dimension of a dense device tensor (f32 / f16 / bf16), f32 arithmetic;
    the role of luma-cuda's softmax_<T> kernels (luma-cuda/kernels/nn.cu:21-76, launched from
    luma-cuda/src/ops/nn_provide.rs:10-70) on the math path. `out` may be `x` itself."""
    if not x.is_contiguous():
        raise E.Unsupported("softmax_last_dim: the input must be contiguous (nn_provide.rs:11-13)")
    if out is None:
        out = torch.empty_like(x)
    elif tuple(out.shape) != tuple(x.shape) or out.dtype != x.dtype or not out.is_contiguous():
        raise E.InvalidShape("softmax_last_dim: out must be contiguous and shaped and typed like the input")
    n = x.shape[-1] if x.dim() > 0 else 1
    rows = x.numel() // n if n > 0 else 0
    code = getattr(ffi.lib, f"luma_softmax_{_suffix(x)}")(_ptr(x), _ptr(out), rows, n, _stream_ptr(stream, x))
    E.from_status(code, ffi.last_error())
    return out



def flash_attn_host(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                    device_index, chunk_rows=0, stream=0):
    """`flash_attn_host_<T>` of include/flash_attn.h: q/k/v/o are HOST tensors (pinned for asynchronous
    copies); the library pipelines copies and kernels over its own three streams of `device_index`."""
    sfx = _suffix(q)
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        if t.is_cuda:
            raise E.Unsupported(f"flash_attn_host: {name} must be a host tensor")
    code = getattr(ffi.lib, f"flash_attn_host_{sfx}")(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads,
        head_size, start_pos, scale, int(device_index), int(chunk_rows), int(stream))
    E.from_status(code, ffi.last_error())
