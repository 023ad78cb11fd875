"""The CUDA backend's override of the nn provider for attention: what one more method in
`impl NnProvide<Cuda> for Cuda` (luma-cuda/src/ops/nn_provide.rs:147-174, beside `softmax` and
`rms_norm`) does for the trait's `scaled_dot_product_attention`
(luma-tensor/src/device/nn_provide.rs:139-150), whose default is the composed
`NnOpDefault::scaled_dot_product_attention_forward` (luma-tensor/src/ops/nn/attention.rs:11-45).

The override follows the pattern of its two neighbours — take the fused kernel where it covers
the call, otherwise return the composed default — with the guards the fused kernel needs
(luma-nn/src/functional/attention.rs:76-100): causal, no gradient required, head size 32 / 64 / 128,
f32 / f16 / bf16 storage, rank-4 tensors of matching shapes on a CUDA device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import error as E

FUSED_HEAD_SIZES = (32, 64, 128)
FUSED_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def takes_fused_kernel(q, k, v, causal: bool) -> bool:
    """The routing rule: True when the call goes to the fused kernel."""
    if not causal:
        return False
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        return False
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        return False
    if q.dtype not in FUSED_DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return False          # the fused kernel has no backward (luma-flash-attn/src/api/high.rs:280-289)
    b, _sq, hq, d = q.shape
    if d not in FUSED_HEAD_SIZES:
        return False
    if tuple(v.shape) != tuple(k.shape) or k.shape[0] != b or k.shape[3] != d or k.shape[2] <= 0 or hq % k.shape[2] != 0:
        return False          # let the composed path raise its own shape error
    return True


def composed_default(q, k, v, scale: Optional[float], causal: bool, start_pos: int):
    """NnOpDefault::scaled_dot_product_attention_forward on torch tensors: expand the KV heads, Q K^T,
    scale, causal mask by global position, softmax, P V; f32 math, output in q's dtype; differentiable.
    On a CUDA device without autograd the row softmax is this library's kernel (the reference's CUDA
    math path runs luma-cuda's softmax there)."""
    from .functional import NnError
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise NnError("scaled_dot_product_attention: q/k/v must be rank 4 (batch, seq, heads, head_size)")
    b, sq, hq, d = q.shape
    bk, skv, hkv, dk = k.shape
    if tuple(v.shape) != tuple(k.shape) or bk != b or dk != d or hkv <= 0 or hq % hkv != 0:
        raise NnError(f"scaled_dot_product_attention: incompatible shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
    s = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    group = hq // hkv
    qf = q.float().permute(0, 2, 1, 3)                                   # (B, Hq, Sq, d)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)   # expand_heads (attention.rs:95-110)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * s
    if causal:
        gpos = torch.arange(sq, device=q.device).unsqueeze(1) + int(start_pos)   # causal_mask (attention.rs:112-127)
        keys = torch.arange(skv, device=q.device).unsqueeze(0)
        scores = scores.masked_fill(keys > gpos, float("-inf"))
    if scores.is_cuda and not (torch.is_grad_enabled() and scores.requires_grad):
        from . import low
        probs = low.softmax_last_dim(scores.contiguous(), out=None)
    else:
        probs = torch.softmax(scores, dim=-1)
    out = torch.matmul(probs, vf).permute(0, 2, 1, 3)
    return out.to(q.dtype).contiguous()


def scaled_dot_product_attention(q, k, v, scale: Optional[float] = None, causal: bool = True, start_pos: int = 0):
    """NnProvide<Cuda>::scaled_dot_product_attention: the fused kernel where it covers the call, the
    composed default otherwise. q (B, Sq, Hq, d), k/v (B, Skv, Hkv, d) -> (B, Sq, Hq, d)."""
    if takes_fused_kernel(q, k, v, causal):
        from . import high
        d = q.shape[3]
        s = float(scale) if scale is not None else 1.0 / math.sqrt(d)
        if s > 0.0:   # the kernels fold the scale into the exponent's base and need it positive
            try:
                return high.flash_attn_func(q, k, v, s, True, int(start_pos))
            except E.Unsupported:
                pass
    return composed_default(q, k, v, scale, causal, start_pos)
