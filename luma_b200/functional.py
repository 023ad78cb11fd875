"""The attention dispatcher one level above the flash-attention crate; mirrors
luma-nn/src/functional/attention.rs:13-117.

`scaled_dot_product_attention(q, k, v, cfg)` picks the implementation the caller names in
`AttentionConfig.imp` — there is deliberately no automatic choice (attention.rs:8-18):

* `AttentionImpl.Math`  : the device's provider. On host tensors the portable path built from core
  tensor ops (expand the KV heads, QK^T, scale, causal mask by global position, softmax, PV —
  luma-tensor/src/ops/nn/attention.rs:11-45), differentiable; it is the cross-check of the fused
  path, as in the reference's own tests (luma-nn/tests/attention.rs:190-235). On CUDA tensors the
  backend's override (`cuda_provide`), which takes the fused kernel for causal inference calls and the
  same composed path otherwise.
* `AttentionImpl.Flash` : the fused kernel behind `high.flash_attn_func`; CUDA tensors only, causal
  only, forward only — the same three guards, in the same order of concern, as attention.rs:76-100,
  and the library's errors come back as `FlashAttentionUnsupported` (attention.rs:110-117).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, replace
from typing import Optional

import torch

from . import error as E


class NnError(Exception):
    """luma-nn/src/error.rs: the user-facing error of the nn layer."""


class FlashAttentionRequiresCuda(NnError):
    def __init__(self):
        super().__init__("flash attention requires a CUDA device")


class FlashAttentionUnsupported(NnError):
    pass


class AttentionImpl(enum.Enum):
    Math = "math"
    Flash = "flash"


@dataclass(frozen=True)
class AttentionConfig:
    """attention.rs:20-55. `scale=None` means 1/sqrt(head_size); `start_pos` is the global position
    of the first query token."""
    imp: AttentionImpl = AttentionImpl.Math
    causal: bool = True
    start_pos: int = 0
    scale: Optional[float] = None

    @staticmethod
    def math() -> "AttentionConfig":
        return AttentionConfig(AttentionImpl.Math, True, 0, None)

    @staticmethod
    def flash() -> "AttentionConfig":
        return AttentionConfig(AttentionImpl.Flash, True, 0, None)

    def with_causal(self, causal: bool) -> "AttentionConfig":
        return replace(self, causal=bool(causal))

    def with_start_pos(self, start_pos: int) -> "AttentionConfig":
        return replace(self, start_pos=int(start_pos))

    def with_scale(self, scale: float) -> "AttentionConfig":
        return replace(self, scale=float(scale))


def _math_path(q, k, v, scale, causal, start_pos):
    """AttentionImpl.Math: the provider's scaled_dot_product_attention of the tensors' device
    (attention.rs:60-73 -> luma-tensor/src/device/nn_provide.rs:139-150). On host tensors that is the
    composed default (luma-tensor/src/ops/nn/attention.rs:11-45,95-127); on CUDA tensors it is the
    backend's override, which sends causal inference calls to the fused kernel and everything else —
    gradients required, non-causal, other head sizes — to the same composed default."""
    from . import cuda_provide
    if q.is_cuda:
        return cuda_provide.scaled_dot_product_attention(q, k, v, scale, causal, start_pos)
    return cuda_provide.composed_default(q, k, v, scale, causal, start_pos)


def scaled_dot_product_attention(q, k, v, cfg: AttentionConfig):
    """Attention(Q, K, V) = softmax(Q K^T * scale) V; q (B, Sq, Hq, d), k/v (B, Skv, Hkv, d) ->
    (B, Sq, Hq, d). The implementation is the one `cfg.imp` names (attention.rs:57-104)."""
    if cfg.imp is AttentionImpl.Math:
        return _math_path(q, k, v, cfg.scale, cfg.causal, cfg.start_pos)
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise FlashAttentionRequiresCuda()
    if not cfg.causal:
        raise FlashAttentionUnsupported("flash attention supports causal=True only")
    # the backward of the fused kernel does not exist: refuse before running anything (attention.rs:84-92)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        raise FlashAttentionUnsupported("flash attention has no backward yet; train with AttentionConfig.math()")
    from . import high   # the compiled library is only needed on this path
    try:
        return high.flash_attn_func(q, k, v, cfg.scale, True, cfg.start_pos)
    except E.FlashAttnError as exc:   # map_flash_error (attention.rs:110-117)
        raise FlashAttentionUnsupported(str(exc)) from exc
