"""Multi-head self-attention module, the caller of the attention dispatcher; mirrors
luma-nn/src/modules/attention.rs:13-127.

`MultiheadAttention` owns four `(embed_dim, embed_dim)` projections (q, k, v, out) and runs
`functional.scaled_dot_product_attention` between them with the implementation its config names.
Input and output are `(batch, seq_len, embed_dim)`. The projections are plain library GEMMs
(`torch.nn.functional.linear`); the head split `(B, S, E) -> (B, S, H, E/H)` and the merge back are
views of the dense projection outputs, so the fused kernel reads and writes them without a copy.

Initialisation follows luma-nn/src/modules/common/linear.rs:25-41: Kaiming-uniform weights
(fan-in, ReLU gain: bound sqrt(6 / in_features)) and biases uniform in +-1/sqrt(in_features).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .functional import AttentionConfig, AttentionImpl, NnError, scaled_dot_product_attention


class HeadSizeCannotDivideByNumhead(NnError):
    """luma-nn/src/modules/attention.rs:74-76: embed_dim is not a multiple of num_heads."""

    def __init__(self, embed_dim: int, num_heads: int):
        super().__init__(f"embed_dim {embed_dim} cannot be divided by num_heads {num_heads}")
        self.embed_dim, self.num_heads = embed_dim, num_heads


@dataclass
class MultiheadAttentionConfig:
    """attention.rs:13-29. Defaults: bias, causal, scale 1/sqrt(head_dim), the Math implementation."""
    embed_dim: int
    num_heads: int
    bias: bool = True
    causal: bool = True
    scale: Optional[float] = None
    imp: AttentionImpl = AttentionImpl.Math


def _linear_params(in_features, out_features, bias, device, dtype):
    w = torch.empty(out_features, in_features, device=device, dtype=torch.float32)
    bound_w = math.sqrt(6.0 / in_features)            # gain sqrt(2) * sqrt(3 / fan_in)
    w.uniform_(-bound_w, bound_w)
    weight = torch.nn.Parameter(w.to(dtype))
    if not bias:
        return weight, None
    b = torch.empty(out_features, device=device, dtype=torch.float32)
    bound_b = 1.0 / math.sqrt(in_features)
    b.uniform_(-bound_b, bound_b)
    return weight, torch.nn.Parameter(b.to(dtype))


class _Linear(torch.nn.Module):
    """`input @ weight^T + bias` (linear.rs:103-106); weight `(out_features, in_features)`."""

    def __init__(self, in_features, out_features, bias, device, dtype):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight, b = _linear_params(in_features, out_features, bias, device, dtype)
        if b is None:
            self.register_parameter("bias", None)
        else:
            self.bias = b

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}"


class MultiheadAttention(torch.nn.Module):
    """attention.rs:36-127: q/k/v projections, head split, attention, head merge, output projection."""

    def __init__(self, embed_dim: int, num_heads: int, device=None, dtype=torch.float32,
                 config: Optional[MultiheadAttentionConfig] = None):
        super().__init__()
        cfg = config if config is not None else MultiheadAttentionConfig(embed_dim, num_heads)
        if cfg.num_heads == 0 or cfg.embed_dim % cfg.num_heads != 0:
            raise HeadSizeCannotDivideByNumhead(cfg.embed_dim, cfg.num_heads)
        e = cfg.embed_dim
        self.q_proj = _Linear(e, e, cfg.bias, device, dtype)
        self.k_proj = _Linear(e, e, cfg.bias, device, dtype)
        self.v_proj = _Linear(e, e, cfg.bias, device, dtype)
        self.out_proj = _Linear(e, e, cfg.bias, device, dtype)
        self.embed_dim, self.num_heads, self.head_dim = e, cfg.num_heads, e // cfg.num_heads
        self.causal, self.scale, self.imp = cfg.causal, cfg.scale, cfg.imp

    @classmethod
    def from_config(cls, config: MultiheadAttentionConfig, device=None, dtype=torch.float32):
        return cls(config.embed_dim, config.num_heads, device=device, dtype=dtype, config=config)

    def extra_repr(self):
        return f"embed_dim={self.embed_dim}, heads={self.num_heads}, causal={self.causal}"

    def forward(self, x):
        return self.forward_with_start_pos(x, 0)

    def forward_with_start_pos(self, x, start_pos: int):
        """`start_pos` is the global position of the first token of `x` (attention.rs:108-110)."""
        if x.dim() != 3:
            raise NnError(f"multihead_attention: expected a rank-3 input, got rank {x.dim()}")
        batch, seq, embed = x.shape
        if embed != self.embed_dim:
            raise NnError(f"multihead_attention: expected embed_dim {self.embed_dim}, got {embed}")
        shape = (batch, seq, self.num_heads, self.head_dim)
        q = self.q_proj(x).reshape(shape)
        k = self.k_proj(x).reshape(shape)
        v = self.v_proj(x).reshape(shape)
        cfg = AttentionConfig(self.imp, self.causal, int(start_pos), self.scale)
        out = scaled_dot_product_attention(q, k, v, cfg)
        return self.out_proj(out.contiguous().reshape(batch, seq, self.embed_dim))
