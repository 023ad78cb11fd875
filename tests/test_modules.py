"""The multi-head attention module (luma-nn/src/modules/attention.rs); the CPU cases follow
luma-nn/tests/modules.rs:45-59, the GPU case checks the module's Flash configuration against its
Math configuration with the same weights (as luma-nn/tests/attention.rs:190-235 does one level down)."""
import math

import pytest
import torch

from luma_b200 import functional as F
from luma_b200 import modules as M


def _ramp(b, s, e):
    # the reference test's input: ((i % 7) - 3) / 7
    return ((torch.arange(b * s * e) % 7).float() - 3.0).div(7.0).reshape(b, s, e)


def test_module_forward_shapes_and_start_pos_zero():
    torch.manual_seed(0)
    cfg = M.MultiheadAttentionConfig(4, 2, bias=False, causal=False)
    attn = M.MultiheadAttention.from_config(cfg)
    x = _ramp(2, 3, 4)
    y = attn(x)
    assert tuple(y.shape) == (2, 3, 4) and torch.isfinite(y).all()
    assert torch.allclose(y, attn.forward_with_start_pos(x, 0), rtol=1e-6, atol=1e-6)
    assert attn.q_proj.bias is None and attn.head_dim == 2
    assert "embed_dim=4, heads=2, causal=False" in repr(attn)


def test_module_matches_manual_composition():
    torch.manual_seed(1)
    attn = M.MultiheadAttention(8, 2)          # defaults: bias, causal, Math
    x = torch.randn(2, 5, 8)
    y = attn(x)
    q = (x @ attn.q_proj.weight.T + attn.q_proj.bias).reshape(2, 5, 2, 4).permute(0, 2, 1, 3)
    k = (x @ attn.k_proj.weight.T + attn.k_proj.bias).reshape(2, 5, 2, 4).permute(0, 2, 1, 3)
    v = (x @ attn.v_proj.weight.T + attn.v_proj.bias).reshape(2, 5, 2, 4).permute(0, 2, 1, 3)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(4)
    s = s.masked_fill(torch.triu(torch.ones(5, 5, dtype=torch.bool), 1), float("-inf"))
    o = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(2, 5, 8)
    want = o @ attn.out_proj.weight.T + attn.out_proj.bias
    assert torch.allclose(y, want, rtol=1e-5, atol=1e-6)
    # gradients reach every projection on the Math path
    y.sum().backward()
    for p in attn.parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all()


def test_module_init_bounds_and_errors():
    torch.manual_seed(2)
    attn = M.MultiheadAttention(64, 4)
    assert attn.q_proj.weight.abs().max().item() <= math.sqrt(6.0 / 64)
    assert attn.q_proj.bias.abs().max().item() <= 1.0 / 8
    with pytest.raises(M.HeadSizeCannotDivideByNumhead):
        M.MultiheadAttention(10, 4)
    with pytest.raises(M.HeadSizeCannotDivideByNumhead):
        M.MultiheadAttention(8, 0)
    with pytest.raises(F.NnError):
        attn(torch.zeros(1, 3, 32))
    flash = M.MultiheadAttention.from_config(M.MultiheadAttentionConfig(64, 2, imp=F.AttentionImpl.Flash))
    with pytest.raises(F.FlashAttentionRequiresCuda):
        flash(torch.zeros(1, 4, 64))


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,seq,start_pos", [(128, 300, 0), (64, 257, 0), (32, 40, 7)])
def test_module_flash_matches_math_on_gpu(head_dim, seq, start_pos):
    from luma_b200 import ffi
    torch.manual_seed(3)
    heads = 4
    e = heads * head_dim
    cfg = M.MultiheadAttentionConfig(e, heads, imp=F.AttentionImpl.Flash)
    flash = M.MultiheadAttention.from_config(cfg, device="cuda", dtype=torch.bfloat16)
    mathm = M.MultiheadAttention.from_config(M.MultiheadAttentionConfig(e, heads), device="cuda", dtype=torch.bfloat16)
    mathm.load_state_dict(flash.state_dict())
    x = torch.randn(2, seq, e, device="cuda").bfloat16()
    with torch.no_grad():
        yf = flash.forward_with_start_pos(x, start_pos)
        path = ffi.last_path()
        ym = mathm.forward_with_start_pos(x, start_pos)
    assert path in ("prefill_tcgen05", "tile_simt")
    if head_dim in (64, 128) and start_pos == 0:
        assert path == "prefill_tcgen05"
    # the attention outputs agree to the fused kernel's bar (max-abs 2e-2, mean-abs 2e-3 at unit scale);
    # the output projection then rounds to bf16 at the magnitude of its results, so the bar scales with it
    scale = max(1.0, ym.float().abs().max().item())
    err = (yf.float() - ym.float()).abs()
    assert err.max().item() <= 2e-2 * scale and err.mean().item() <= 2e-3 * scale
    # with autograd on and parameters requiring grad, the Flash configuration refuses (no backward)
    with pytest.raises(F.FlashAttentionUnsupported):
        flash(x)
