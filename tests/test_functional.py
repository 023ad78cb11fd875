"""The Math / Flash dispatcher (luma-nn/src/functional/attention.rs): the Math path against the f64
oracle on the reference's CPU-runnable case and with GQA / start_pos (CPU), the Flash guards, and on
a GPU Flash against Math against the oracle at the reference's tolerance (luma-nn/tests/attention.rs:190-235)."""
import numpy as np
import pytest
import torch

from luma_b200 import functional as F
from oracle import binding as ob
from tests import helpers as H


def _case(b, sq, skv, hq, hkv, d, seed):
    q = H.normal((b, sq, hq, d), seed)
    k = H.normal((b, skv, hkv, d), seed + 1)
    v = H.normal((b, skv, hkv, d), seed + 2)
    return q, k, v


@pytest.mark.parametrize("shape", [(1, 256, 256, 8, 8, 64, 0), (2, 17, 40, 6, 2, 32, 23), (1, 5, 5, 4, 1, 128, 0)])
def test_math_path_matches_oracle_cpu(shape):
    b, sq, skv, hq, hkv, d, sp = shape
    q, k, v = _case(b, sq, skv, hq, hkv, d, 3)
    want = ob.attn_f64_batch(q, k, v, start_pos=sp)
    cfg = F.AttentionConfig.math().with_start_pos(sp)
    got = F.scaled_dot_product_attention(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), cfg)
    assert got.is_contiguous() and tuple(got.shape) == (b, sq, hq, d)
    np.testing.assert_allclose(got.numpy(), want, rtol=0, atol=1e-4)   # luma-nn/tests/attention.rs:100-128


def test_config_builders_and_flash_guards_cpu():
    cfg = F.AttentionConfig.flash().with_scale(0.25).with_start_pos(3)
    assert cfg.imp is F.AttentionImpl.Flash and cfg.causal and cfg.start_pos == 3 and cfg.scale == 0.25
    assert F.AttentionConfig.math().imp is F.AttentionImpl.Math
    q = torch.zeros(1, 4, 2, 32)
    with pytest.raises(F.FlashAttentionRequiresCuda):
        F.scaled_dot_product_attention(q, q, q, F.AttentionConfig.flash())
    # the Math path is differentiable
    qg = torch.randn(1, 4, 2, 32, requires_grad=True)
    F.scaled_dot_product_attention(qg, qg, qg, F.AttentionConfig.math()).sum().backward()
    assert qg.grad is not None
    with pytest.raises(F.NnError):
        F.scaled_dot_product_attention(q, q[:, :, :1], q, F.AttentionConfig.math())


@pytest.mark.gpu
def test_flash_against_math_against_oracle_gpu():
    b, sq, skv, hq, hkv, d, sp = 2, 200, 264, 8, 2, 128, 64
    q, k, v = _case(b, sq, skv, hq, hkv, d, 9)
    want = ob.attn_f64_batch(q, k, v, start_pos=sp)
    qd, kd, vd = (torch.from_numpy(t).cuda() for t in (q, k, v))
    flash = F.scaled_dot_product_attention(qd, kd, vd, F.AttentionConfig.flash().with_start_pos(sp))
    mathp = F.scaled_dot_product_attention(qd, kd, vd, F.AttentionConfig.math().with_start_pos(sp))
    np.testing.assert_allclose(flash.cpu().numpy(), want, rtol=0, atol=3e-3)
    np.testing.assert_allclose(mathp.cpu().numpy(), want, rtol=0, atol=3e-3)
    np.testing.assert_allclose(flash.cpu().numpy(), mathp.cpu().numpy(), rtol=0, atol=3e-3)
    with pytest.raises(F.FlashAttentionUnsupported):
        F.scaled_dot_product_attention(qd, kd, vd, F.AttentionConfig.flash().with_causal(False))
    qg = qd.clone().requires_grad_(True)
    with pytest.raises(F.FlashAttentionUnsupported):
        F.scaled_dot_product_attention(qg, kd, vd, F.AttentionConfig.flash())
    with torch.no_grad():   # grad disabled: allowed, as in the reference
        F.scaled_dot_product_attention(qg, kd, vd, F.AttentionConfig.flash())
    with pytest.raises(F.FlashAttentionUnsupported):   # the library's own error comes back mapped
        F.scaled_dot_product_attention(qd[..., :48].contiguous(), kd[..., :48].contiguous(), vd[..., :48].contiguous(),
                                       F.AttentionConfig.flash())
