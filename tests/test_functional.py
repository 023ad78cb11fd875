"""The Math / Flash dispatcher (luma-nn/src/functional/attention.rs): the Math path against the f64
oracle on the reference's CPU-runnable case and with GQA / start_pos (CPU), the Flash guards, and on
a GPU Flash against Math against the oracle at the reference's tolerance (luma-nn/tests/attention.rs:190-235)."""
import numpy as np
import pytest
import torch

from luma_b200 import cuda_provide
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
    # the composed path itself (what Math runs wherever the fused kernel does not cover the call): the independent cross-check
    mathp = cuda_provide.composed_default(qd, kd, vd, None, True, sp)
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


@pytest.mark.gpu
def test_math_on_cuda_routes_inference_to_the_fused_kernel():
    """The CUDA backend's provider override (luma-cuda/src/ops/nn_provide.rs:147-174 with one more
    method): Math on CUDA tensors takes the fused kernel for causal inference calls and the composed
    path otherwise, and both agree with the oracle."""
    from luma_b200 import ffi, low
    b, sq, skv, hq, hkv, d, sp = 2, 200, 264, 8, 2, 128, 64
    q, k, v = (H.round_to(t, "bf16") for t in _case(b, sq, skv, hq, hkv, d, 19))
    want = ob.attn_f64_batch(q, k, v, start_pos=sp)
    qd, kd, vd = (H.to_dev(t, "bf16") for t in (q, k, v))
    cfg = F.AttentionConfig.math().with_start_pos(sp)

    def reset_path():   # any other library call, so that last_path() tells what the next call did
        low.softmax_last_dim(torch.zeros(2, 8, device="cuda"))
        assert ffi.last_path() != "prefill_tcgen05"

    reset_path()
    out = F.scaled_dot_product_attention(qd, kd, vd, cfg)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(out), want, "Math on CUDA, inference")
    # gradients required: the composed path, differentiable, same values
    reset_path()
    qg = qd.clone().requires_grad_(True)
    out_g = F.scaled_dot_product_attention(qg, kd, vd, cfg)
    assert ffi.last_path() != "prefill_tcgen05" and out_g.requires_grad
    out_g.float().sum().backward()
    assert qg.grad is not None and bool(torch.isfinite(qg.grad.float()).all())
    H.assert_bf16_close(H.to_np(out_g), want, "Math on CUDA, with autograd")
    with torch.no_grad():   # the same tensors with autograd off: fused again
        F.scaled_dot_product_attention(qg, kd, vd, cfg)
        assert ffi.last_path() == "prefill_tcgen05"
    # non-causal and a head size the kernel does not have: composed path
    reset_path()
    nc = F.scaled_dot_product_attention(qd, kd, vd, F.AttentionConfig.math().with_causal(False))
    assert ffi.last_path() != "prefill_tcgen05" and tuple(nc.shape) == (b, sq, hq, d)
    q48, k48, v48 = (t[..., :48].contiguous() for t in (qd, kd, vd))
    o48 = F.scaled_dot_product_attention(q48, k48, v48, cfg)
    assert ffi.last_path() != "prefill_tcgen05"
    want48 = ob.attn_f64_batch(q[..., :48].copy(), k[..., :48].copy(), v[..., :48].copy(), start_pos=sp)
    H.assert_bf16_close(H.to_np(o48), want48, "head size 48 on the composed path")
    assert cuda_provide.takes_fused_kernel(qd, kd, vd, True) and not cuda_provide.takes_fused_kernel(qd, kd, vd, False)
    assert not cuda_provide.takes_fused_kernel(q48, k48, v48, True)


def test_provider_routing_rule_on_cpu():
    q = torch.zeros(1, 4, 2, 64)
    assert not cuda_provide.takes_fused_kernel(q, q, q, True)        # host tensors never take the fused kernel
    out = F.scaled_dot_product_attention(q, q, q, F.AttentionConfig.math())
    assert tuple(out.shape) == (1, 4, 2, 64)
