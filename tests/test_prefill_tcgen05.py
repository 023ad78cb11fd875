"""The tcgen05 prefill kernel through the C ABI against the oracle: tile-aligned and ragged
lengths, GQA widths that pair two heads per CTA and MHA that pairs two row blocks, odd groups,
start_pos that is not tile aligned, kv longer and shorter than q, LSE, f16 and bf16."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

# (batch, sq, skv, hq, hkv, start_pos)
SHAPES = [
    (1, 128, 128, 1, 1, 0),      # one tile, one CTA half empty
    (1, 256, 256, 2, 2, 0),      # MHA: two row blocks of one head share a CTA
    (2, 384, 384, 8, 2, 0),      # GQA 4: two heads of a group share a CTA
    (1, 100, 100, 4, 4, 0),      # ragged single tile
    (3, 129, 200, 6, 6, 0),      # one row into the second tile, kv longer than q
    (1, 256, 256, 6, 2, 0),      # odd group (3): pairs straddle row blocks
    (2, 50, 120, 4, 4, 70),      # start_pos not tile aligned
    (1, 300, 812, 8, 2, 512),    # chunk appended to a long prefix
    (1, 640, 640, 8, 8, 0),      # 5 row blocks: odd count, last pair half empty
    (1, 200, 150, 4, 2, 0),      # kv shorter than q: late rows see all keys
    (1, 1024, 1024, 4, 1, 0),    # several K/V ring wrap-arounds
    (1, 33, 100, 8, 4, 67),
]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(s) for s in SHAPES])
def test_prefill_matches_oracle(shape, dt):
    b, sq, skv, hq, hkv, sp = shape
    d = 128
    q = H.round_to(H.normal((b, sq, hq, d), 1 + sq), dt)
    k = H.round_to(H.normal((b, skv, hkv, d), 2 + sq), dt)
    v = H.round_to(H.normal((b, skv, hkv, d), 3 + sq), dt)
    want, lse_want = ob.attn_f64_batch(q, k, v, start_pos=sp, return_lse=True)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    o = torch.full_like(qd, float("nan"))
    lse = torch.full((b, hq, sq), float("nan"), device="cuda", dtype=torch.float32)
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), None, None, lse)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"prefill {shape} {dt}")
    np.testing.assert_allclose(lse.cpu().numpy(), lse_want, rtol=0, atol=1e-3)


def test_prefill_matches_luma_cpu_math_path_config1_style():
    # BASELINE config 1 layout (B=1, H=8, S=256, seed 0) at head size 128: compared with the f32
    # restatement of luma-cpu's math path, the oracle north_star names
    b, s, h, d = 1, 256, 8, 128
    q = H.round_to(H.normal((b, s, h, d), 0), "bf16")
    k = H.round_to(H.normal((b, s, h, d), 100), "bf16")
    v = H.round_to(H.normal((b, s, h, d), 200), "bf16")
    want = ob.sdpa_math_f32(q, k, v, causal=True)
    o = torch.empty(b, s, h, d, device="cuda", dtype=torch.bfloat16)
    low.flash_attn(H.to_dev(q, "bf16"), H.to_dev(k, "bf16"), H.to_dev(v, "bf16"), o, b, s, s, h, h, d, 0, 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    H.assert_bf16_close(H.to_np(o), want, "config-1 style vs math path")


def test_prefill_large_logits_and_custom_scale():
    # large-magnitude scores exercise the lazy rescale (row max moves by far more than 2^8)
    b, s, hq, hkv, d = 1, 512, 4, 2, 128
    q = H.round_to(H.normal((b, s, hq, d), 7, 3.0), "bf16")
    k = H.round_to(H.normal((b, s, hkv, d), 8, 3.0), "bf16")
    v = H.round_to(H.normal((b, s, hkv, d), 9), "bf16")
    want = ob.attn_f64_batch(q, k, v, scale=0.5)
    o = torch.empty(b, s, hq, d, device="cuda", dtype=torch.bfloat16)
    low.flash_attn(H.to_dev(q, "bf16"), H.to_dev(k, "bf16"), H.to_dev(v, "bf16"), o, b, s, s, hq, hkv, d, 0, 0.5)
    torch.cuda.synchronize()
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, "large logits")


def test_prefill_agrees_with_simt_kernel():
    b, s, hq, hkv, d = 2, 700, 8, 4, 128
    q, k, v = (H.to_dev(H.normal(sh, sd), "bf16") for sh, sd in
               (((b, s, hq, d), 31), ((b, s, hkv, d), 32), ((b, s, hkv, d), 33)))
    fast, slow = torch.empty_like(q), torch.empty_like(q)
    low.flash_attn(q, k, v, fast, b, s, s, hq, hkv, d, 0, 0.088)
    assert ffi.last_path() == "prefill_tcgen05"
    ffi.set_option("force_generic", 1)
    try:
        low.flash_attn(q, k, v, slow, b, s, s, hq, hkv, d, 0, 0.088)
        assert ffi.last_path() == "tile_simt"
    finally:
        ffi.set_option("force_generic", 0)
    torch.cuda.synchronize()
    assert (fast.float() - slow.float()).abs().max().item() <= 2e-2
