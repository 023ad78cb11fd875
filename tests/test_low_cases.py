"""C-ABI numeric cases of the reference's low-level suite (luma-flash-attn/tests/low.rs:201-265),
same shapes, seeds, generator and tolerance, for every storage type, on every kernel family."""
import numpy as np
import pytest
import torch

import luma_b200 as L
from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

# (seed, batch, sq, skv, hq, hkv, d, start_pos, mask)
CASES = [
    (1, 2, 64, 64, 4, 4, 32, 0, None),       # mha_head32_exact_tiles
    (2, 1, 100, 100, 4, 4, 64, 0, None),     # mha_head64_unaligned_seq
    (3, 3, 129, 200, 6, 6, 32, 0, None),     # mha_head32_uneven_seq
    (4, 2, 70, 70, 8, 2, 128, 0, None),      # gqa_head128
    (5, 1, 32, 32, 1, 1, 64, 0, None),       # causal_zero_start_pos
    (6, 2, 128, 128, 4, 4, 32, 0, "random"),  # mask_random_padding
    (7, 1, 64, 64, 2, 2, 64, 0, "ones"),     # mask_all_ones_equals_no_mask
    (8, 1, 40, 72, 8, 2, 64, 32, None),      # kv_cache_start_pos_offset
    (9, 2, 50, 120, 4, 4, 32, 70, None),     # start_pos_unaligned_to_block
    (10, 2, 33, 100, 8, 4, 128, 67, "random"),  # gqa_mask_with_start_pos
    (11, 1, 1, 96, 4, 4, 64, 95, None),      # single_token_decode
]


def _inputs(seed, b, sq, skv, hq, hkv, d, mask_kind):
    rng = ob.XorShift(seed)  # one stream: q, k, v, then the mask (tests/low.rs:148-152)
    q = rng.f32(b * sq * hq * d).reshape(b, sq, hq, d)
    k = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    v = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    mask = None
    if mask_kind == "ones":
        mask = np.ones((b, skv), dtype=np.uint8)
    elif mask_kind == "random":
        mask = (rng.f32(b * skv) > -0.2).astype(np.uint8).reshape(b, skv)
    return q, k, v, mask


@pytest.mark.parametrize("dt,tol", [("f32", H.F32_TOL), ("f16", H.F16_TOL), ("bf16", H.BF16_REF_TOL)])
@pytest.mark.parametrize("case", CASES, ids=[f"seed{c[0]}" for c in CASES])
def test_low_numeric_cases(case, dt, tol):
    seed, b, sq, skv, hq, hkv, d, sp, mask_kind = case
    q, k, v, mask = _inputs(seed, b, sq, skv, hq, hkv, d, mask_kind)
    q, k, v = H.round_to(q, dt), H.round_to(k, dt), H.round_to(v, dt)
    want = ob.attn_f64_batch(q, k, v, start_pos=sp, mask=mask)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    md = None if mask is None else torch.from_numpy(mask).cuda()
    o = torch.full_like(qd, float("nan"))  # the op must overwrite every element
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), md)
    torch.cuda.synchronize()
    H.assert_ref_close(H.to_np(o), want, tol, f"{dt} case seed={seed} path={ffi.last_path()}")


def test_all_ones_mask_equals_no_mask():
    seed, b, sq, skv, hq, hkv, d, sp, _ = CASES[6]
    q, k, v, _ = _inputs(seed, b, sq, skv, hq, hkv, d, None)
    qd, kd, vd = H.to_dev(q, "f32"), H.to_dev(k, "f32"), H.to_dev(v, "f32")
    a = torch.empty_like(qd)
    c = torch.empty_like(qd)
    low.flash_attn(qd, kd, vd, a, b, sq, skv, hq, hkv, d, sp, 0.125)
    low.flash_attn(qd, kd, vd, c, b, sq, skv, hq, hkv, d, sp, 0.125, torch.ones(b, skv, dtype=torch.uint8, device="cuda"))
    torch.cuda.synchronize()
    H.assert_ref_close(H.to_np(c), H.to_np(a), H.F32_TOL, "all-ones mask")


def test_null_pointer_from_c_abi_with_live_stream():
    # tests/low.rs:329-358
    stream = torch.cuda.current_stream().cuda_stream
    code = ffi.lib.flash_attn_f32(None, None, None, None, 1, 1, 1, 1, 1, 32, 0, 1.0, None, stream)
    assert code == 1
    assert ffi.last_error() != ""
    with pytest.raises(L.NullPtr):
        from luma_b200.error import from_status
        from_status(code, ffi.last_error())


def test_lse_output_f32():
    rng = ob.XorShift(21)
    b, sq, skv, hq, hkv, d, sp = 2, 37, 53, 4, 2, 64, 16
    q = rng.f32(b * sq * hq * d).reshape(b, sq, hq, d)
    k = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    v = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    want, lse_want = ob.attn_f64_batch(q, k, v, start_pos=sp, return_lse=True)
    qd, kd, vd = H.to_dev(q, "f32"), H.to_dev(k, "f32"), H.to_dev(v, "f32")
    o = torch.empty_like(qd)
    lse = torch.empty(b, hq, sq, device="cuda", dtype=torch.float32)
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), None, None, lse)
    torch.cuda.synchronize()
    H.assert_ref_close(H.to_np(o), want, H.F32_TOL, "lse variant output")
    np.testing.assert_allclose(lse.cpu().numpy(), lse_want, rtol=0, atol=1e-3)
