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
    # the CPU-runnable case's layout (B=1, H=8, S=256, seed 0) at head size 128: compared with the f32
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


D64_SHAPES = [(1, 128, 128, 2, 2, 0), (2, 300, 300, 8, 2, 0), (1, 129, 200, 6, 6, 0), (2, 50, 120, 4, 4, 70),
              (1, 640, 640, 3, 3, 0), (1, 1024, 1024, 4, 1, 128)]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", D64_SHAPES, ids=[str(s) for s in D64_SHAPES])
def test_prefill_head_size_64(shape, dt):
    """head_size 64 runs on the same kernel (one 64-column half per tile, N = 64 for P.V)."""
    b, sq, skv, hq, hkv, sp = shape
    d = 64
    q = H.round_to(H.normal((b, sq, hq, d), 41 + sq), dt)
    k = H.round_to(H.normal((b, skv, hkv, d), 42 + sq), dt)
    v = H.round_to(H.normal((b, skv, hkv, d), 43 + sq), dt)
    want, lse_want = ob.attn_f64_batch(q, k, v, start_pos=sp, return_lse=True)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    o = torch.full_like(qd, float("nan"))
    lse = torch.full((b, hq, sq), float("nan"), device="cuda", dtype=torch.float32)
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), None, None, lse)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"prefill d=64 {shape} {dt}")
    np.testing.assert_allclose(lse.cpu().numpy(), lse_want, rtol=0, atol=1e-3)


def test_varlen_and_paged_head_size_64():
    dt, d = "bf16", 64
    ql, kl, hq, hkv = [100, 37, 260], [100, 37, 260], 4, 2
    cu = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    tq = int(cu[-1])
    q = H.round_to(H.normal((tq, hq, d), 51), dt)
    k = H.round_to(H.normal((tq, hkv, d), 52), dt)
    v = H.round_to(H.normal((tq, hkv, d), 53), dt)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    o = torch.full_like(qd, float("nan"))
    c = torch.from_numpy(cu).cuda()
    low.flash_attn_varlen(qd, kd, vd, o, c, c, len(ql), max(ql), max(kl), hq, hkv, d, 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), ob.attn_f64_varlen(q, k, v, cu, cu), "varlen d=64")

    # chunked prefill over a paged cache, page size 16
    bs, lens, sq = 16, np.array([300, 1000], dtype=np.int32), 64
    need = (lens + bs - 1) // bs
    rng = np.random.Generator(np.random.Philox(9))
    nblocks = int(need.sum()) + 2
    perm = rng.permutation(nblocks).astype(np.int32)
    table = np.zeros((2, int(need.max()) + 1), dtype=np.int32)
    pos = 0
    for s_, n in enumerate(need):
        table[s_, :n] = perm[pos:pos + n]
        pos += int(n)
    kc = H.round_to(H.normal((nblocks, bs, hkv, d), 54), dt)
    vc = H.round_to(H.normal((nblocks, bs, hkv, d), 55), dt)
    q2 = H.round_to(H.normal((2, sq, hq, d), 56), dt)
    o2 = torch.full((2, sq, hq, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn_with_kvcache(H.to_dev(q2, dt), H.to_dev(kc, dt), H.to_dev(vc, dt), o2, torch.from_numpy(table).cuda(),
                                torch.from_numpy(lens).cuda(), 2, sq, hq, hkv, d, bs, table.shape[1], 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o2), ob.attn_f64_kvcache(q2, kc, vc, lens, table), "paged prefill d=64")


@pytest.mark.parametrize("kind", ["right_padding", "left_padding", "random", "all_ones", "one_row_all_masked"])
@pytest.mark.parametrize("shape", [(2, 300, 300, 4, 2, 128, 0), (3, 130, 515, 6, 2, 64, 385), (1, 1024, 1024, 2, 2, 128, 0)])
def test_key_padding_mask_on_the_tensor_core_kernel(kind, shape):
    """The (batch, kv_seq_len) padding mask of the batched entry point (flash_attn_func.cu:96-104,
    1 = valid key): tiles whose keys are all valid run unmasked, mixed tiles apply the bits, rows left
    without any visible key output zeros."""
    b, sq, skv, hq, hkv, d, sp = shape
    rng = np.random.Generator(np.random.Philox(sum(map(ord, kind)) + sq))
    mask = np.ones((b, skv), dtype=np.uint8)
    if kind == "right_padding":
        for i in range(b):
            mask[i, rng.integers(1, skv):] = 0
    elif kind == "left_padding":
        for i in range(b):
            mask[i, :rng.integers(1, skv - 1)] = 0
    elif kind == "random":
        mask = (rng.random((b, skv)) > 0.3).astype(np.uint8)
    elif kind == "one_row_all_masked":
        mask[0, :] = 0
    q = H.round_to(H.normal((b, sq, hq, d), 81), "bf16")
    k = H.round_to(H.normal((b, skv, hkv, d), 82), "bf16")
    v = H.round_to(H.normal((b, skv, hkv, d), 83), "bf16")
    want = ob.attn_f64_batch(q, k, v, start_pos=sp, mask=mask)
    qd = H.to_dev(q, "bf16")
    o = torch.full_like(qd, float("nan"))
    low.flash_attn(qd, H.to_dev(k, "bf16"), H.to_dev(v, "bf16"), o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d),
                   torch.from_numpy(mask).cuda())
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    got = H.to_np(o)
    assert np.isfinite(got).all()
    H.assert_bf16_close(got, want, f"padding mask {kind} {shape}")
    if kind == "one_row_all_masked":
        assert np.all(got[0] == 0.0)
