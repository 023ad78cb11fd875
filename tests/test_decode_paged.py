"""Paged single-token decode through the C ABI against the oracle: permuted block tables, ragged
and empty contexts, every GQA group width, page sizes that are not powers of two, and the
bit-exact check of the page-index arithmetic."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _run_decode(lens, hq, hkv, d, bs, dt, seed, scale=None, poison=True, chunk=0):
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=seed)
    kc, vc = H.round_to(kc, dt), H.round_to(vc, dt)
    q = H.round_to(H.normal((len(lens), 1, hq, d), seed + 3), dt)
    scale = scale if scale is not None else 1.0 / np.sqrt(d)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan")) if poison else torch.empty_like(qd)
    ffi.set_option("decode_chunk_tokens", chunk)
    try:
        low.flash_attn_with_kvcache(qd, H.to_dev(kc, dt), H.to_dev(vc, dt), o, torch.from_numpy(table).cuda(),
                                    torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 1, hq, hkv, d,
                                    bs, table.shape[1], scale)
        torch.cuda.synchronize()
    finally:
        ffi.set_option("decode_chunk_tokens", 0)
    path = ffi.last_path()
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table, scale=scale)
    return H.to_np(o), want, path


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("hq,hkv,d,bs", [
    (32, 8, 128, 16),   # the head layout of the batch-64 decode benchmark (Hq=32, Hkv=8, d=128, page 16)
    (64, 8, 128, 16),   # the head layout of the batch-256 decode benchmark (group 8)
    (8, 8, 128, 16),    # MHA
    (16, 1, 64, 16),    # group 16, d=64
    (40, 1, 128, 8),    # group 40 > 16: several head blocks per KV head
    (6, 2, 128, 5),     # page size not a power of two
    (4, 2, 64, 1),      # one token per page
    (4, 4, 128, 32),
    (8, 2, 32, 16),     # head size 32 (rows of four 16-byte chunks)
    (12, 1, 32, 8),
])
def test_decode_matches_oracle(hq, hkv, d, bs, dt):
    lens = [1, 15, 16, 17, 64, 100, 513, 777, 1500]
    got, want, path = _run_decode(lens, hq, hkv, d, bs, dt, seed=100 + hq + bs)
    assert path == "decode_splitk"
    H.assert_bf16_close(got, want, f"decode {hq}/{hkv} d={d} bs={bs} {dt}")


def test_decode_empty_context_outputs_zeros():
    lens = [0, 33, 0, 5]
    got, want, _ = _run_decode(lens, 8, 2, 128, 16, "bf16", seed=5)
    assert np.all(got[0] == 0.0) and np.all(got[2] == 0.0)
    H.assert_bf16_close(got, want, "empty contexts")


@pytest.mark.parametrize("chunk", [64, 128, 256, 1024])
def test_decode_is_invariant_to_the_split(chunk):
    lens = [2000, 64, 65, 1023, 1025]
    base, want, _ = _run_decode(lens, 32, 8, 128, 16, "bf16", seed=9, chunk=0)
    got, _, _ = _run_decode(lens, 32, 8, 128, 16, "bf16", seed=9, chunk=chunk)
    H.assert_bf16_close(got, want, f"chunk={chunk}")
    assert np.abs(got - base).max() <= 2 ** -6  # different merge order, same answer to bf16 noise


def test_decode_f32_takes_the_generic_path():
    kc, vc, table = H.make_paged_cache([3, 50, 129], 8, 2, 64, seed=12)
    q = H.normal((3, 1, 4, 64), 13)
    o = torch.empty(3, 1, 4, 64, device="cuda")
    low.flash_attn_with_kvcache(H.to_dev(q, "f32"), H.to_dev(kc, "f32"), H.to_dev(vc, "f32"), o,
                                torch.from_numpy(table).cuda(), torch.tensor([3, 50, 129], dtype=torch.int32, device="cuda"),
                                3, 1, 4, 2, 64, 8, table.shape[1], 0.125)
    torch.cuda.synchronize()
    assert ffi.last_path() == "tile_simt"
    H.assert_ref_close(H.to_np(o), ob.attn_f64_kvcache(q, kc, vc, [3, 50, 129], table, scale=0.125), H.F32_TOL, "f32 decode")


@pytest.mark.parametrize("bs", [1, 5, 16, 32])
def test_block_slot_indexing_is_bit_exact(bs):
    rng = np.random.default_rng(bs)
    lens = rng.integers(0, 700, size=37).astype(np.int32)
    _, _, table = H.make_paged_cache(lens, bs, 1, 8, seed=bs, pool_blocks=int(sum((l + bs - 1) // bs for l in lens)) + 50)
    want = ob.block_slots(table, lens, bs)
    offsets = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    out = torch.full((int(lens.sum()),), -7, dtype=torch.int32, device="cuda")
    low.debug_block_slots(torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda(),
                          torch.from_numpy(offsets).cuda(), len(lens), bs, table.shape[1], out)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), want)


def test_decode_is_invariant_to_where_pages_live():
    # moving every page to another physical block (and updating the table) must not change a bit
    lens = [300, 47, 1000]
    hq, hkv, d, bs = 32, 8, 128, 16
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=21, pool_blocks=200)
    q = H.normal((3, 1, hq, d), 22)
    perm = np.random.default_rng(5).permutation(200)
    kc2, vc2 = np.empty_like(kc), np.empty_like(vc)
    kc2[perm], vc2[perm] = kc, vc
    table2 = np.where(table >= 0, perm[np.maximum(table, 0)], -1).astype(np.int32)
    outs = []
    for a, b_, t in ((kc, vc, table), (kc2, vc2, table2)):
        o = torch.empty(3, 1, hq, d, device="cuda", dtype=torch.bfloat16)
        low.flash_attn_with_kvcache(H.to_dev(q, "bf16"), H.to_dev(a, "bf16"), H.to_dev(b_, "bf16"), o,
                                    torch.from_numpy(t).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                    3, 1, hq, hkv, d, bs, t.shape[1], 1.0 / np.sqrt(d))
        torch.cuda.synchronize()
        outs.append(o.clone())
    assert torch.equal(outs[0], outs[1])
