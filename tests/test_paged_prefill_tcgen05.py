"""Chunked prefill over a paged KV cache on the tcgen05 kernel (one TMA box per page), through the
C ABI against the oracle: permuted block tables, page sizes 8..128, contexts shorter than the
query chunk (rows before the cache output zeros), empty contexts, GQA and MHA."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _run(lens, sq, hq, hkv, bs, dt, seed):
    d = 128
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=seed)
    kc, vc = H.round_to(kc, dt), H.round_to(vc, dt)
    q = H.round_to(H.normal((len(lens), sq, hq, d), seed + 5), dt)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_with_kvcache(qd, H.to_dev(kc, dt), H.to_dev(vc, dt), o, torch.from_numpy(table).cuda(),
                                torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), sq, hq, hkv, d,
                                bs, table.shape[1], 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    path = ffi.last_path()
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    return H.to_np(o), want, path


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("sq,hq,hkv,bs", [
    (64, 8, 2, 16),     # GQA 4, chunk smaller than a tile
    (128, 4, 4, 16),    # MHA, exactly one tile
    (200, 8, 8, 32),    # ragged second tile
    (130, 6, 2, 8),     # odd group, small pages
    (256, 4, 1, 128),   # one page per K/V tile
    (96, 8, 2, 64),
])
def test_paged_chunked_prefill_matches_oracle(sq, hq, hkv, bs, dt):
    lens = [sq + 300, sq, sq + 1, 1000 + sq, sq + 129]
    got, want, path = _run(lens, sq, hq, hkv, bs, dt, seed=500 + sq + bs)
    assert path == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(got, want, f"paged prefill sq={sq} {hq}/{hkv} bs={bs} {dt}")


@pytest.mark.parametrize("sq", [2, 5, 15])
def test_short_query_chunks_run_on_the_tensor_core_kernel(sq):
    """A few query tokens per sequence over a long cache (speculative decoding, small prefill chunks):
    every chunk longer than one token takes the tensor-core kernel, most rows of its tiles empty."""
    lens = [sq, sq + 1, 700, 16, 1500 + sq, 129]
    got, want, path = _run(lens, sq, 8, 2, 16, "bf16", seed=900 + sq)
    assert path == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(got, want, f"paged prefill, {sq}-token chunks")


@pytest.mark.parametrize("s,hq,hkv", [(2, 2, 2), (7, 8, 2), (15, 6, 3)])
def test_short_sequences_batched_entry_point(s, hq, hkv):
    d = 128
    q = H.round_to(H.normal((3, s, hq, d), 70 + s), "bf16")
    k = H.round_to(H.normal((3, s, hkv, d), 71 + s), "bf16")
    v = H.round_to(H.normal((3, s, hkv, d), 72 + s), "bf16")
    qd = H.to_dev(q, "bf16")
    o = torch.full_like(qd, float("nan"))
    low.flash_attn(qd, H.to_dev(k, "bf16"), H.to_dev(v, "bf16"), o, 3, s, s, hq, hkv, d, 0, 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), ob.attn_f64_batch(q, k, v, start_pos=0), f"batched, S={s}")


def test_paged_prefill_short_and_empty_contexts():
    # contexts shorter than the chunk: rows that sit before the cache see nothing and output zeros
    # (flash_attn_with_kvcache.cu:185-195,270-275); an empty context outputs zeros everywhere
    sq = 160
    lens = [40, 0, 160, 159, 700]
    got, want, path = _run(lens, sq, 8, 2, 16, "bf16", seed=77)
    assert path == "prefill_tcgen05"
    assert np.all(got[1] == 0.0)
    assert np.all(got[0, : sq - 40] == 0.0)
    H.assert_bf16_close(got, want, "short / empty contexts")


def test_paged_prefill_page_size_that_does_not_tile_takes_the_simt_kernel():
    got, want, path = _run([300, 77], 48, 4, 2, 5, "bf16", seed=9)
    assert path == "tile_simt"
    H.assert_bf16_close(got, want, "page size 5")


def test_paged_prefill_is_invariant_to_where_pages_live():
    sq, hq, hkv, bs, d = 128, 8, 2, 16, 128
    lens = [500, 128, 333]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=31, pool_blocks=120)
    q = H.normal((3, sq, hq, d), 32)
    perm = np.random.default_rng(6).permutation(120)
    kc2, vc2 = np.empty_like(kc), np.empty_like(vc)
    kc2[perm], vc2[perm] = kc, vc
    table2 = np.where(table >= 0, perm[np.maximum(table, 0)], -1).astype(np.int32)
    outs = []
    for a, b_, t in ((kc, vc, table), (kc2, vc2, table2)):
        o = torch.empty(3, sq, hq, d, device="cuda", dtype=torch.bfloat16)
        low.flash_attn_with_kvcache(H.to_dev(q, "bf16"), H.to_dev(a, "bf16"), H.to_dev(b_, "bf16"), o,
                                    torch.from_numpy(t).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                    3, sq, hq, hkv, d, bs, t.shape[1], 1.0 / np.sqrt(d))
        torch.cuda.synchronize()
        outs.append(o.clone())
    assert torch.equal(outs[0], outs[1])
