"""Seeded sweeps, against the f64 oracle, of the two paths the batched-prefill sweep does not reach:
* paged single-token decode: batch sizes, GQA widths (groups above 16 take several head blocks), head
  sizes, page sizes (also 1 and non-powers of two, which take the SIMT kernel), contexts from empty to
  a few thousand tokens with permuted block tables, forced split-K chunk lengths;
* packed variable-length prefill, contiguous and paged: ragged query / key lengths (bottom-right
  causal), one-row sequences, head sizes, page sizes.
A guard against shape-dependent slips in the split, page and band arithmetic."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _decode_cases(n, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    out = []
    for i in range(n):
        hkv = int(rng.choice([1, 2, 4, 8]))
        group = int(rng.choice([1, 2, 4, 8, 20]))
        d = int(rng.choice([32, 64, 128, 128]))
        bs = int(rng.choice([1, 5, 8, 16, 16, 32, 64]))
        batch = int(rng.integers(1, 9))
        lens = [int(x) for x in rng.choice([0, 1, int(rng.integers(2, 200)), int(rng.integers(200, 3000))], size=batch)]
        chunk = int(rng.choice([0, 0, 64, 256, 1024]))
        dt = "bf16" if i % 3 else "f16"
        out.append((tuple(lens), hkv * group, hkv, d, bs, chunk, dt))
    return out


DECODE_CASES = _decode_cases(30, 77)


@pytest.mark.parametrize("case", DECODE_CASES, ids=[f"{i}-{c[1]}/{c[2]}-d{c[3]}-p{c[4]}-c{c[5]}-{c[6]}" for i, c in enumerate(DECODE_CASES)])
def test_decode_sweep(case):
    lens, hq, hkv, d, bs, chunk, dt = case
    lens = list(lens)
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=500 + hq + bs)
    kc, vc = H.round_to(kc, dt), H.round_to(vc, dt)
    q = H.round_to(H.normal((len(lens), 1, hq, d), 600 + d), dt)
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan"))
    ffi.set_option("decode_chunk_tokens", chunk)
    try:
        low.flash_attn_with_kvcache(qd, H.to_dev(kc, dt), H.to_dev(vc, dt), o, torch.from_numpy(table).cuda(),
                                    torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), 1, hq, hkv, d, bs,
                                    table.shape[1], 1.0 / np.sqrt(d))
        torch.cuda.synchronize()
    finally:
        ffi.set_option("decode_chunk_tokens", 0)
    assert ffi.last_path() in ("decode_splitk", "tile_simt")
    got = H.to_np(o)
    for s_, length in enumerate(lens):
        if length == 0:
            assert np.all(got[s_] == 0.0)          # an empty context outputs zeros
    H.assert_bf16_close(got, want, f"decode sweep {case}")


def _varlen_cases(n, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    out = []
    for i in range(n):
        hkv = int(rng.choice([1, 2, 4]))
        group = int(rng.choice([1, 2, 4, 3]))
        d = int(rng.choice([64, 128, 128]))
        nseq = int(rng.integers(1, 6))
        ql = [int(x) for x in rng.choice([1, int(rng.integers(2, 130)), int(rng.integers(130, 600))], size=nseq)]
        kl = [q_ + int(rng.choice([0, 0, int(rng.integers(1, 300))])) for q_ in ql]    # prefixes: kv at least as long as q
        paged = bool(i % 2)
        bs = int(rng.choice([8, 16, 32, 128])) if paged else 0
        dt = "bf16" if i % 3 else "f16"
        out.append((tuple(ql), tuple(kl), hkv * group, hkv, d, bs, dt))
    return out


VARLEN_CASES = _varlen_cases(24, 78)


@pytest.mark.parametrize("case", VARLEN_CASES, ids=[f"{i}-{c[2]}/{c[3]}-d{c[4]}-p{c[5]}-{c[6]}" for i, c in enumerate(VARLEN_CASES)])
def test_varlen_sweep(case):
    ql, kl, hq, hkv, d, bs, dt = case
    ql, kl = list(ql), list(kl)
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(kl)]).astype(np.int32)
    tq = int(cu_q[-1])
    q = H.round_to(H.normal((tq, hq, d), 700 + tq), dt)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan"))
    cq, ck = torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda()
    scale = 1.0 / np.sqrt(d)
    if bs:
        kc, vc, table = H.make_paged_cache(kl, bs, hkv, d, seed=800 + tq)
        kc, vc = H.round_to(kc, dt), H.round_to(vc, dt)
        want = ob.attn_f64_varlen(q, kc, vc, cu_q, cu_k, block_table=table)
        low.flash_attn_varlen(qd, H.to_dev(kc, dt), H.to_dev(vc, dt), o, cq, ck, len(ql), max(ql), max(kl), hq, hkv, d, scale,
                              block_tables=torch.from_numpy(table).cuda(), block_size=bs)
    else:
        tk = int(cu_k[-1])
        k = H.round_to(H.normal((tk, hkv, d), 801 + tq), dt)
        v = H.round_to(H.normal((tk, hkv, d), 802 + tq), dt)
        want = ob.attn_f64_varlen(q, k, v, cu_q, cu_k)
        low.flash_attn_varlen(qd, H.to_dev(k, dt), H.to_dev(v, dt), o, cq, ck, len(ql), max(ql), max(kl), hq, hkv, d, scale)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"varlen sweep {case}")
