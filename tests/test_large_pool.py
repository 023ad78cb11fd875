"""Paged K/V pools of more than 2^31 elements per tensor (the 8-GPU decode configuration's pool at one
GPU is 5 G elements): pages that live past the 32-bit element range must be reached through 64-bit
offsets, by the split-K decode kernel's plain loads and by the tensor-map copies of the paged
prefill kernel. The same logical cache is laid out twice — in a small pool, and in a 2.2 G-element
pool with every used page above element 2^31 — and the outputs must be bit-identical; the small
layout is checked against the oracle."""
import math

import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

HKV, D, PAGE = 8, 128, 16
PAGE_ELEMS = PAGE * HKV * D                    # 16384 elements per page
BIG_POOL = (1 << 31) // PAGE_ELEMS + 4096      # 135168 pages = 2.2 G elements (4.4 GB per tensor in bf16)


def _layouts(lens, seed):
    """(small caches, small table, big caches, big table): the same pages, the big pool's at its top."""
    kc, vc, table = H.make_paged_cache(lens, PAGE, HKV, D, seed=seed)
    kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
    n_small = kc.shape[0]
    rng = np.random.Generator(np.random.Philox(seed))
    # page p of the small pool moves to a distinct page among the last 4000 of the big pool
    where = (BIG_POOL - 4000 + rng.permutation(4000)[:n_small]).astype(np.int64)
    assert (where * PAGE_ELEMS > (1 << 31)).all()
    big_table = table.copy()
    valid = table >= 0
    big_table[valid] = where[table[valid]].astype(np.int32)
    kd, vd = H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16")
    kbig = torch.empty(BIG_POOL, PAGE, HKV, D, device="cuda", dtype=torch.bfloat16)
    vbig = torch.empty_like(kbig)
    idx = torch.from_numpy(where).cuda()
    kbig[idx] = kd
    vbig[idx] = vd
    return (kc, vc, kd, vd, table), (kbig, vbig, big_table)


def test_decode_reaches_pages_past_2g_elements():
    lens = [700, 33, 1500, 16, 257]
    hq = 32
    (kc, vc, kd, vd, table), (kbig, vbig, big_table) = _layouts(lens, seed=41)
    q = H.round_to(H.normal((len(lens), 1, hq, D), 44), "bf16")
    qd = H.to_dev(q, "bf16")
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(D)
    outs = []
    for kk, vv, tab in ((kd, vd, table), (kbig, vbig, big_table)):
        o = torch.full_like(qd, float("nan"))
        low.flash_attn_with_kvcache(qd, kk, vv, o, torch.from_numpy(tab).cuda(), lens_d, len(lens), 1, hq, HKV, D,
                                    PAGE, tab.shape[1], scale)
        torch.cuda.synchronize()
        assert ffi.last_path() == "decode_splitk"
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table, scale=scale)
    H.assert_bf16_close(H.to_np(outs[0]), want, "decode, small pool")


def test_paged_prefill_reaches_pages_past_2g_elements():
    lens = [300, 640]          # cached lengths, the query chunk included
    sq, hq = 130, 16
    (kc, vc, kd, vd, table), (kbig, vbig, big_table) = _layouts(lens, seed=43)
    q = H.round_to(H.normal((len(lens), sq, hq, D), 45), "bf16")
    qd = H.to_dev(q, "bf16")
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(D)
    outs = []
    for kk, vv, tab in ((kd, vd, table), (kbig, vbig, big_table)):
        o = torch.full_like(qd, float("nan"))
        low.flash_attn_with_kvcache(qd, kk, vv, o, torch.from_numpy(tab).cuda(), lens_d, len(lens), sq, hq, HKV, D,
                                    PAGE, tab.shape[1], scale)
        torch.cuda.synchronize()
        assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table, scale=scale)
    H.assert_bf16_close(H.to_np(outs[0]), want, "paged prefill, small pool")
