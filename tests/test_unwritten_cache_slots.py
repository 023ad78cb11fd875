"""Cache slots that no token was written to may hold anything — NaN or Inf bit patterns in a pool
that came from an uninitialised allocation, or in a page recycled from other use. The reference
kernels read only keys j < context_len (luma-flash-attn/kernels/flash_attn_with_kvcache.cu:60-100,
206-260), so such slots never reach the result. Here every slot past each sequence's length — the
rest of its last page and every unused page — is filled with NaN, and the outputs must still match
the oracle: chunked prefill over the paged cache (tensor-core kernel; the V rows of a sequence's
last, partly filled tile are cleared in shared memory before P.V), paged packed varlen, single-token
decode (split-K), and the rows of the NEXT sequence in a packed contiguous buffer."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu
D = 128


def _poison_unwritten(cache, table, lens, bs):
    """Copy of `cache` with NaN in every slot that holds no token of any sequence."""
    written = np.zeros(cache.shape[:2], dtype=bool)
    for s, L in enumerate(lens):
        j = np.arange(L)
        written[table[s, j // bs], j % bs] = True
    out = cache.copy()
    out[~written] = np.nan
    return out


@pytest.mark.parametrize("bs", [8, 16, 128])
@pytest.mark.parametrize("sq", [1, 3, 130])
def test_kvcache_entry_point_ignores_unwritten_slots(bs, sq):
    hq, hkv = 8, 2
    lens = [sq + 300, sq + 1, sq + 127, 1000 + sq, sq + 129, sq + 5]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, D, seed=40 + bs + sq)
    kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
    q = H.round_to(H.normal((len(lens), sq, hq, D), 41 + sq), "bf16")
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    kp, vp = _poison_unwritten(kc, table, lens, bs), _poison_unwritten(vc, table, lens, bs)
    assert np.isnan(vp).any()
    qd = H.to_dev(q, "bf16")
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_with_kvcache(qd, H.to_dev(kp, "bf16"), H.to_dev(vp, "bf16"), o, torch.from_numpy(table).cuda(),
                                torch.tensor(lens, dtype=torch.int32, device="cuda"), len(lens), sq, hq, hkv, D, bs,
                                table.shape[1], 1.0 / np.sqrt(D))
    torch.cuda.synchronize()
    assert ffi.last_path() == ("decode_splitk" if sq == 1 else "prefill_tcgen05")
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"NaN in unwritten slots, page {bs}, {sq} query tokens")


@pytest.mark.parametrize("bs", [16, 64])
def test_paged_varlen_ignores_unwritten_slots(bs):
    hq, hkv = 4, 2
    ql, kl = [100, 37, 260], [300, 37, 700]
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(kl)]).astype(np.int32)
    kc, vc, table = H.make_paged_cache(kl, bs, hkv, D, seed=60 + bs)
    kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
    q = H.round_to(H.normal((int(cu_q[-1]), hq, D), 61), "bf16")
    want = ob.attn_f64_varlen(q, kc, vc, cu_q, cu_k, block_table=table)
    kp, vp = _poison_unwritten(kc, table, kl, bs), _poison_unwritten(vc, table, kl, bs)
    qd = H.to_dev(q, "bf16")
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_varlen(qd, H.to_dev(kp, "bf16"), H.to_dev(vp, "bf16"), o, torch.from_numpy(cu_q).cuda(),
                          torch.from_numpy(cu_k).cuda(), len(ql), max(ql), max(kl), hq, hkv, D, 1.0 / np.sqrt(D),
                          block_tables=torch.from_numpy(table).cuda(), block_size=bs, total_q=int(cu_q[-1]))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"paged varlen with NaN in unwritten slots, page {bs}")


def test_packed_varlen_is_not_poisoned_by_the_next_sequence():
    """Contiguous packed K/V: the last tile of a sequence reaches into the next sequence's rows. Those
    are another request's data; if they are NaN, only that request's output may be NaN."""
    hq, hkv = 4, 2
    lens = [100, 200, 77]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    q = H.round_to(H.normal((total, hq, D), 71), "bf16")
    k = H.round_to(H.normal((total, hkv, D), 72), "bf16")
    v = H.round_to(H.normal((total, hkv, D), 73), "bf16")
    want = ob.attn_f64_varlen(q, k, v, cu, cu)
    kp, vp = k.copy(), v.copy()
    kp[cu[1]:cu[2]] = np.nan       # the middle sequence is garbage
    vp[cu[1]:cu[2]] = np.nan
    qd = H.to_dev(q, "bf16")
    for totals in (dict(total_q=total, total_k=total), dict()):
        o = torch.full_like(qd, float("nan"))
        low.flash_attn_varlen(qd, H.to_dev(kp, "bf16"), H.to_dev(vp, "bf16"), o, torch.from_numpy(cu).cuda(),
                              torch.from_numpy(cu).cuda(), len(lens), max(lens), max(lens), hq, hkv, D, 1.0 / np.sqrt(D),
                              **totals)
        torch.cuda.synchronize()
        assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
        got = H.to_np(o)
        for s in (0, 2):
            H.assert_bf16_close(got[cu[s]:cu[s + 1]], want[cu[s]:cu[s + 1]], f"sequence {s} next to a NaN sequence")
        assert np.isnan(got[cu[1]:cu[2]]).all()
