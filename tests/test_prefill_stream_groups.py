"""The prefill grid can run the (batch element, KV head) streams in groups, one group after the other
(grid z axis; automatic for many short streams whose K/V exceed L2, option "prefill_groups" otherwise).
Grouping only changes which CTA computes which stream, never the arithmetic: every group count —
divisors, non-divisors, more groups than streams — must give the same bits as one group, for the
batched, the packed variable-length and the paged chunked-prefill entry points."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

D = 128


def _with_groups(groups, fn):
    ffi.set_option("prefill_groups", groups)
    try:
        out = fn()
        torch.cuda.synchronize()
        assert ffi.last_path() == "prefill_tcgen05"
        assert ffi.device_status() == 0
        return out
    finally:
        ffi.set_option("prefill_groups", 0)


@pytest.mark.parametrize("b,hq,hkv,s", [(3, 4, 4, 600), (2, 6, 2, 384), (5, 2, 1, 300)])
def test_batched_call_is_invariant_to_the_group_count(b, hq, hkv, s):
    q = H.to_dev(H.normal((b, s, hq, D), 1), "bf16")
    k = H.to_dev(H.normal((b, s, hkv, D), 2), "bf16")
    v = H.to_dev(H.normal((b, s, hkv, D), 3), "bf16")

    def run():
        o = torch.full_like(q, float("nan"))
        low.flash_attn(q, k, v, o, b, s, s, hq, hkv, D, 0, 1.0 / np.sqrt(D))
        return o

    base = _with_groups(1, run)
    want = ob.attn_f64_batch(H.to_np(q), H.to_np(k), H.to_np(v))
    H.assert_bf16_close(H.to_np(base), want, "one group")
    for g in (2, 3, 5, b * hkv, b * hkv + 7):
        assert torch.equal(_with_groups(g, run), base), g


def test_varlen_call_is_invariant_to_the_group_count():
    ql = [100, 37, 260, 513, 64]
    hq, hkv = 4, 4
    cu = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    t = int(cu[-1])
    q = H.to_dev(H.normal((t, hq, D), 4), "bf16")
    k = H.to_dev(H.normal((t, hkv, D), 5), "bf16")
    v = H.to_dev(H.normal((t, hkv, D), 6), "bf16")
    cd = torch.from_numpy(cu).cuda()

    def run():
        o = torch.full_like(q, float("nan"))
        low.flash_attn_varlen(q, k, v, o, cd, cd, len(ql), max(ql), max(ql), hq, hkv, D, 1.0 / np.sqrt(D))
        return o

    base = _with_groups(1, run)
    H.assert_bf16_close(H.to_np(base), ob.attn_f64_varlen(H.to_np(q), H.to_np(k), H.to_np(v), cu, cu), "one group")
    for g in (2, 3, 7, 20, 64):
        assert torch.equal(_with_groups(g, run), base), g


def test_paged_chunked_prefill_is_invariant_to_the_group_count():
    lens = [300, 1000, 129, 640]
    sq, hq, hkv, bs = 128, 4, 2, 16
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, D, seed=7)
    q = H.to_dev(H.normal((len(lens), sq, hq, D), 8), "bf16")
    kd, vd = H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16")
    td = torch.from_numpy(table).cuda()
    ld = torch.tensor(lens, dtype=torch.int32, device="cuda")

    def run():
        o = torch.full_like(q, float("nan"))
        low.flash_attn_with_kvcache(q, kd, vd, o, td, ld, len(lens), sq, hq, hkv, D, bs, table.shape[1], 1.0 / np.sqrt(D))
        return o

    base = _with_groups(1, run)
    want = ob.attn_f64_kvcache(H.to_np(q), H.round_to(kc, "bf16"), H.round_to(vc, "bf16"), lens, table)
    H.assert_bf16_close(H.to_np(base), want, "one group")
    for g in (2, 3, 8, 11):
        assert torch.equal(_with_groups(g, run), base), g
