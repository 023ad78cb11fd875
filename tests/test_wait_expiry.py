"""A bounded wait inside the tensor-core prefill kernel that runs out must be visible through the
ABI. The kernel cannot hang: every wait has a limit, after which the CTA records the wait's code
in a host-mapped status word, drains its copies, frees its tensor memory and returns. The launch
is asynchronous, so the call that made it has already returned OK; the NEXT entry-point call for
that device reports the failure (status 5, a message naming the wait) without launching anything,
and the call after that is clean — the error contract of luma-flash-attn/src/error.rs:38-51
(FlashAttnError::Cuda carrying the library's message).

The expiry is provoked the permitted way: the limit is shortened to about a millisecond and a test
hook makes the K producer leave out one tile, so that the issuer's wait for it runs out and the
kernel returns. Nothing traps, faults or spins without bound."""
import math

import numpy as np
import pytest
import torch

from luma_b200 import error as E
from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_by_the_next_call_and_then_cleared():
    b, s, hq, hkv, d = 1, 512, 4, 2, 128
    q = H.round_to(H.normal((b, s, hq, d), 1), "bf16")
    k = H.round_to(H.normal((b, s, hkv, d), 2), "bf16")
    v = H.round_to(H.normal((b, s, hkv, d), 3), "bf16")
    qd, kd, vd = (H.to_dev(x, "bf16") for x in (q, k, v))
    o = torch.empty_like(qd)
    scale = 1.0 / math.sqrt(d)
    torch.cuda.synchronize()
    assert ffi.device_status() == 0
    try:
        ffi.set_option("prefill_wait_us", 1000)
        ffi.set_option("prefill_test_skip_k", 3)          # K tile 2 is never requested
        low.flash_attn(qd, kd, vd, o, b, s, s, hq, hkv, d, 0, scale)   # returns OK: the launch is asynchronous
        assert ffi.last_path() == "prefill_tcgen05"
    finally:
        ffi.set_option("prefill_test_skip_k", 0)
        ffi.set_option("prefill_wait_us", 0)
    torch.cuda.synchronize()                               # the kernel has given up and returned by now
    with pytest.raises(E.CudaError) as exc:
        low.flash_attn(qd, kd, vd, o, b, s, s, hq, hkv, d, 0, scale)
    assert "bounded wait" in str(exc.value) and "code" in str(exc.value)
    # the word was cleared by that report: the next call runs and is right
    o.fill_(float("nan"))
    low.flash_attn(qd, kd, vd, o, b, s, s, hq, hkv, d, 0, scale)
    torch.cuda.synchronize()
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), ob.attn_f64_batch(q, k, v), "call after the reported expiry")


def test_workspaces_are_bounded_and_releasable():
    # the decode path keeps one split-K workspace per (device, stream), at most 32, and gives them back on request
    hq, hkv, d, bs = 8, 2, 128, 16
    lens = [300, 40]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=5)
    q = H.round_to(H.normal((2, 1, hq, d), 6), "bf16")
    want = ob.attn_f64_kvcache(q, H.round_to(kc, "bf16"), H.round_to(vc, "bf16"), lens, table)
    qd, kd, vd = H.to_dev(q, "bf16"), H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16")
    td, ld = torch.from_numpy(table).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda")
    ffi.lib.flash_attn_release_workspaces()
    streams = [torch.cuda.Stream() for _ in range(40)]
    torch.cuda.synchronize()
    outs = []
    for st in streams:
        o = torch.full_like(qd, float("nan"))
        with torch.cuda.stream(st):
            low.flash_attn_with_kvcache(qd, kd, vd, o, td, ld, 2, 1, hq, hkv, d, bs, table.shape[1], 1.0 / math.sqrt(d), st)
        outs.append(o)
    torch.cuda.synchronize()
    for o in outs:
        H.assert_bf16_close(H.to_np(o), want, "decode on one of many streams")
    held = ffi.lib.flash_attn_release_workspaces()
    assert 1 <= held <= 32
    assert ffi.lib.flash_attn_release_workspaces() == 0
