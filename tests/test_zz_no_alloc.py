"""The allocation-free decode entry point, flash_attn_decode_bf16_noalloc.

Some callers of the decode path cannot let the library allocate: an engine that has already given
all device memory to its own pool (a cudaMalloc inside the library would fail), or a step that must
not stall on the driver's allocation lock. For them the split-K scratch is a fixed 16 MiB array
inside the library. This test drives that entry point through the C ABI and checks that it returns
what the ordinary entry point (flash_attn_with_kvcache_bf16) returns, on two calls in a row that
share the scratch array, and that a problem too large for the array is refused with a message.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest
import torch

from luma_b200 import ffi
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _problem(lens, hq, hkv, d, bs, seed):
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=seed)
    q = H.normal((len(lens), 1, hq, d), seed + 3)
    dev = dict(q=H.to_dev(q, "bf16"), k=H.to_dev(kc, "bf16"), v=H.to_dev(vc, "bf16"),
               bt=torch.from_numpy(table).cuda(), cl=torch.tensor(lens, dtype=torch.int32, device="cuda"))
    host = dict(q=H.round_to(q, "bf16"), k=H.round_to(kc, "bf16"), v=H.round_to(vc, "bf16"), table=table)
    return dev, host


def _call(fn_name, dev, n, hq, hkv, d, bs, scale, with_q_seq_len):
    o = torch.full_like(dev["q"], float("nan"))
    st = torch.cuda.current_stream().cuda_stream
    fn = getattr(ffi.lib, fn_name)
    if with_q_seq_len:
        rc = fn(dev["q"].data_ptr(), dev["k"].data_ptr(), dev["v"].data_ptr(), o.data_ptr(), dev["bt"].data_ptr(),
                dev["cl"].data_ptr(), n, 1, hq, hkv, d, bs, dev["bt"].shape[1], scale, st)
    else:
        rc = fn(dev["q"].data_ptr(), dev["k"].data_ptr(), dev["v"].data_ptr(), o.data_ptr(), dev["bt"].data_ptr(),
                dev["cl"].data_ptr(), n, hq, hkv, d, bs, dev["bt"].shape[1], scale, st)
    assert rc == 0, ffi.last_error()
    torch.cuda.synchronize()
    return H.to_np(o)


def test_noalloc_decode_matches_the_allocating_entry_point_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's partials in the
    # shared scratch array and must not be disturbed by them
    problems = [([1500, 64, 1, 777, 513, 16], 32, 8, 128, 16, 401),
                ([90, 0, 2049, 33], 16, 2, 64, 8, 402)]
    for lens, hq, hkv, d, bs, seed in problems:
        dev, host = _problem(lens, hq, hkv, d, bs, seed)
        scale = 1.0 / np.sqrt(d)
        want = _call("flash_attn_with_kvcache_bf16", dev, len(lens), hq, hkv, d, bs, scale, True)
        assert ffi.last_path() == "decode_splitk"
        got = _call("flash_attn_decode_bf16_noalloc", dev, len(lens), hq, hkv, d, bs, scale, False)
        assert ffi.last_path() == "decode_splitk_static"
        H.assert_bf16_close(got, want, f"noalloc vs allocating entry point, lens={lens}")
        oracle = ob.attn_f64_kvcache(host["q"], host["k"], host["v"], lens, host["table"], scale=scale)
        H.assert_bf16_close(got, oracle, f"noalloc vs oracle, lens={lens}")
    # and the very same call repeated gives the very same bits
    again = _call("flash_attn_decode_bf16_noalloc", dev, len(lens), hq, hkv, d, bs, scale, False)
    assert np.array_equal(again, got)


def test_noalloc_decode_refuses_what_does_not_fit():
    # 16 MiB / (128*4 + 8) bytes = 32 263 (sequence, head) rows at most; ask for 40 000
    n, hq = 625, 64
    t = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = ffi.lib.flash_attn_decode_bf16_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                                t.data_ptr(), n, hq, 8, 128, 16, 4, 0.1, None)
    assert rc == 2
    assert "static scratch" in ffi.last_error()
    rc = ffi.lib.flash_attn_decode_bf16_noalloc(None, None, None, None, None, None, 1, 1, 1, 128, 16, 1, 0.1, None)
    assert rc == 1
    rc = ffi.lib.flash_attn_decode_bf16_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                                t.data_ptr(), 1, 1, 1, 32, 16, 1, 0.1, None)
    assert rc == 2
