"""The allocation-free decode entry point, flash_attn_decode_bf16_noalloc.

Some callers of the decode path cannot let the library allocate: an engine that has already given
all device memory to its own pool (a cudaMalloc inside the library would fail), or a step that must
not stall on the driver's allocation lock. For them the split-K scratch is a fixed 16 MiB array
inside the library. This test drives that entry point through the C ABI and checks that it returns
what the ordinary entry point (flash_attn_with_kvcache_bf16) returns, on two calls in a row that
share the scratch array; that a call really leaves the device's free memory and torch's allocator
untouched; that the largest problem the array holds runs and one row more is refused with a message.

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
    # and the very same call repeated gives the very same bits — with the device's free memory and
    # torch's own books unchanged across it: by now the array's module is loaded, so a call that
    # allocated anything anywhere would show here (the first call on a device is the one that may
    # still have to back the array, which is why it is not the one measured)
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info()
    held_before = torch.cuda.memory_allocated()
    o = torch.full_like(dev["q"], float("nan"))           # the caller's output buffer, allocated before the measurement
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info()
    held_before = torch.cuda.memory_allocated()
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        rc = ffi.lib.flash_attn_decode_bf16_noalloc(dev["q"].data_ptr(), dev["k"].data_ptr(), dev["v"].data_ptr(), o.data_ptr(),
                                                    dev["bt"].data_ptr(), dev["cl"].data_ptr(), len(lens), hq, hkv, d, bs,
                                                    dev["bt"].shape[1], scale, st)
        assert rc == 0, ffi.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == held_before
    assert np.array_equal(H.to_np(o), got)


def test_noalloc_decode_at_exactly_the_largest_size_that_fits():
    # 16 MiB / (128*4 + 8) bytes = 32 263 (sequence, head) rows: 32 263 sequences of one head each, one
    # token cached per sequence, is the largest call the array holds; one more row is refused
    d, bs = 128, 16
    n = (16 << 20) // (d * 4 + 8)
    assert n == 32263
    rng = np.random.Generator(np.random.Philox(77))
    kc = torch.from_numpy(rng.standard_normal((64, bs, 1, d), dtype=np.float32)).cuda().bfloat16()
    vc = torch.from_numpy(rng.standard_normal((64, bs, 1, d), dtype=np.float32)).cuda().bfloat16()
    q = torch.from_numpy(rng.standard_normal((n + 1, 1, 1, d), dtype=np.float32)).cuda().bfloat16()
    table = torch.from_numpy(rng.integers(0, 64, size=(n + 1, 1)).astype(np.int32)).cuda()
    lens = torch.from_numpy(rng.integers(1, bs + 1, size=n + 1).astype(np.int32)).cuda()
    st = torch.cuda.current_stream().cuda_stream
    o = torch.full_like(q, float("nan"))
    rc = ffi.lib.flash_attn_decode_bf16_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), table.data_ptr(),
                                                lens.data_ptr(), n, 1, 1, d, bs, 1, 0.1, st)
    assert rc == 0, ffi.last_error()
    torch.cuda.synchronize()
    want = torch.full_like(q, float("nan"))
    rc = ffi.lib.flash_attn_with_kvcache_bf16(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), want.data_ptr(), table.data_ptr(),
                                              lens.data_ptr(), n, 1, 1, 1, d, bs, 1, 0.1, st)
    assert rc == 0, ffi.last_error()
    torch.cuda.synchronize()
    assert torch.isfinite(o[:n].float()).all()
    H.assert_bf16_close(H.to_np(o[:n]), H.to_np(want[:n]), "largest call that fits")
    rc = ffi.lib.flash_attn_decode_bf16_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), table.data_ptr(),
                                                lens.data_ptr(), n + 1, 1, 1, d, bs, 1, 0.1, st)
    assert rc == 2 and "static scratch" in ffi.last_error()


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
