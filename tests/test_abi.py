"""CPU tests of the drop-in boundary: the library loads, exports every symbol the header declares,
and rejects bad arguments with the reference's status codes before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import luma_b200 as L
from luma_b200 import ffi, low, high

ROOT = Path(__file__).resolve().parent.parent


def _header_functions():
    """Every function the C headers under include/ declare (flash_attn.h, luma_nn_kernels.h, luma_dist_comm.h)."""
    names = set()
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b((?:flash_attn|luma_softmax|luma_comm|luma_ipc|luma_peer)_\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    names = _header_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(ffi.lib, n), f"{n} declared under include/ but not exported"
    assert sorted(ffi.EXPORTED_SYMBOLS) == names
    # the ten symbols luma-flash-attn/src/api/ffi.rs binds
    for n in ["flash_attn_f32", "flash_attn_f16", "flash_attn_bf16",
              "flash_attn_varlen_f32", "flash_attn_varlen_f16", "flash_attn_varlen_bf16",
              "flash_attn_with_kvcache_f32", "flash_attn_with_kvcache_f16",
              "flash_attn_with_kvcache_bf16", "flash_attn_last_error"]:
        assert n in names


def test_version_and_last_error_never_null():
    assert b"sm_100a" in ffi.lib.flash_attn_version()
    assert ffi.lib.flash_attn_last_error() is not None


def _batch(q=1, k=1, v=1, o=1, batch=1, sq=1, skv=1, hq=1, hkv=1, d=32, sp=0):
    return ffi.lib.flash_attn_f32(q, k, v, o, batch, sq, skv, hq, hkv, d, sp, 1.0, None, None)


def test_batch_status_codes_in_reference_order():
    # luma-flash-attn/kernels/flash_attn_func.cu:273-303; tests/low.rs:279-358
    assert _batch(q=None) == 1 and ffi.last_error()
    assert _batch(batch=0) == 2 and "positive" in ffi.last_error()
    assert _batch(hq=3, hkv=2) == 2 and "GQA" in ffi.last_error()
    assert _batch(sp=-1) == 4
    assert _batch(d=48) == 3 and "32/64/128" in ffi.last_error()
    # null beats bad shape; bad shape beats bad start_pos; start_pos beats head size
    assert _batch(q=None, batch=0, sp=-1, d=48) == 1
    assert _batch(batch=0, sp=-1, d=48) == 2
    assert _batch(sp=-1, d=48) == 4


def test_kvcache_and_varlen_status_codes():
    f = ffi.lib.flash_attn_with_kvcache_bf16
    ok = dict(q=1, k=1, v=1, o=1, bt=1, cl=1, n=1, sq=1, hq=1, hkv=1, d=64, bs=16, mb=1)

    def call(**kw):
        a = {**ok, **kw}
        return f(a["q"], a["k"], a["v"], a["o"], a["bt"], a["cl"], a["n"], a["sq"], a["hq"], a["hkv"],
                 a["d"], a["bs"], a["mb"], 1.0, None)
    # flash_attn_with_kvcache.cu:356-371: head size is a SHAPE error here
    assert call(bt=None) == 1
    assert call(cl=None) == 1
    assert call(n=0) == 2
    assert call(hq=3, hkv=2) == 2
    assert call(d=48) == 2
    assert call(sq=0) == 2
    assert call(bs=0) == 2

    g = ffi.lib.flash_attn_varlen_f16

    def vcall(q=1, k=1, v=1, o=1, cq=1, ck=1, bt=None, n=1, mq=1, mk=1, hq=1, hkv=1, d=32, bs=1, mb=0, paged=0):
        return g(q, k, v, o, cq, ck, bt, n, mq, mk, hq, hkv, d, bs, mb, paged, 1.0, None)
    # flash_attn_varlen_func.cu:271-286
    assert vcall(cq=None) == 1
    assert vcall(k=None) == 1
    assert vcall(paged=1, bt=None) == 1
    assert vcall(n=0) == 2
    assert vcall(d=16) == 2
    assert vcall(mq=0) == 2
    assert vcall(bs=0) == 2


def test_every_call_clears_the_previous_message():
    assert _batch(q=None) == 1 and ffi.last_error() != ""
    assert _batch(batch=0) == 2 and "null" not in ffi.last_error()


def test_low_level_validation_errors_before_any_launch():
    # tests/low.rs:278-327 — raised host-side, so CPU buffers suffice
    t = torch.zeros(1)
    with pytest.raises(L.InvalidHeadSize):
        low.flash_attn(t, t, t, t, 1, 1, 1, 1, 1, 48, 0, 1.0)
    with pytest.raises(L.InvalidShape):
        low.flash_attn(t, t, t, t, 1, 1, 1, 3, 2, 32, 0, 1.0)
    with pytest.raises(L.InvalidStartPos):
        low.flash_attn(t, t, t, t, 1, 1, 1, 1, 1, 32, -1, 1.0)
    with pytest.raises(L.InvalidShape):
        low.flash_attn(t, t, t, t, 0, 1, 1, 1, 1, 32, 0, 1.0)
    with pytest.raises(L.BufferTooSmall):
        low.flash_attn(t, t, t, t, 1, 64, 64, 4, 4, 32, 0, 1.0)
    big = torch.zeros(64 * 4 * 32)
    with pytest.raises(L.BufferTooSmall, match="attn_mask"):
        low.flash_attn(big, big, big, big, 1, 64, 64, 4, 4, 32, 0, 1.0, torch.zeros(1, dtype=torch.uint8))
    with pytest.raises(L.InvalidShape):
        low.flash_attn_with_kvcache(t, t, t, t, t, t, 1, 0, 1, 1, 32, 16, 1, 1.0)
    with pytest.raises(L.BufferTooSmall):
        low.flash_attn_with_kvcache(t, t, t, t, t, t, 4, 1, 8, 2, 64, 16, 1, 1.0)


def test_high_level_guards():
    # high.rs:46-50 (non-causal unsupported), f64 rejected (tests/high.rs f64 rejection)
    q = torch.zeros(1, 2, 1, 32)
    with pytest.raises(L.Unsupported):
        high.flash_attn_func(q, q, q, causal=False)
    with pytest.raises(L.Unsupported):
        high.flash_attn_func(q.double(), q.double(), q.double())
    with pytest.raises(L.Unsupported):
        high.flash_attn_varlen_func(q[0], q[0], q[0], torch.zeros(2, dtype=torch.int32),
                                    torch.zeros(2, dtype=torch.int32), 1, 1, causal=False)


def test_error_display_strings_match_reference():
    # error.rs:9-31
    assert str(L.NullPtr("x")) == "flash_attn: null pointer parameter (x)"
    assert str(L.BufferTooSmall("q: need at least 2 elements, got 1")).startswith("flash_attn: buffer too small")
    assert str(L.Unknown(9)) == "flash_attn: unknown error code 9"
    with pytest.raises(L.Unknown):
        from luma_b200.error import from_status
        from_status(9, "")


def test_compute_without_device_fails_loudly():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert _batch() == 5
    assert "no CPU fallback" in ffi.last_error()


def test_head_sharded_launch_order_is_a_permutation():
    """The grid rows of a head-sharded prefill run the bands of tile pairs in another order than
    heaviest-first (a first wave that mixes all weights, then heaviest first): the index arithmetic,
    shared by the kernel and this host entry point, must hit every band exactly once."""
    rank = ffi.lib.flash_attn_debug_launch_rank
    for rows in (2, 5, 7, 10, 64, 65, 128, 1000):
        for w in (1, 2, 3, 5, 19, 32, 148):
            m = rows // w
            if m < 2:
                continue                                   # the launcher keeps heaviest-first then
            got = [rank(by, w, m) for by in range(rows)]
            assert sorted(got) == list(range(rows)), (rows, w, m)
            assert got[:w] == [i * m for i in range(w)]   # the first wave samples every m-th band
            rest = got[w:]
            assert rest == sorted(rest)                    # the others follow heaviest first
        assert [rank(by, 0, 0) for by in range(rows)] == list(range(rows))


def test_host_pipeline_steps_tile_every_batch_element():
    """flash_attn_host_<T> cuts a call into (batch element, first row, end row) steps: per element they
    must cover [0, q_seq_len) once, in order, in whole 128-row tiles except at the very end, and the
    first and last steps of a long call are the short ones (host arithmetic only, no device)."""
    from luma_b200 import high
    for b, sq, rows in [(2, 8192, 0), (1, 16384, 0), (1, 8192, 0), (3, 1000, 0), (2, 8192, 1024), (1, 300, 128),
                        (2, 4096, 0), (1, 1, 0), (4, 129, 64), (1, 5000, 0)]:
        steps = high.host_steps(b, sq, rows)
        assert [e for e, _, _ in steps] == sorted(e for e, _, _ in steps)
        for e in range(b):
            mine = [(r0, r1) for i, r0, r1 in steps if i == e]
            assert mine[0][0] == 0 and mine[-1][1] == sq
            assert all(a[1] == n[0] for a, n in zip(mine, mine[1:]))
            assert all(r1 > r0 for r0, r1 in mine)
            assert all(r0 % 128 == 0 for r0, _ in mine) or rows not in (0,) and rows % 128 != 0
    long_call = high.host_steps(2, 8192, 0)
    sizes = [r1 - r0 for _, r0, r1 in long_call]
    assert sizes[0] == min(sizes) and sizes[-1] == min(sizes) and max(sizes) == 4096 and sum(sizes) == 2 * 8192
