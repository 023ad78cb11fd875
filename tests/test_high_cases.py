"""Tensor-level cases of the reference's suite (luma-flash-attn/tests/high.rs:112-864): batched,
varlen (equal / prefix / paged), kv-cache decode and chunked prefill, 16-bit variants, and the
bit-identity of offset views."""
import numpy as np
import pytest
import torch

import luma_b200 as L
from luma_b200 import high
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = {"f32": H.F32_TOL, "f16": H.F16_TOL, "bf16": H.BF16_REF_TOL}


def _data(shape, seed, dt):
    return H.round_to(ob.data_f64(int(np.prod(shape)), seed).reshape(shape), dt)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 16, 16, 2, 2, 32), (2, 33, 33, 8, 2, 64), (1, 70, 70, 4, 4, 128),
                                   (2, 128, 128, 4, 1, 128)])
def test_flash_attn_func_matches_reference(shape, dt):
    b, sq, skv, hq, hkv, d = shape
    q, k, v = _data((b, sq, hq, d), 1, dt), _data((b, skv, hkv, d), 2, dt), _data((b, skv, hkv, d), 3, dt)
    out = high.flash_attn_func(H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt), None, True, 0)
    assert tuple(out.shape) == (b, sq, hq, d)
    H.assert_ref_close(H.to_np(out), ob.attn_f64_batch(q, k, v), TOL[dt], f"flash_attn_func {shape} {dt}")


def test_flash_attn_func_decode_via_start_pos_and_custom_scale():
    # tests/high.rs:140-155 and the custom-scale case
    b, skv, hq, hkv, d = 2, 57, 4, 2, 64
    q, k, v = _data((b, 1, hq, d), 4, "f32"), _data((b, skv, hkv, d), 5, "f32"), _data((b, skv, hkv, d), 6, "f32")
    out = high.flash_attn_func(H.to_dev(q, "f32"), H.to_dev(k, "f32"), H.to_dev(v, "f32"), 0.37, True, skv - 1)
    H.assert_ref_close(H.to_np(out), ob.attn_f64_batch(q, k, v, scale=0.37, start_pos=skv - 1), H.F32_TOL, "decode via start_pos")


def test_flash_attn_func_rejections():
    q = torch.zeros(1, 4, 2, 32, device="cuda")
    with pytest.raises(L.Unsupported):
        high.flash_attn_func(q, q, q, None, False, 0)
    with pytest.raises(L.Unsupported):
        high.flash_attn_func(q.double(), q.double(), q.double())
    bad = torch.zeros(1, 4, 2, 48, device="cuda")
    with pytest.raises(L.InvalidHeadSize):
        high.flash_attn_func(bad, bad, bad)
    q3 = torch.zeros(1, 4, 3, 32, device="cuda")
    k2 = torch.zeros(1, 4, 2, 32, device="cuda")
    with pytest.raises(L.InvalidShape):
        high.flash_attn_func(q3, k2, k2)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_varlen_equal_prefix_and_paged(dt):
    dev = "cuda"
    # equal lengths, GQA 4:2, d=32 (tests/high.rs:208-247)
    hq, hkv, d = 4, 2, 32
    cu = np.array([0, 3, 8], dtype=np.int32)
    q, k, v = _data((8, hq, d), 41, dt), _data((8, hkv, d), 42, dt), _data((8, hkv, d), 43, dt)
    cu_t = torch.from_numpy(cu).to(dev)
    out = high.flash_attn_varlen_func(H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt), cu_t, cu_t, 5, 5)
    H.assert_ref_close(H.to_np(out), ob.attn_f64_varlen(q, k, v, cu, cu), TOL[dt], "varlen equal")
    # prefix K/V (tests/high.rs:249-290)
    hq, hkv, d = 2, 2, 64
    cu_q, cu_k = np.array([0, 3, 7], dtype=np.int32), np.array([0, 5, 9], dtype=np.int32)
    q, k, v = _data((7, hq, d), 51, dt), _data((9, hkv, d), 52, dt), _data((9, hkv, d), 53, dt)
    out = high.flash_attn_varlen_func(H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt),
                                      torch.from_numpy(cu_q).to(dev), torch.from_numpy(cu_k).to(dev), 4, 5)
    H.assert_ref_close(H.to_np(out), ob.attn_f64_varlen(q, k, v, cu_q, cu_k), TOL[dt], "varlen prefix")
    # paged (tests/high.rs:292-379) — identity table as upstream, then a permuted one
    batch, bs, bps = 2, 4, 2
    hq, hkv, d = 4, 2, 64
    q_lens, k_lens = [2, 3], [6, 7]
    cu_q = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(k_lens)]).astype(np.int32)
    q = _data((5, hq, d), 111, dt)
    kc, vc = _data((batch * bps, bs, hkv, d), 112, dt), _data((batch * bps, bs, hkv, d), 113, dt)
    for table in (np.arange(batch * bps, dtype=np.int32).reshape(batch, bps),
                  np.array([[3, 1], [0, 2]], dtype=np.int32)):
        out = high.flash_attn_varlen_func(H.to_dev(q, dt), H.to_dev(kc, dt), H.to_dev(vc, dt),
                                          torch.from_numpy(cu_q).to(dev), torch.from_numpy(cu_k).to(dev),
                                          3, 7, None, True, torch.from_numpy(table).to(dev))
        H.assert_ref_close(H.to_np(out), ob.attn_f64_varlen(q, kc, vc, cu_q, cu_k, block_table=table),
                           TOL[dt], "varlen paged")


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("sq", [1, 3, 20])
def test_kvcache_decode_and_chunked_prefill(dt, sq):
    # tests/high.rs:386-531: decode (sq == 1) and chunked prefill (sq > 1), here with permuted pages
    hq, hkv, d, bs = 8, 2, 64, 4
    lens = [sq + 5, sq, sq + 22, 37 + sq]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=60 + sq)
    kc, vc = H.round_to(kc, dt), H.round_to(vc, dt)
    q = _data((len(lens), sq, hq, d), 61, dt)
    out = high.flash_attn_with_kvcache(H.to_dev(q, dt), H.to_dev(kc, dt), H.to_dev(vc, dt),
                                       torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                       torch.from_numpy(table).cuda())
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    H.assert_ref_close(H.to_np(out), want, TOL[dt], f"kvcache sq={sq} {dt}")


def test_kvcache_rows_before_the_cache_output_zeros():
    # context shorter than the query chunk: rows at negative positions see nothing
    # (flash_attn_with_kvcache.cu:185-195,270-275)
    hq, hkv, d, bs, sq = 2, 1, 32, 4, 6
    lens = [4, 9]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=70)
    q = _data((2, sq, hq, d), 71, "f32")
    out = high.flash_attn_with_kvcache(H.to_dev(q, "f32"), H.to_dev(kc, "f32"), H.to_dev(vc, "f32"),
                                       torch.tensor(lens, dtype=torch.int32, device="cuda"), torch.from_numpy(table).cuda())
    got = H.to_np(out)
    assert np.all(got[0, :2] == 0.0)
    H.assert_ref_close(got, ob.attn_f64_kvcache(q, kc, vc, lens, table), H.F32_TOL, "short context")


def test_offset_views_are_bit_identical():
    # tests/high.rs:769-864: a tensor that starts at a non-zero element offset of a larger
    # allocation must give exactly the bits of a direct call
    b, s, hq, hkv, d = 1, 40, 4, 2, 64
    for dt in ("f32", "bf16"):
        q, k, v = _data((b, s, hq, d), 81, dt), _data((b, s, hkv, d), 82, dt), _data((b, s, hkv, d), 83, dt)
        direct = high.flash_attn_func(H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt))
        pad = 24  # elements; keeps 16-byte alignment for both storage widths
        def shifted(x):
            flat = torch.empty(x.size + pad, dtype=H.TORCH_DT[dt], device="cuda")
            flat[pad:] = H.to_dev(x, dt).reshape(-1)
            return flat[pad:].view(*x.shape)
        viewed = high.flash_attn_func(shifted(q), shifted(k), shifted(v))
        assert torch.equal(direct, viewed)


def test_host_tensor_call_matches_device_call():
    """flash_attn_func_host (pinned host tensors, batch elements and row chunks pipelined over the library's streams) gives
    the same bits as the device call, twice in a row (staging buffers and events are reused)."""
    torch.manual_seed(7)
    b, s, hq, hkv, d = 3, 300, 4, 2, 128
    q = torch.randn(b, s, hq, d).bfloat16().pin_memory()
    k = torch.randn(b, s, hkv, d).bfloat16().pin_memory()
    v = torch.randn(b, s, hkv, d).bfloat16().pin_memory()
    want = high.flash_attn_func(q.cuda(), k.cuda(), v.cuda()).cpu()
    out = torch.empty_like(q).pin_memory()
    for _ in range(2):
        out.zero_()
        got = high.flash_attn_func_host(q, k, v, out)
        torch.cuda.current_stream().synchronize()
        assert got is out
        assert torch.equal(out, want)
    with pytest.raises(L.Unsupported):
        high.flash_attn_func_host(q.cuda(), k, v)


@pytest.mark.parametrize("chunk_rows,start_pos,skv", [(128, 0, 700), (256, 0, 700), (200, 100, 800), (256, 50, 600)])
def test_host_tensor_call_in_row_chunks(chunk_rows, start_pos, skv):
    """The host call cut into row chunks (a chunked prefill whose K/V rows travel with the chunk that
    first sees them): same values as the one-piece device call, also with a start position, with a
    ragged last chunk and with K/V shorter than start_pos + the query rows."""
    torch.manual_seed(8)
    b, s, hq, hkv, d = 2, 700, 4, 2, 128
    q = torch.randn(b, s, hq, d).bfloat16().pin_memory()
    k = torch.randn(b, skv, hkv, d).bfloat16().pin_memory()
    v = torch.randn(b, skv, hkv, d).bfloat16().pin_memory()
    want = high.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), start_pos=start_pos).float().cpu()
    for _ in range(2):
        got = high.flash_attn_func_host(q, k, v, start_pos=start_pos, chunk_rows=chunk_rows)
        torch.cuda.current_stream().synchronize()
        # a chunk that starts inside a tile of the one-piece call groups the keys differently: same values, other rounding
        assert (got.float() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 4e-3), (torch.float32, 2e-4)])
def test_host_tensor_call_long_sequence_automatic_steps(dtype, tol):
    """A sequence long enough for the automatic cut (half-sequence chunks, the first and last one in
    pieces down to a sixteenth; K/V of the last chunk in one copy), after a smaller call, so that the
    staging buffers grow in between; pageable (not pinned) inputs are accepted as well; the buffers
    come back after flash_attn_release_workspaces."""
    from luma_b200 import ffi
    torch.manual_seed(9)
    small = [torch.randn(1, 200, 2, 64).to(dtype) for _ in range(3)]
    got = high.flash_attn_func_host(*small)
    torch.cuda.current_stream().synchronize()
    want = high.flash_attn_func(*(t.cuda() for t in small)).float().cpu()
    assert (got.float() - want).abs().max().item() <= tol
    b, s, hq, hkv, d = 2, 4608, 2, 1, 64
    assert len(high.host_steps(b, s)) > 2 * b
    q, k, v = torch.randn(b, s, hq, d).to(dtype), torch.randn(b, s, hkv, d).to(dtype), torch.randn(b, s, hkv, d).to(dtype)
    want = high.flash_attn_func(q.cuda(), k.cuda(), v.cuda()).float().cpu()
    for pinned in (True, False):
        args = [t.pin_memory() for t in (q, k, v)] if pinned else [q, k, v]
        got = high.flash_attn_func_host(*args)
        torch.cuda.current_stream().synchronize()
        assert (got.float() - want).abs().max().item() <= tol
    assert ffi.lib.flash_attn_release_workspaces() >= 1
    got = high.flash_attn_func_host(q, k, v)
    torch.cuda.current_stream().synchronize()
    assert (got.float() - want).abs().max().item() <= tol


def test_host_entry_point_status_codes():
    """flash_attn_host_<T> validates in the batched entry point's order before touching the device."""
    from luma_b200 import ffi
    q = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    f = ffi.lib.flash_attn_host_bf16
    p = q.data_ptr()
    assert f(None, p, p, p, 1, 8, 8, 2, 2, 64, 0, 0.125, 0, 0, None) == 1
    assert f(p, p, p, p, 1, 0, 8, 2, 2, 64, 0, 0.125, 0, 0, None) == 2
    assert f(p, p, p, p, 1, 8, 8, 3, 2, 64, 0, 0.125, 0, 0, None) == 2
    assert f(p, p, p, p, 1, 8, 8, 2, 2, 64, -1, 0.125, 0, 0, None) == 4
    assert f(p, p, p, p, 1, 8, 8, 2, 2, 48, 0, 0.125, 0, 0, None) == 3
    assert f(p, p, p, p, 1, 8, 8, 2, 2, 64, 0, 0.125, 99, 0, None) == 5
    assert b"no CUDA device 99" in ffi.lib.flash_attn_last_error()
