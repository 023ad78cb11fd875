"""Head size 32 with 16-bit storage on the tensor-core prefill kernel: the tiles are the 64-column tiles
of the head-size-64 kernel whose upper 32 columns the copy engine fills with zeros (the tensor maps
carry the real inner extent), so every entry point that kernel serves takes head size 32 too — batched
(start positions, key-padding mask, LSE), packed varlen (contiguous with and without the buffers' row
counts, and paged), chunked prefill over the paged cache. Outputs are NaN-poisoned first and the
buffers are followed by NaN rows: nothing beyond a row's 32 columns may be read into the result or
written. A single-token step over the paged cache takes the split-K decode kernel at head size 32 as well."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu
D = 32


def _guarded(x, dt):
    """Device copy of x with 64 NaN rows after it (same allocation), to catch reads and writes past the end."""
    t = H.to_dev(x, dt)
    flat = torch.full((t.numel() + 64 * t.shape[-1] * t.shape[-2],), float("nan"), device="cuda", dtype=t.dtype)
    flat[:t.numel()] = t.reshape(-1)
    return flat[:t.numel()].view(*t.shape), flat


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 64, 64, 4, 4, 0), (3, 129, 200, 6, 6, 0), (2, 50, 120, 4, 4, 70),
                                   (1, 700, 700, 8, 2, 0), (2, 300, 428, 5, 5, 128), (1, 1, 96, 4, 4, 95)])
def test_batched_head_size_32(shape, dt):
    b, sq, skv, hq, hkv, sp = shape
    q = H.round_to(H.normal((b, sq, hq, D), 1 + sq), dt)
    k = H.round_to(H.normal((b, skv, hkv, D), 2 + skv), dt)
    v = H.round_to(H.normal((b, skv, hkv, D), 3 + sq), dt)
    want, lse_want = ob.attn_f64_batch(q, k, v, start_pos=sp, return_lse=True)
    (qd, _), (kd, _), (vd, _) = _guarded(q, dt), _guarded(k, dt), _guarded(v, dt)
    o, o_all = _guarded(np.full(q.shape, np.nan, dtype=np.float32), dt)
    lse = torch.full((b, hq, sq), float("nan"), device="cuda", dtype=torch.float32)
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, D, sp, 1.0 / np.sqrt(D), None, None, lse)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"head size 32 batched {shape} {dt}")
    np.testing.assert_allclose(lse.cpu().numpy(), lse_want, rtol=0, atol=1e-3)
    assert torch.isnan(o_all[o.numel():].float()).all()          # nothing written past the output


def test_batched_head_size_32_with_padding_mask():
    b, sq, skv, hq, hkv, sp = 2, 33, 100, 8, 4, 67
    q = H.round_to(H.normal((b, sq, hq, D), 11), "bf16")
    k = H.round_to(H.normal((b, skv, hkv, D), 12), "bf16")
    v = H.round_to(H.normal((b, skv, hkv, D), 13), "bf16")
    mask = (np.random.Generator(np.random.Philox(14)).random((b, skv)) > 0.3).astype(np.uint8)
    want = ob.attn_f64_batch(q, k, v, start_pos=sp, mask=mask)
    o = torch.full((b, sq, hq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn(H.to_dev(q, "bf16"), H.to_dev(k, "bf16"), H.to_dev(v, "bf16"), o, b, sq, skv, hq, hkv, D, sp,
                   1.0 / np.sqrt(D), torch.from_numpy(mask).cuda())
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, "head size 32 with a key-padding mask")


@pytest.mark.parametrize("totals", [True, False])
def test_varlen_head_size_32(totals):
    hq, hkv = 4, 2
    ql, kl = [100, 37, 260, 1], [300, 37, 260, 129]
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(kl)]).astype(np.int32)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q = H.round_to(H.normal((tq, hq, D), 21), "bf16")
    k = H.round_to(H.normal((tk, hkv, D), 22), "bf16")
    v = H.round_to(H.normal((tk, hkv, D), 23), "bf16")
    want = ob.attn_f64_varlen(q, k, v, cu_q, cu_k)
    (qd, _), (kd, _), (vd, _) = _guarded(q, "bf16"), _guarded(k, "bf16"), _guarded(v, "bf16")
    o, o_all = _guarded(np.full(q.shape, np.nan, dtype=np.float32), "bf16")
    kw = dict(total_q=tq, total_k=tk) if totals else {}
    low.flash_attn_varlen(qd, kd, vd, o, torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda(), len(ql), max(ql),
                          max(kl), hq, hkv, D, 1.0 / np.sqrt(D), **kw)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"head size 32 packed varlen (row counts given: {totals})")
    assert torch.isnan(o_all[o.numel():].float()).all()


@pytest.mark.parametrize("bs", [8, 16, 128])
def test_paged_head_size_32(bs):
    hq, hkv, sq = 8, 2, 130
    lens = [sq + 300, sq, sq + 1, 1000 + sq, sq + 129]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, D, seed=30 + bs)
    kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
    q = H.round_to(H.normal((len(lens), sq, hq, D), 31), "bf16")
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    o = torch.full((len(lens), sq, hq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    td, ld = torch.from_numpy(table).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda")
    low.flash_attn_with_kvcache(H.to_dev(q, "bf16"), H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16"), o, td, ld, len(lens), sq, hq,
                                hkv, D, bs, table.shape[1], 1.0 / np.sqrt(D))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"head size 32 chunked prefill over pages of {bs}")
    # the packed entry point over the same paged cache
    cu_q = (np.arange(len(lens) + 1) * sq).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    o2 = torch.full((len(lens) * sq, hq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn_varlen(H.to_dev(q.reshape(-1, hq, D), "bf16"), H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16"), o2,
                          torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda(), len(lens), sq, max(lens), hq, hkv, D,
                          1.0 / np.sqrt(D), block_tables=td, block_size=bs, total_q=len(lens) * sq)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    assert torch.equal(o2.view_as(o), o)
    # one token per sequence: the split-K decode kernel
    q1 = H.round_to(H.normal((len(lens), 1, hq, D), 32), "bf16")
    o1 = torch.full((len(lens), 1, hq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn_with_kvcache(H.to_dev(q1, "bf16"), H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16"), o1, td, ld, len(lens), 1, hq,
                                hkv, D, bs, table.shape[1], 1.0 / np.sqrt(D))
    torch.cuda.synchronize()
    assert ffi.last_path() == "decode_splitk"
    H.assert_bf16_close(H.to_np(o1), ob.attn_f64_kvcache(q1, kc, vc, lens, table), "head size 32 single-token step")
