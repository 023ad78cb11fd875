"""Packed variable-length prefill on the tcgen05 kernel against the f64 oracle, through the reference
signature (no row counts: the tiles at the very end of the packed buffers come in by plain loads)
and through the additive `_total` entry point (row counts as tensor-map bounds): ragged sequences
whose tiles overhang into the next sequence's rows, a last sequence that ends inside a tile (no
copy may reach past the buffers' ends), prefixes (kv longer than q, bottom-right causal), sequences
shorter than the grid's row range, GQA and MHA pairing, contiguous and paged K/V with permuted
block tables."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

D = 128
# (q lengths, kv lengths, hq, hkv)
CASES = [
    ([128, 128], [128, 128], 2, 2),                 # tile aligned
    ([100, 37, 260], [100, 37, 260], 4, 2),         # ragged: tiles overhang into the next sequence
    ([16, 300, 1, 129], [16, 300, 1, 129], 8, 2),   # a 1-row sequence between longer ones
    ([64, 200], [500, 333], 4, 4),                  # prefixes: kv longer than q
    ([513], [513], 2, 1),                           # one sequence ending one row into its fifth tile
    ([40, 700, 90], [300, 700, 1000], 6, 2),        # odd group, very different lengths
]


def _cu(lens):
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=[str(c[:2]) for c in CASES])
def test_varlen_contiguous_matches_oracle(case, dt):
    ql, kl, hq, hkv = case
    cu_q, cu_k = _cu(ql), _cu(kl)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q = H.round_to(H.normal((tq, hq, D), 11 + tq), dt)
    k = H.round_to(H.normal((tk, hkv, D), 12 + tq), dt)
    v = H.round_to(H.normal((tk, hkv, D), 13 + tq), dt)
    want = ob.attn_f64_varlen(q, k, v, cu_q, cu_k)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    cq = torch.from_numpy(cu_q).cuda()
    ck = torch.from_numpy(cu_k).cuda()
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_varlen(qd, kd, vd, o, cq, ck, len(ql), max(ql), max(kl), hq, hkv, D, 1.0 / np.sqrt(D),
                          total_q=tq, total_k=tk)      # the additive entry point: row counts bound the tensor maps
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"varlen {case} {dt}")

    # the reference signature carries no totals: same kernel, bit-identical output. The packed buffers
    # are followed by rows of NaN here: whatever is read past the last row would poison the result.
    def with_nan_tail(t):
        buf = torch.full((t.shape[0] + 160,) + tuple(t.shape[1:]), float("nan"), device="cuda", dtype=t.dtype)
        buf[:t.shape[0]] = t
        return buf[:t.shape[0]]
    qd, kd, vd = with_nan_tail(qd), with_nan_tail(kd), with_nan_tail(vd)
    o2 = torch.full_like(qd, float("nan"))
    sfx = "bf16" if dt == "bf16" else "f16"
    rc = getattr(ffi.lib, f"flash_attn_varlen_{sfx}")(
        qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o2.data_ptr(), cq.data_ptr(), ck.data_ptr(), None,
        len(ql), max(ql), max(kl), hq, hkv, D, 1, 0, 0, 1.0 / np.sqrt(D), None)
    torch.cuda.synchronize()
    assert rc == 0 and ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    assert torch.equal(o2, o)
    H.assert_bf16_close(H.to_np(o2), want, f"varlen (reference signature) {case} {dt}")


@pytest.mark.parametrize("block_size", [16, 64])
def test_varlen_paged_matches_oracle(block_size):
    dt = "bf16"
    ql, kl, hq, hkv = [50, 300, 129], [400, 300, 1000], 8, 2
    cu_q, cu_k = _cu(ql), _cu(kl)
    tq = int(cu_q[-1])
    rng = np.random.Generator(np.random.Philox(5))
    need = [(n + block_size - 1) // block_size for n in kl]
    max_blocks = max(need) + 1
    n_blocks = sum(need) + 3
    perm = rng.permutation(n_blocks).astype(np.int32)
    table = np.zeros((len(kl), max_blocks), dtype=np.int32)
    pos = 0
    for s, n in enumerate(need):
        table[s, :n] = perm[pos:pos + n]
        pos += n
    q = H.round_to(H.normal((tq, hq, D), 21), dt)
    kc = H.round_to(H.normal((n_blocks, block_size, hkv, D), 22), dt)
    vc = H.round_to(H.normal((n_blocks, block_size, hkv, D), 23), dt)
    want = ob.attn_f64_varlen(q, kc, vc, cu_q, cu_k, block_table=table)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(kc, dt), H.to_dev(vc, dt)
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_varlen(qd, kd, vd, o, torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda(), len(ql),
                          max(ql), max(kl), hq, hkv, D, 1.0 / np.sqrt(D),
                          block_tables=torch.from_numpy(table).cuda(), block_size=block_size)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"varlen paged bs={block_size}")
    # with the row count of q given (the additive entry point): the same bits
    o2 = torch.full_like(qd, float("nan"))
    low.flash_attn_varlen(qd, kd, vd, o2, torch.from_numpy(cu_q).cuda(), torch.from_numpy(cu_k).cuda(), len(ql),
                          max(ql), max(kl), hq, hkv, D, 1.0 / np.sqrt(D),
                          block_tables=torch.from_numpy(table).cuda(), block_size=block_size, total_q=tq)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and torch.equal(o2, o)


def test_varlen_neighbouring_rows_are_not_touched():
    """A tile that overhangs its sequence must not write the next sequence's rows (nor past the
    end of the buffer): rows are compared against a run in which each sequence is computed alone."""
    dt = "bf16"
    ql, hq, hkv = [70, 130, 5], 2, 2
    cu = _cu(ql)
    tq = int(cu[-1])
    q = H.round_to(H.normal((tq, hq, D), 31), dt)
    k = H.round_to(H.normal((tq, hkv, D), 32), dt)
    v = H.round_to(H.normal((tq, hkv, D), 33), dt)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    c = torch.from_numpy(cu).cuda()
    o = torch.zeros(tq + 128, hq, D, device="cuda", dtype=qd.dtype)   # slack rows after the packed end
    o[tq:] = 7.0
    low.flash_attn_varlen(qd, kd, vd, o[:tq], c, c, len(ql), max(ql), max(ql), hq, hkv, D, 1.0 / np.sqrt(D),
                          total_q=tq, total_k=tq)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert torch.all(o[tq:] == 7.0)
    want = ob.attn_f64_varlen(q, k, v, cu, cu)
    H.assert_bf16_close(H.to_np(o[:tq]), want, "varlen overhang")


def test_single_token_sequences_through_the_packed_entry_point():
    """A decode step written as a packed batch (every sequence one query token over a paged cache,
    the form continuous-batching callers use): takes the tensor-core kernel."""
    dt, block_size, hq, hkv = "bf16", 16, 8, 2
    kl = [1, 17, 400, 129, 1000]
    ql = [1] * len(kl)
    cu_q, cu_k = _cu(ql), _cu(kl)
    rng = np.random.Generator(np.random.Philox(9))
    need = [(n + block_size - 1) // block_size for n in kl]
    n_blocks = sum(need) + 2
    perm = rng.permutation(n_blocks).astype(np.int32)
    table = np.zeros((len(kl), max(need)), dtype=np.int32)
    pos = 0
    for s, n in enumerate(need):
        table[s, :n] = perm[pos:pos + n]
        pos += n
    q = H.round_to(H.normal((len(kl), hq, D), 91), dt)
    kc = H.round_to(H.normal((n_blocks, block_size, hkv, D), 92), dt)
    vc = H.round_to(H.normal((n_blocks, block_size, hkv, D), 93), dt)
    want = ob.attn_f64_varlen(q, kc, vc, cu_q, cu_k, block_table=table)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan"))
    low.flash_attn_varlen(qd, H.to_dev(kc, dt), H.to_dev(vc, dt), o, torch.from_numpy(cu_q).cuda(),
                          torch.from_numpy(cu_k).cuda(), len(kl), 1, max(kl), hq, hkv, D, 1.0 / np.sqrt(D),
                          block_tables=torch.from_numpy(table).cuda(), block_size=block_size)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, "single-token packed batch")


def test_single_row_batched_entry_point_with_start_pos():
    dt, b, skv, hq, hkv = "bf16", 3, 777, 8, 4
    q = H.round_to(H.normal((b, 1, hq, D), 94), dt)
    k = H.round_to(H.normal((b, skv, hkv, D), 95), dt)
    v = H.round_to(H.normal((b, skv, hkv, D), 96), dt)
    qd = H.to_dev(q, dt)
    o = torch.full_like(qd, float("nan"))
    low.flash_attn(qd, H.to_dev(k, dt), H.to_dev(v, dt), o, b, 1, skv, hq, hkv, D, skv - 1, 1.0 / np.sqrt(D))
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), ob.attn_f64_batch(q, k, v, start_pos=skv - 1), "single row, batched")
