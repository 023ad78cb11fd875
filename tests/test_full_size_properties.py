"""Every benchmarked configuration at its full size, through properties that need no full-size
oracle run, plus an oracle slice of each:

* prefill B=4, Hq=Hkv=32, S=2048, d=128 (bf16, LSE);
* GQA prefill B=2, Hq=32, Hkv=8, S=8192, d=128 (inputs N(0,1)*0.5);
* the head-sharded shape on one GPU: prefill B=1, Hq=64, Hkv=8, S=16384, and paged decode batch 256,
  contexts in [1024, 32768], page 16 (a pool of more than 2^31 elements per tensor);
* paged decode batch 64, Hq=32, Hkv=8, d=128, page 16, contexts in [512, 8192] from a 40 000-page pool;
* the CPU-runnable case exactly: f32, B=1, H=8, S=256, d=64, inputs from seed 0, against the f32 math path.

* V of all ones -> every output is 1 (the weights of a row sum to one);
* linearity in V: attn(q, k, a*v1 + v2) = a*attn(q, k, v1) + attn(q, k, v2) within the output rounding;
* causality: changing K/V after position t leaves the rows up to t bit-identical;
* permuting where the pages of the cache live leaves the decode output bit-identical;
* a slice (one batch element and two heads / three sequences) against the f64 oracle.
"""
import math

import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _prefill(q, k, v, lse=None):
    b, s, hq, d = q.shape
    o = torch.empty_like(q)
    low.flash_attn(q, k, v, o, b, s, k.shape[1], hq, k.shape[2], d, 0, 1.0 / math.sqrt(d), None, None, lse)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    return o


def test_prefill_full_config_properties():
    b, h, s, d = 4, 32, 2048, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    q = torch.randn(b, s, h, d, generator=g, device="cuda").bfloat16()
    k = torch.randn(b, s, h, d, generator=g, device="cuda").bfloat16()
    v1 = torch.randn(b, s, h, d, generator=g, device="cuda").bfloat16()
    v2 = torch.randn(b, s, h, d, generator=g, device="cuda").bfloat16()
    lse = torch.empty(b, h, s, device="cuda", dtype=torch.float32)

    ones = _prefill(q, k, torch.ones_like(v1))
    assert (ones.float() - 1.0).abs().max().item() <= 2.0 ** -7      # bf16 rounding of P and of the result

    o1 = _prefill(q, k, v1, lse)
    o2 = _prefill(q, k, v2)
    v3 = (2.0 * v1.float() + v2.float()).bfloat16()
    o3 = _prefill(q, k, v3)
    err = (o3.float() - (2.0 * o1.float() + o2.float())).abs()
    assert err.max().item() <= 6e-2 and err.mean().item() <= 4e-3    # three roundings of values of size ~3

    # causality: perturb K and V from position 1000 on
    t = 1000
    k2, v4 = k.clone(), v1.clone()
    k2[:, t:] = torch.randn(b, s - t, h, d, generator=g, device="cuda").bfloat16()
    v4[:, t:] = 0
    o4 = _prefill(q, k2, v4)
    assert torch.equal(o4[:, :t], o1[:, :t])
    assert not torch.equal(o4[:, t:], o1[:, t:])

    # a slice against the oracle: batch element 1, heads 5 and 30
    heads = [5, 30]
    qs, ks, vs = (x[1:2, :, heads].float().cpu().numpy() for x in (q, k, v1))
    want, lse_want = ob.attn_f64_batch(qs, ks, vs, start_pos=0, return_lse=True)
    H.assert_bf16_close(o1[1:2, :, heads].float().cpu().numpy(), want, "config-2 slice")
    np.testing.assert_allclose(lse[1:2, heads].cpu().numpy(), lse_want, rtol=0, atol=1e-3)


def test_decode_full_config_properties():
    batch, hq, hkv, d, page, lo, hi, pool = 64, 32, 8, 128, 16, 512, 8192, 40000
    rng = np.random.Generator(np.random.Philox(4))
    lens = rng.integers(lo, hi + 1, size=batch).astype(np.int32)
    need = (lens.astype(np.int64) + page - 1) // page
    perm = rng.permutation(pool).astype(np.int32)
    max_blocks = hi // page
    table = np.full((batch, max_blocks), -1, dtype=np.int32)
    pos = 0
    for i, n in enumerate(need):
        table[i, :n] = perm[pos:pos + n]
        pos += int(n)
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    kc = torch.randn(pool, page, hkv, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    vc = torch.randn(pool, page, hkv, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    q = torch.randn(batch, 1, hq, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    lens_d, table_d = torch.from_numpy(lens).cuda(), torch.from_numpy(table).cuda()
    scale = 1.0 / math.sqrt(d)

    def decode(kcache, vcache, tab):
        o = torch.empty_like(q)
        low.flash_attn_with_kvcache(q, kcache, vcache, o, tab, lens_d, batch, 1, hq, hkv, d, page, max_blocks, scale)
        torch.cuda.synchronize()
        assert ffi.last_path() == "decode_splitk"
        return o

    o = decode(kc, vc, table_d)
    ones = decode(kc, torch.ones_like(vc), table_d)
    assert (ones.float() - 1.0).abs().max().item() <= 2.0 ** -7

    # move every page to another physical slot: same logical cache, same bits out
    where = torch.from_numpy(rng.permutation(pool).astype(np.int64)).cuda()    # old page p now lives at where[p]
    kc2, vc2 = torch.empty_like(kc), torch.empty_like(vc)
    kc2[where] = kc
    vc2[where] = vc
    table2 = table.copy()
    valid = table >= 0
    table2[valid] = where.cpu().numpy()[table[valid]].astype(np.int32)
    o2 = decode(kc2, vc2, torch.from_numpy(table2).cuda())
    assert torch.equal(o2, o)

    # three sequences against the oracle (the shortest, the longest and one in between)
    order = np.argsort(lens)
    pick = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
    used = np.unique(table[pick][table[pick] >= 0])
    remap = {int(p): i for i, p in enumerate(used)}
    sub_table = np.full((len(pick), max_blocks), 0, dtype=np.int32)
    for r, sidx in enumerate(pick):
        n = int(need[sidx])
        sub_table[r, :n] = [remap[int(p)] for p in table[sidx, :n]]
    used_d = torch.from_numpy(used.astype(np.int64)).cuda()
    want = ob.attn_f64_kvcache(q[pick].float().cpu().numpy(), kc[used_d].float().cpu().numpy(),
                               vc[used_d].float().cpu().numpy(), lens[pick], sub_table, scale)
    H.assert_bf16_close(o[pick].float().cpu().numpy(), want, "config-4 slice")


def _linearity_and_ones(q, k, v1, v2):
    ones = _prefill(q, k, torch.ones_like(v1))
    assert (ones.float() - 1.0).abs().max().item() <= 2.0 ** -7
    o1 = _prefill(q, k, v1)
    o2 = _prefill(q, k, v2)
    o3 = _prefill(q, k, (2.0 * v1.float() + v2.float()).bfloat16())
    err = (o3.float() - (2.0 * o1.float() + o2.float())).abs()
    scale = max(1.0, float(v1.float().abs().max()))
    assert err.max().item() <= 6e-2 * scale and err.mean().item() <= 4e-3 * scale
    return o1


def _math_path_slice(q, k, v, o, batch_index, q_heads, group, what):
    """Query heads `q_heads` (each with its own KV head) of one batch element against the f32 math
    path of luma-cpu as the oracle restates it (matmul, scale, causal mask, softmax, matmul)."""
    for h in q_heads:
        kvh = h // group
        qs = q[batch_index:batch_index + 1, :, h:h + 1].float().cpu().numpy()
        ks = k[batch_index:batch_index + 1, :, kvh:kvh + 1].float().cpu().numpy()
        vs = v[batch_index:batch_index + 1, :, kvh:kvh + 1].float().cpu().numpy()
        want = ob.sdpa_math_f32(qs, ks, vs, causal=True)
        H.assert_bf16_close(o[batch_index:batch_index + 1, :, h:h + 1].float().cpu().numpy(), want, f"{what}, head {h}")


def test_gqa_prefill_s8192_full_config_properties():
    b, hq, hkv, s, d = 2, 32, 8, 8192, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    q = (torch.randn(b, s, hq, d, generator=g, device="cuda") * 0.5).bfloat16()
    k = (torch.randn(b, s, hkv, d, generator=g, device="cuda") * 0.5).bfloat16()
    v1 = (torch.randn(b, s, hkv, d, generator=g, device="cuda") * 0.5).bfloat16()
    v2 = (torch.randn(b, s, hkv, d, generator=g, device="cuda") * 0.5).bfloat16()
    o1 = _linearity_and_ones(q, k, v1, v2)
    # causality: perturb K and V from position 5000 on
    t = 5000
    k2, v4 = k.clone(), v1.clone()
    k2[:, t:] = torch.randn(b, s - t, hkv, d, generator=g, device="cuda").bfloat16()
    v4[:, t:] = 0
    o4 = _prefill(q, k2, v4)
    assert torch.equal(o4[:, :t], o1[:, :t]) and not torch.equal(o4[:, t:], o1[:, t:])
    _math_path_slice(q, k, v1, o1, 1, [5, 30], hq // hkv, "GQA S=8192 slice")


def test_head_sharded_shape_prefill_s16384_on_one_gpu():
    b, hq, hkv, s, d = 1, 64, 8, 16384, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(50)
    q = torch.randn(b, s, hq, d, generator=g, device="cuda").bfloat16()
    k = torch.randn(b, s, hkv, d, generator=g, device="cuda").bfloat16()
    v1 = torch.randn(b, s, hkv, d, generator=g, device="cuda").bfloat16()
    v2 = torch.randn(b, s, hkv, d, generator=g, device="cuda").bfloat16()
    o1 = _linearity_and_ones(q, k, v1, v2)
    _math_path_slice(q, k, v1, o1, 0, [41], hq // hkv, "Hq=64 S=16384 slice")
    # the same heads computed as the 8-way shard would compute them: one KV head and its 8 query heads alone
    kvh = 5
    qs = q[:, :, kvh * 8:(kvh + 1) * 8].contiguous()
    o_shard = _prefill(qs, k[:, :, kvh:kvh + 1].contiguous(), v1[:, :, kvh:kvh + 1].contiguous())
    assert torch.equal(o_shard, o1[:, :, kvh * 8:(kvh + 1) * 8])


def test_head_sharded_shape_decode_batch256_on_one_gpu():
    batch, hq, hkv, d, page, lo, hi = 256, 64, 8, 128, 16, 1024, 32768
    rng = np.random.Generator(np.random.Philox(51))
    lens = rng.integers(lo, hi + 1, size=batch).astype(np.int32)
    need = (lens.astype(np.int64) + page - 1) // page
    pool = int(need.sum() * 1.15) + 1
    assert pool * page * hkv * d > 2 ** 31      # element offsets need 64 bits
    perm = rng.permutation(pool).astype(np.int32)
    max_blocks = hi // page
    table = np.full((batch, max_blocks), -1, dtype=np.int32)
    pos = 0
    for i, n in enumerate(need):
        table[i, :n] = perm[pos:pos + n]
        pos += int(n)
    g = torch.Generator(device="cuda")
    g.manual_seed(51)
    kc = torch.empty(pool, page, hkv, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.empty_like(kc)
    step = 8192
    for i in range(0, pool, step):
        n = min(step, pool - i)
        kc[i:i + n] = torch.randn(n, page, hkv, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
        vc[i:i + n] = torch.randn(n, page, hkv, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    q = torch.randn(batch, 1, hq, d, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    lens_d, table_d = torch.from_numpy(lens).cuda(), torch.from_numpy(table).cuda()
    scale = 1.0 / math.sqrt(d)

    def decode(kcache, vcache, tab):
        o = torch.full_like(q, float("nan"))
        low.flash_attn_with_kvcache(q, kcache, vcache, o, tab, lens_d, batch, 1, hq, hkv, d, page, max_blocks, scale)
        torch.cuda.synchronize()
        assert ffi.last_path() == "decode_splitk"
        return o

    o = decode(kc, vc, table_d)
    assert torch.isfinite(o.float()).all()
    # three sequences against the oracle (the shortest, the longest and one in between)
    order = np.argsort(lens)
    pick = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
    used = np.unique(table[pick][table[pick] >= 0])
    remap = {int(p): i for i, p in enumerate(used)}
    sub_table = np.full((len(pick), max_blocks), 0, dtype=np.int32)
    for r, sidx in enumerate(pick):
        n = int(need[sidx])
        sub_table[r, :n] = [remap[int(p)] for p in table[sidx, :n]]
    used_d = torch.from_numpy(used.astype(np.int64)).cuda()
    want = ob.attn_f64_kvcache(q[pick].float().cpu().numpy(), kc[used_d].float().cpu().numpy(),
                               vc[used_d].float().cpu().numpy(), lens[pick], sub_table, scale)
    H.assert_bf16_close(o[pick].float().cpu().numpy(), want, "batch-256 decode slice")
    # one KV head's cache slice alone (what one of eight ranks holds): the same values for its 8 query heads
    kvh = 3
    o_shard = torch.full((batch, 1, 8, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn_with_kvcache(q[:, :, kvh * 8:(kvh + 1) * 8].contiguous(), kc[:, :, kvh:kvh + 1].contiguous(),
                                vc[:, :, kvh:kvh + 1].contiguous(), o_shard, table_d, lens_d, batch, 1, 8, 1, d, page,
                                max_blocks, scale)
    torch.cuda.synchronize()
    # (the split-K chunk is chosen by the number of work items, so the shard may cut its contexts elsewhere: same values, other rounding)
    assert (o_shard.float() - o[:, :, kvh * 8:(kvh + 1) * 8].float()).abs().max().item() <= 2e-3
    # V of all ones -> every output is 1 (V overwritten in place: the pool is 10 GB)
    vc.fill_(1.0)
    ones = decode(kc, vc, table_d)
    assert (ones.float() - 1.0).abs().max().item() <= 2.0 ** -7
    # move every page to another physical slot: same logical cache, same bits out (K in place of V's buffer)
    where = torch.from_numpy(rng.permutation(pool).astype(np.int64)).cuda()    # old page p now lives at where[p]
    vc[where] = kc                                                              # vc now holds the relocated K
    table2 = table.copy()
    valid = table >= 0
    table2[valid] = where.cpu().numpy()[table[valid]].astype(np.int32)
    table2_d = torch.from_numpy(table2).cuda()
    # attention with V := K at the old and at the new placement
    o_kk = decode(kc, kc, table_d)
    o_kk2 = decode(vc, vc, table2_d)
    assert torch.equal(o_kk2, o_kk)


def test_cpu_runnable_case_exactly():
    """f32, B=1, H=8, S=256, d=64, Q/K/V ~ N(0,1) drawn in that order from one Philox stream of seed 0,
    scale 1/sqrt(64), causal: the f32 entry point against the f32 math path at the reference's f32
    bar, and the same values rounded to bf16 through the tensor-core kernel at the 16-bit bar. The
    result is (B, S, H, d); the head-major (1, 8, 256, 64) view is its transpose."""
    b, h, s, d = 1, 8, 256, 64
    rng = np.random.Generator(np.random.Philox(0))
    q = rng.standard_normal((b, s, h, d), dtype=np.float32)
    k = rng.standard_normal((b, s, h, d), dtype=np.float32)
    v = rng.standard_normal((b, s, h, d), dtype=np.float32)
    want = ob.sdpa_math_f32(q, k, v, scale=1.0 / 8.0, causal=True)
    qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    o = torch.full_like(qd, float("nan"))
    low.flash_attn(qd, kd, vd, o, b, s, s, h, h, d, 0, 1.0 / 8.0)
    torch.cuda.synchronize()
    H.assert_ref_close(o.cpu().numpy(), want, H.F32_TOL, "f32 case against the math path")
    assert o.permute(0, 2, 1, 3).shape == (1, 8, 256, 64)
    qb, kb, vb = (H.round_to(x, "bf16") for x in (q, k, v))
    want_b = ob.sdpa_math_f32(qb, kb, vb, scale=1.0 / 8.0, causal=True)
    ob16 = torch.full((b, s, h, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    low.flash_attn(H.to_dev(qb, "bf16"), H.to_dev(kb, "bf16"), H.to_dev(vb, "bf16"), ob16, b, s, s, h, h, d, 0, 1.0 / 8.0)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05" and ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(ob16), want_b, "bf16 case against the math path")
