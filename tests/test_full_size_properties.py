"""The two headline configurations at their full sizes, through properties that need no full-size
oracle run: prefill B=4, Hq=Hkv=32, S=2048, d=128 (bf16, LSE) and paged decode batch 64, Hq=32,
Hkv=8, d=128, page 16, contexts in [512, 8192] from a 40 000-page pool.

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
