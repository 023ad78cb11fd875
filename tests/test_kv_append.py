"""KV-cache append (additive kernel): rows must land bit for bit in the slots a host walk of the
block table gives, for every storage width, ragged lengths and page sizes; then a decode over
the appended cache must equal a decode over a cache that was filled on the host."""
import numpy as np
import pytest
import torch

from luma_b200 import low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("bs,n_new", [(16, 1), (16, 40), (5, 7), (1, 3), (32, 64)])
def test_append_writes_exactly_the_slots_of_the_table(bs, n_new, dt):
    hkv, d = 4, 64
    lens = np.array([n_new, n_new + 13, 200, 3 if n_new > 3 else n_new, 129], dtype=np.int32)
    pool = int(sum((l + bs - 1) // bs for l in lens)) + 7
    _, _, table = H.make_paged_cache(lens, bs, hkv, d, seed=bs + n_new, pool_blocks=pool)
    tdt = H.TORCH_DT[dt]
    k_new = torch.randn(len(lens), n_new, hkv, d, device="cuda").to(tdt)
    v_new = torch.randn(len(lens), n_new, hkv, d, device="cuda").to(tdt)
    k_cache = torch.full((pool, bs, hkv, d), -7.0, device="cuda").to(tdt)
    v_cache = torch.full((pool, bs, hkv, d), -9.0, device="cuda").to(tdt)
    want_k, want_v = k_cache.clone().cpu(), v_cache.clone().cpu()
    low.kvcache_append(k_new, v_new, k_cache, v_cache, torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda(),
                       len(lens), n_new, hkv, d, bs, table.shape[1])
    torch.cuda.synchronize()
    slots = ob.block_slots(table, lens, bs)
    offs = np.concatenate([[0], np.cumsum(lens)])
    wk, wv = want_k.view(pool * bs, hkv, d), want_v.view(pool * bs, hkv, d)
    for s, L in enumerate(lens):
        for t in range(n_new):
            j = L - n_new + t
            if j < 0:
                continue
            wk[slots[offs[s] + j]] = k_new[s, t].cpu()
            wv[slots[offs[s] + j]] = v_new[s, t].cpu()
    assert torch.equal(k_cache.cpu(), want_k) and torch.equal(v_cache.cpu(), want_v)


def test_append_then_decode_equals_host_filled_cache():
    hq, hkv, d, bs = 8, 2, 128, 16
    lens = [33, 500, 64]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=3)
    kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
    q = H.round_to(H.normal((3, 1, hq, d), 4), "bf16")
    want = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    # device cache that lacks the newest token of every sequence, then append it
    k_dev, v_dev = H.to_dev(kc, "bf16"), H.to_dev(vc, "bf16")
    last = [H.gather_paged(kc, table[s], L, bs)[-1] for s, L in enumerate(lens)]
    lastv = [H.gather_paged(vc, table[s], L, bs)[-1] for s, L in enumerate(lens)]
    slots = ob.block_slots(table, lens, bs)
    offs = np.concatenate([[0], np.cumsum(lens)])
    for s, L in enumerate(lens):
        k_dev.view(-1, hkv, d)[slots[offs[s] + L - 1]] = 0
        v_dev.view(-1, hkv, d)[slots[offs[s] + L - 1]] = 0
    k_new = H.to_dev(np.stack(last)[:, None], "bf16")
    v_new = H.to_dev(np.stack(lastv)[:, None], "bf16")
    tb, cl = torch.from_numpy(table).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda")
    low.kvcache_append(k_new, v_new, k_dev, v_dev, tb, cl, 3, 1, hkv, d, bs, table.shape[1])
    o = torch.empty(3, 1, hq, d, device="cuda", dtype=torch.bfloat16)
    low.flash_attn_with_kvcache(H.to_dev(q, "bf16"), k_dev, v_dev, o, tb, cl, 3, 1, hq, hkv, d, bs, table.shape[1], 1.0 / np.sqrt(d))
    torch.cuda.synchronize()
    H.assert_bf16_close(H.to_np(o), want, "append then decode")
