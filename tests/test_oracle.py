"""CPU tests of the oracle itself: it must reproduce everything the reference's own tests pin for
this path before it is trusted as the checker."""
import math

import numpy as np
import pytest

from oracle import binding as ob


def test_known_answer_closed_form():
    # luma-tensor/src/tests/nn.rs:289-304: 2 tokens, 1 head, d=2, non-causal, default scale
    q = np.array([1, 0, 0, 1], dtype=np.float32).reshape(1, 2, 1, 2)
    k = q.copy()
    v = np.array([0, 1, 2, 0], dtype=np.float32).reshape(1, 2, 1, 2)
    y = ob.sdpa_math_f32(q, k, v, causal=False)
    s = 1.0 / math.sqrt(2.0)
    a = math.exp(s)
    e0, e1 = a / (a + 1.0), 1.0 / (a + 1.0)
    np.testing.assert_allclose(y.ravel(), [2 * e1, e0, 2 * e0, e1], rtol=0, atol=1e-6)
    # same case through the f64 loop is exact to 1e-12 (non-causal == start_pos large enough)
    y64 = ob.attn_f64_batch(q, k, v, start_pos=1)
    np.testing.assert_allclose(y64.ravel(), [2 * e1, e0, 2 * e0, e1], rtol=0, atol=1e-12)


def test_known_answer_causal():
    # causal variant of the same inputs: row 0 sees only key 0 -> v[0]; row 1 as above
    q = np.array([1, 0, 0, 1], dtype=np.float32).reshape(1, 2, 1, 2)
    v = np.array([0, 1, 2, 0], dtype=np.float32).reshape(1, 2, 1, 2)
    y = ob.sdpa_math_f32(q, q, v, causal=True)
    a = math.exp(1.0 / math.sqrt(2.0))
    np.testing.assert_allclose(y.ravel(), [0.0, 1.0, 2 * a / (a + 1), 1 / (a + 1)], atol=1e-6)


def _ramp(n):
    # luma-nn/tests/attention.rs:25-27
    i = np.arange(n, dtype=np.int64)
    return (((i * 7 + 3) % 17).astype(np.float64) / 17.0 - 0.5).astype(np.float32)


@pytest.mark.parametrize("b,lq,lk,hq,hkv,d,start_pos", [
    (2, 3, 5, 4, 2, 8, 2),     # causal GQA with start_pos=2 (luma-nn/tests/attention.rs:100-128)
    (1, 6, 6, 2, 2, 16, 0),
    (1, 5, 9, 8, 2, 32, 4),    # d=32 GQA 4:1
    (2, 33, 33, 8, 2, 64, 0),
])
def test_math_path_matches_f64_loop(b, lq, lk, hq, hkv, d, start_pos):
    q = _ramp(b * lq * hq * d).reshape(b, lq, hq, d)
    k = _ramp(b * lk * hkv * d + 5)[5:].reshape(b, lk, hkv, d)
    v = _ramp(b * lk * hkv * d + 11)[11:].reshape(b, lk, hkv, d)
    got, lse = ob.sdpa_math_f32(q, k, v, causal=True, start_pos=start_pos, return_lse=True)
    want, lse64 = ob.attn_f64_batch(q, k, v, start_pos=start_pos, return_lse=True)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-4)  # the reference's bar for Math vs f64
    np.testing.assert_allclose(lse, lse64, rtol=0, atol=1e-4)


def test_gqa_expansion_is_consecutive():
    # expand_heads repeats each KV head `group` times consecutively (attention.rs:95-103):
    # q heads 0,1 -> kv head 0; q heads 2,3 -> kv head 1
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 4, 4, 8), dtype=np.float32)
    k = rng.standard_normal((1, 4, 2, 8), dtype=np.float32)
    v = rng.standard_normal((1, 4, 2, 8), dtype=np.float32)
    y = ob.sdpa_math_f32(q, k, v)
    k_rep = np.repeat(k, 2, axis=2)
    v_rep = np.repeat(v, 2, axis=2)
    y_rep = ob.sdpa_math_f32(q, k_rep, v_rep)
    np.testing.assert_array_equal(y, y_rep)


def _xorshift_py(seed, n):
    mask = (1 << 64) - 1
    x = seed | 1
    out = []
    for _ in range(n):
        x ^= x >> 12
        x ^= (x << 25) & mask
        x ^= x >> 27
        r = (x * 0x2545F4914F6CDD1D) & mask
        out.append(r >> 40)
    return out


def test_xorshift_matches_definition():
    # tests/low.rs:363-384 and tests/high.rs:13-24, restated bit by bit in Python
    bits = _xorshift_py(6, 64)
    f32 = ob.XorShift(6).f32(64)
    want32 = (np.array(bits, dtype=np.float32) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    np.testing.assert_array_equal(f32, want32)
    f64 = ob.data_f64(64, 6)
    want64 = np.array(bits, dtype=np.float64) / float(1 << 24) * 2.0 - 1.0
    np.testing.assert_array_equal(f64, want64)
    assert f32.min() >= -1.0 and f32.max() < 1.0


def test_padding_mask_semantics():
    # tests/low.rs:63-98: masked keys invisible; a query whose own position is masked outputs zeros
    rng = ob.XorShift(10)
    b, sq, skv, hq, hkv, d, sp = 2, 5, 9, 2, 1, 8, 4
    q = rng.f32(b * sq * hq * d).reshape(b, sq, hq, d)
    k = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    v = rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d)
    mask = np.ones((b, skv), dtype=np.uint8)
    mask[0, 5] = 0   # query row 1 of batch 0 sits at position 5
    mask[1, 0] = 0
    o = ob.attn_f64_batch(q, k, v, start_pos=sp, mask=mask)
    assert np.all(o[0, 1] == 0.0)
    assert np.all(o[0, 0] != 0.0)
    # all-ones mask == no mask (tests/low.rs:236-243)
    np.testing.assert_array_equal(ob.attn_f64_batch(q, k, v, start_pos=sp, mask=np.ones_like(mask)),
                                  ob.attn_f64_batch(q, k, v, start_pos=sp))
    # dropping key 0 of batch 1 changes batch 1 only
    base = ob.attn_f64_batch(q, k, v, start_pos=sp)
    assert np.array_equal(o[0, 0], base[0, 0]) and not np.array_equal(o[1], base[1])


def test_block_slots_and_paged_equivalence():
    from tests.helpers import make_paged_cache, gather_paged
    lens = [1, 16, 17, 40, 0, 33]
    bs, hkv, d = 4, 2, 8
    kc, vc, table = make_paged_cache(lens, bs, hkv, d, seed=3)
    slots = ob.block_slots(table, lens, bs)
    want = np.concatenate([table[s, np.arange(l) // bs].astype(np.int64) * bs + np.arange(l) % bs
                           for s, l in enumerate(lens)]).astype(np.int32)
    np.testing.assert_array_equal(slots, want)
    # paged f64 attention == contiguous f64 attention on the gathered rows
    rng = np.random.default_rng(1)
    q = rng.standard_normal((len(lens), 1, 4, d))
    o = ob.attn_f64_kvcache(q, kc, vc, lens, table)
    for s, l in enumerate(lens):
        if l == 0:
            assert np.all(o[s] == 0.0)
            continue
        ks = gather_paged(kc, table[s], l, bs)[None]
        vs = gather_paged(vc, table[s], l, bs)[None]
        ref = ob.attn_f64_batch(q[s:s + 1], ks, vs, start_pos=l - 1)
        np.testing.assert_allclose(o[s:s + 1], ref, rtol=0, atol=1e-12)


def test_varlen_bottom_right_alignment():
    # tests/high.rs:249-290: seq0 q_len=3,k_len=5; seq1 q_len=4,k_len=4
    hq, hkv, d = 2, 2, 16
    cu_q, cu_k = [0, 3, 7], [0, 5, 9]
    q = ob.data_f64(7 * hq * d, 51).reshape(7, hq, d)
    k = ob.data_f64(9 * hkv * d, 52).reshape(9, hkv, d)
    v = ob.data_f64(9 * hkv * d, 53).reshape(9, hkv, d)
    o = ob.attn_f64_varlen(q, k, v, cu_q, cu_k)
    r0 = ob.attn_f64_batch(q[None, 0:3], k[None, 0:5], v[None, 0:5], start_pos=2)
    r1 = ob.attn_f64_batch(q[None, 3:7], k[None, 5:9], v[None, 5:9], start_pos=0)
    np.testing.assert_allclose(o[0:3], r0[0], atol=1e-12)
    np.testing.assert_allclose(o[3:7], r1[0], atol=1e-12)
