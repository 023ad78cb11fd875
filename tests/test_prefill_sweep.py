"""Seeded sweep of the tcgen05 prefill kernel against the f64 oracle over shapes drawn at random:
batch, GQA widths, ragged and tile-aligned lengths, start positions that are and are not multiples
of the tile (aligned diagonal tiles take a specialised softmax step), kv longer than needed, head
sizes 64 and 128, bf16 and f16 — a guard against shape-dependent slips in the tile, band and mask arithmetic."""
import numpy as np
import pytest
import torch

from luma_b200 import ffi, low
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    out = []
    for i in range(n):
        hkv = int(rng.choice([1, 2, 3, 4]))
        group = int(rng.choice([1, 2, 4, 5]))
        b = int(rng.integers(1, 4))
        sq = int(rng.choice([int(rng.integers(16, 700)), 128 * int(rng.integers(1, 6))]))
        sp_kind = int(rng.integers(0, 3))
        sp = 0 if sp_kind == 0 else (128 * int(rng.integers(1, 4)) if sp_kind == 1 else int(rng.integers(1, 300)))
        extra = int(rng.choice([0, 0, int(rng.integers(1, 200))]))
        skv = sp + sq + extra if rng.random() < 0.8 else max(1, sp + sq - int(rng.integers(1, sq)))
        dt = "bf16" if i % 3 else "f16"
        d = 64 if i % 4 == 1 else 128
        out.append((b, sq, skv, hkv * group, hkv, sp, dt, d))
    return out


CASES = _cases(36, 2024)


@pytest.mark.parametrize("case", CASES, ids=[str(c) for c in CASES])
def test_prefill_sweep(case):
    b, sq, skv, hq, hkv, sp, dt, d = case
    q = H.round_to(H.normal((b, sq, hq, d), 101 + sq), dt)
    k = H.round_to(H.normal((b, skv, hkv, d), 102 + skv), dt)
    v = H.round_to(H.normal((b, skv, hkv, d), 103 + sq + skv), dt)
    want, lse_want = ob.attn_f64_batch(q, k, v, start_pos=sp, return_lse=True)
    qd, kd, vd = H.to_dev(q, dt), H.to_dev(k, dt), H.to_dev(v, dt)
    o = torch.full_like(qd, float("nan"))
    lse = torch.full((b, hq, sq), float("nan"), device="cuda", dtype=torch.float32)
    low.flash_attn(qd, kd, vd, o, b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), None, None, lse)
    torch.cuda.synchronize()
    assert ffi.last_path() == "prefill_tcgen05"
    assert ffi.device_status() == 0
    H.assert_bf16_close(H.to_np(o), want, f"sweep {case}")
    np.testing.assert_allclose(lse.cpu().numpy(), lse_want, rtol=0, atol=1e-3)
