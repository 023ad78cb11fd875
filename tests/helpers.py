"""Shared helpers of the parity tests: seeded inputs, bf16 rounding, tolerances, paged caches."""
from __future__ import annotations

import numpy as np
import torch

# north_star tolerance for bf16 outputs against the f32 oracle on identical inputs
BF16_MAX_ABS = 2e-2
BF16_MEAN_ABS = 2e-3
# the reference's own bars (luma-flash-attn/tests/low.rs:129, tests/high.rs:135,537)
F32_TOL = 3e-3
F16_TOL = 1e-2
BF16_REF_TOL = 5e-2

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def normal(shape, seed, scale=1.0):
    """Seeded N(0,1)*scale as float32 (counter-based Philox stream, one per seed)."""
    rng = np.random.Generator(np.random.Philox(seed))
    return (rng.standard_normal(size=shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def round_to(x: np.ndarray, dt: str) -> np.ndarray:
    """Values of `x` after rounding to the storage type, widened back to float32."""
    if dt == "f32":
        return np.asarray(x, dtype=np.float32)
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(TORCH_DT[dt]).to(torch.float32).numpy()


def to_dev(x: np.ndarray, dt: str, device="cuda:0") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device).to(TORCH_DT[dt])


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def assert_ref_close(got, want, tol, what=""):
    """The reference's criterion: |got - want| <= tol + tol*|want| elementwise, all finite."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    diff = np.abs(got - want)
    bad = diff > tol + tol * np.abs(want)
    if bad.any():
        i = np.unravel_index(np.argmax(diff * bad), diff.shape)
        raise AssertionError(f"{what}: idx {i} got {got[i]} want {want[i]} diff {diff[i]} (tol {tol}); {bad.sum()} bad")


def assert_bf16_close(got, want, what=""):
    """north_star criterion for 16-bit outputs: max abs <= 2e-2 and mean abs <= 2e-3."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    diff = np.abs(got - want)
    assert diff.max() <= BF16_MAX_ABS, f"{what}: max abs err {diff.max()} > {BF16_MAX_ABS}"
    assert diff.mean() <= BF16_MEAN_ABS, f"{what}: mean abs err {diff.mean()} > {BF16_MEAN_ABS}"


def make_paged_cache(lens, block_size, hkv, d, seed, pool_blocks=None, permute=True, scale=1.0):
    """Builds a paged K/V cache with a seeded random permutation of physical pages.

    Returns (k_cache, v_cache, block_table) as numpy: caches (num_blocks, block_size, hkv, d)
    float32 filled with N(0,1) for the WHOLE pool, block_table (num_seqs, max_blocks) int32 with -1
    in unused entries (never dereferenced by a correct kernel).
    """
    lens = np.asarray(lens, dtype=np.int64)
    need = [int((l + block_size - 1) // block_size) for l in lens]
    total = int(sum(need))
    if pool_blocks is None:
        pool_blocks = max(total + 3, 1)
    assert pool_blocks >= total
    rng = np.random.Generator(np.random.Philox(seed + 7919))
    perm = rng.permutation(pool_blocks) if permute else np.arange(pool_blocks)
    max_blocks = max(max(need), 1)
    table = np.full((len(lens), max_blocks), -1, dtype=np.int32)
    pos = 0
    for s, n in enumerate(need):
        table[s, :n] = perm[pos:pos + n]
        pos += n
    k_cache = normal((pool_blocks, block_size, hkv, d), seed + 1, scale)
    v_cache = normal((pool_blocks, block_size, hkv, d), seed + 2, scale)
    return k_cache, v_cache, table


def gather_paged(cache, table_row, length, block_size):
    """Contiguous (length, hkv, d) view of one sequence of a paged cache (numpy)."""
    j = np.arange(length)
    slots = table_row[j // block_size].astype(np.int64) * block_size + j % block_size
    flat = cache.reshape(-1, cache.shape[2], cache.shape[3])
    return flat[slots]
