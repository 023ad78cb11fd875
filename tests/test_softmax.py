"""Row softmax of the math path: the oracle (luma-cpu's online softmax) against an f64 formula on
CPU, and the CUDA kernels through the C ABI against the oracle — row lengths that take the
warp-per-row, CTA-per-row and two-pass kernels, unaligned lengths, -inf entries, an all -inf row,
in-place operation, f32 / f16 / bf16."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests import helpers as H


def _ref64(x):
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def test_oracle_softmax_matches_f64_formula():
    x = H.normal((37, 513), 5) * 3.0
    np.testing.assert_allclose(ob.softmax_last_dim_f32(x), _ref64(x), rtol=5e-6, atol=1e-9)   # f32 running sum of 513 terms
    x[3, 10:] = -np.inf   # masked tail, as the causal mask produces
    got = ob.softmax_last_dim_f32(x)
    assert np.all(got[3, 10:] == 0.0) and abs(got[3].sum() - 1.0) < 1e-6


# (rows, row_size): up to 1024 -> warp kernel; up to 32768 -> CTA kernel; beyond or unaligned -> two-pass
SHAPES = [(64, 8), (33, 256), (5, 1000), (17, 2048), (9, 4096), (3, 16384), (2, 40000), (7, 1001), (4, 77), (2, 33000)]


@pytest.mark.gpu
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(s) for s in SHAPES])
def test_softmax_kernel_matches_oracle(shape, dt):
    from luma_b200 import ffi, low
    rows, n = shape
    x = H.round_to(H.normal((rows, n), 11 + n) * 2.5, dt)
    if n > 20:
        x[0, n // 2:] = -np.inf   # a causally masked row
    want = ob.softmax_last_dim_f32(x)
    xd = H.to_dev(x, dt)
    got = low.softmax_last_dim(xd)
    torch.cuda.synchronize()
    assert ffi.last_path().startswith("softmax_")
    g = H.to_np(got)
    if dt == "f32":
        np.testing.assert_allclose(g, want, rtol=2e-5, atol=1e-9)   # f32 sums in a different order, ex2.approx
    else:
        # one rounding of the result to 8 (bf16) or 11 (f16) significant bits
        rel = 2.0 ** -8 if dt == "bf16" else 2.0 ** -11
        atol = 4e-8 if dt == "f16" else 1e-9   # f16 results below 6.1e-5 are subnormal: spacing 6e-8
        assert np.all(np.abs(g - want) <= (rel + 2e-5) * want + atol), np.abs(g - want).max()
    assert np.all(g[0, n // 2:] == 0.0) if n > 20 else True
    # in place gives the same bits
    y = xd.clone()
    low.softmax_last_dim(y, out=y)
    torch.cuda.synchronize()
    assert torch.equal(y, got)


@pytest.mark.gpu
def test_softmax_all_minus_inf_row_and_errors():
    import luma_b200 as L
    from luma_b200 import low
    x = torch.full((3, 64), float("-inf"), device="cuda")
    x[1] = 0.0
    y = low.softmax_last_dim(x)
    torch.cuda.synchronize()
    assert torch.isnan(y[0]).all() and torch.isnan(y[2]).all()      # as the reference's arithmetic gives
    assert torch.allclose(y[1], torch.full((64,), 1.0 / 64, device="cuda"))
    with pytest.raises(L.Unsupported):
        low.softmax_last_dim(torch.zeros(4, 8, device="cuda").t())
