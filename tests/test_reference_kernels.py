"""Cross-check against the reference's OWN CUDA kernels, compiled unmodified from the reference
tree into oracle/_ref/libflash_attn_ref.so (oracle/Makefile, target `ref`). Both libraries export
the same ten symbols, so the same ctypes call drives either. Skipped where that file was not
built (the reference tree is not mounted on every machine)."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from luma_b200 import ffi
from oracle import binding as ob
from tests import helpers as H

pytestmark = pytest.mark.gpu

REF_PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libflash_attn_ref.so"


@pytest.fixture(scope="module")
def ref_lib():
    if not REF_PATH.exists():
        pytest.skip("oracle/_ref/libflash_attn_ref.so not built")
    lib = ctypes.CDLL(str(REF_PATH), mode=ctypes.RTLD_LOCAL)
    for s in ffi.DTYPE_SUFFIX:
        getattr(lib, f"flash_attn_{s}").argtypes = ffi._BATCH_ARGS
        getattr(lib, f"flash_attn_varlen_{s}").argtypes = ffi._VARLEN_ARGS
        getattr(lib, f"flash_attn_with_kvcache_{s}").argtypes = ffi._KVCACHE_ARGS
    return lib


@pytest.mark.parametrize("dt,tol", [("f32", 1e-4), ("f16", 2e-3), ("bf16", 2e-2)])
@pytest.mark.parametrize("shape", [(2, 70, 70, 8, 2, 128, 0), (1, 40, 72, 8, 2, 64, 32), (2, 300, 300, 4, 4, 128, 0),
                                   (1, 513, 513, 8, 2, 128, 0)])
def test_batched_matches_reference_kernels(ref_lib, shape, dt, tol):
    b, sq, skv, hq, hkv, d, sp = shape
    rng = ob.XorShift(sum(shape))
    q = H.to_dev(rng.f32(b * sq * hq * d).reshape(b, sq, hq, d), dt)
    k = H.to_dev(rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d), dt)
    v = H.to_dev(rng.f32(b * skv * hkv * d).reshape(b, skv, hkv, d), dt)
    mine, theirs = torch.empty_like(q), torch.empty_like(q)
    st = torch.cuda.current_stream().cuda_stream
    args = (b, sq, skv, hq, hkv, d, sp, 1.0 / np.sqrt(d), None, st)
    assert getattr(ffi.lib, f"flash_attn_{dt}")(q.data_ptr(), k.data_ptr(), v.data_ptr(), mine.data_ptr(), *args) == 0
    assert getattr(ref_lib, f"flash_attn_{dt}")(q.data_ptr(), k.data_ptr(), v.data_ptr(), theirs.data_ptr(), *args) == 0
    torch.cuda.synchronize()
    H.assert_ref_close(H.to_np(mine), H.to_np(theirs), tol, f"vs reference kernels {shape} {dt}")


@pytest.mark.parametrize("dt,tol", [("f32", 1e-4), ("bf16", 2e-2)])
@pytest.mark.parametrize("sq", [1, 7])
def test_kvcache_matches_reference_kernels(ref_lib, dt, tol, sq):
    hq, hkv, d, bs = 32, 8, 128, 16   # the reference decode kernel cannot launch beyond 32 q heads
    lens = [sq + 3, 200, 513, 64]
    kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=300)
    q = H.to_dev(H.normal((len(lens), sq, hq, d), 301), dt)
    kd, vd = H.to_dev(kc, dt), H.to_dev(vc, dt)
    bt = torch.from_numpy(table).cuda()
    cl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    mine, theirs = torch.empty_like(q), torch.empty_like(q)
    st = torch.cuda.current_stream().cuda_stream
    args = (bt.data_ptr(), cl.data_ptr(), len(lens), sq, hq, hkv, d, bs, table.shape[1], 1.0 / np.sqrt(d), st)
    assert getattr(ffi.lib, f"flash_attn_with_kvcache_{dt}")(q.data_ptr(), kd.data_ptr(), vd.data_ptr(), mine.data_ptr(), *args) == 0
    assert getattr(ref_lib, f"flash_attn_with_kvcache_{dt}")(q.data_ptr(), kd.data_ptr(), vd.data_ptr(), theirs.data_ptr(), *args) == 0
    torch.cuda.synchronize()
    H.assert_ref_close(H.to_np(mine), H.to_np(theirs), tol, f"kvcache vs reference kernels sq={sq} {dt}")
