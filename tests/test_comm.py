"""The collective boundary (include/luma_dist_comm.h through luma_b200/comm.py): NCCL called
directly, `all_gather(tensor, dim)` as luma-dist's Comm has it (luma-dist/src/base/comm.rs:212-214),
communicators made the two ways the reference makes them (from_rank / from_devices,
luma-dist/src/backends/nccl/mod.rs:26-64) and the thread-per-rank scheme
(luma-dist/src/scheme/multi_thread.rs:25-48). The reference checks its collectives on every rank
against the concatenation (luma-dist/src/backends/nccl/tests.rs:60-90); so do these."""
import pytest
import torch

from luma_b200 import comm as C


def test_gather_shape_arithmetic_needs_no_device():
    # (outer, chunk_bytes) of a (2, 5, 3, 4) bf16 tensor along each axis
    shape = [2, 5, 3, 4]
    assert C.gather_extents(shape, 0, 2) == (1, 240)
    assert C.gather_extents(shape, 1, 2) == (2, 120)
    assert C.gather_extents(shape, 2, 2) == (10, 24)
    assert C.gather_extents(shape, 3, 2) == (30, 8)
    with pytest.raises(C.CommError):
        C.Comm(0).all_gather(torch.zeros(2, 3), 0)          # host tensors are refused before anything is called


@pytest.mark.gpu
def test_single_rank_communicator_on_gpu():
    (comm,) = C.Comm.from_devices([0])
    try:
        assert comm.rank == 0 and comm.world_size == 1 and comm.device == 0
        x = torch.randn(3, 7, 2, 8, device="cuda:0").bfloat16()
        for dim in range(4):
            assert torch.equal(comm.all_gather(x, dim), x)
        comm.barrier()
        torch.cuda.synchronize()
    finally:
        comm.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_thread_per_rank_all_gather_along_every_axis(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    shape = (3, 6, 4, 16)
    full = [torch.randn(*shape, generator=torch.Generator().manual_seed(r)).bfloat16() for r in range(world)]

    def work(comm):
        dev = torch.device("cuda", comm.device)
        mine = full[comm.rank].to(dev)
        ok = True
        for dim in range(4):
            got = comm.all_gather(mine, dim)
            want = torch.cat([f.to(dev) for f in full], dim=dim)
            ok = ok and torch.equal(got, want)
        # uneven byte counts take the byte-wise interleave
        odd = torch.arange(5 * 3, dtype=torch.uint8, device=dev).view(5, 3) + comm.rank
        got = comm.all_gather(odd, 1)
        want = torch.cat([torch.arange(5 * 3, dtype=torch.uint8, device=dev).view(5, 3) + r for r in range(comm.world_size)], dim=1)
        ok = ok and torch.equal(got, want)
        comm.barrier()
        torch.cuda.synchronize(dev)
        return ok

    assert C.MultiThread.run(list(range(world)), work) == [True] * world
