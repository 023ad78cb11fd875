"""Host-side logic of the head-sharded path on CPU ranks (gloo, world_size 2): which heads a rank
owns, and that the all-gather along the head axis reassembles the unsharded tensor — the way
luma-dist tests its collectives with CPU ranks over loopback (luma-dist/src/backends/tcp/tests.rs)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from luma_b200.dist import shard_heads


def test_shard_heads_keeps_kv_groups_together():
    # Llama-3-70B attention shape over 8 ranks: 1 KV head + its 8 query heads per rank
    for world in (1, 2, 4, 8):
        seen_q, seen_kv = [], []
        for rank in range(world):
            q, kv = shard_heads(64, 8, world, rank)
            assert (q.stop - q.start) == 64 // world and (kv.stop - kv.start) == 8 // world
            assert q.start == kv.start * 8 and q.stop == kv.stop * 8
            seen_q += list(range(q.start, q.stop))
            seen_kv += list(range(kv.start, kv.stop))
        assert seen_q == list(range(64)) and seen_kv == list(range(8))
    # more ranks than KV heads: every KV head is replicated and its query heads are split
    for hq, hkv, world in ((32, 2, 8), (64, 8, 16), (8, 1, 4)):
        seen_q = []
        for rank in range(world):
            q, kv = shard_heads(hq, hkv, world, rank)
            assert kv.stop - kv.start == 1 and kv.start == rank // (world // hkv)
            assert q.stop - q.start == hq // world
            assert q.start // (hq // hkv) == kv.start and (q.stop - 1) // (hq // hkv) == kv.start   # inside that head's group
            seen_q += list(range(q.start, q.stop))
        assert seen_q == list(range(hq))
    with pytest.raises(ValueError):
        shard_heads(64, 8, 3, 0)
    with pytest.raises(ValueError):
        shard_heads(12, 4, 8, 0)      # 8 ranks over 4 KV heads would need the 3 heads of a group split in two
    with pytest.raises(ValueError):
        shard_heads(10, 4, 2, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from luma_b200.dist import HeadAllGather, all_gather_heads
        b, s, hq, hkv, d = 2, 5, 8, 4, 16
        g = torch.Generator().manual_seed(0)
        full = torch.randn(b, s, hq, d, generator=g)           # what an unsharded op would return
        qs, _ = shard_heads(hq, hkv, world, rank)
        local = full[:, :, qs, :].contiguous()
        out = all_gather_heads(local)
        ok = torch.equal(out, full)
        # the persistent form reuses its buffers across calls
        gather = HeadAllGather(dist.group.WORLD, local.shape, local.dtype, local.device)
        ok = ok and torch.equal(gather(local), full) and torch.equal(gather(local * 2), full * 2)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_all_gather_heads_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=120)
    finally:
        for p in procs:   # a rank that stalled must not stay behind
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
    assert [p.exitcode for p in procs] == [0] * world
    assert dict(ret) == {0: True, 1: True}
