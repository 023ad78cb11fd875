"""Head-sharded prefill on two GPUs: the fused path (epilogue stores into every rank's output over
peer memory) and the two-step path (attention, then all-gather) must both reproduce the unsharded
result. One process per GPU over NCCL; skipped on a box with a single GPU."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from luma_b200 import ffi, high
        from luma_b200.dist import HeadAllGather, PeerOutput, shard_heads
        from oracle import binding as ob
        from tests import helpers as H
        b, s, hq, hkv, d = 1, 640, 8, 4, 128
        q = H.round_to(H.normal((b, s, hq, d), 1), "bf16")
        k = H.round_to(H.normal((b, s, hkv, d), 2), "bf16")
        v = H.round_to(H.normal((b, s, hkv, d), 3), "bf16")
        want = ob.attn_f64_batch(q, k, v)
        qs, kvs = shard_heads(hq, hkv, world, rank)
        ql = H.to_dev(q[:, :, qs], "bf16", dev).contiguous()
        kl = H.to_dev(k[:, :, kvs], "bf16", dev).contiguous()
        vl = H.to_dev(v[:, :, kvs], "bf16", dev).contiguous()
        # two-step: attention on the shard, then the all-gather along the head axis
        o_local = high.flash_attn_func(ql, kl, vl)
        gathered = HeadAllGather(dist.group.WORLD, o_local.shape, o_local.dtype, dev)(o_local)
        torch.cuda.synchronize()
        ok_two_step = float(np.abs(H.to_np(gathered) - want).max()) <= H.BF16_MAX_ABS
        # fused: the kernel stores into every rank's output; whole sequence, then in two row chunks
        peer = PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev)
        peer.out.fill_(float("nan"))
        dist.barrier()
        peer.fused_attention(ql, kl, vl, hq, qs.start)
        out = peer.sync()
        torch.cuda.synchronize()
        ok_fused = float(np.abs(H.to_np(out) - want).max()) <= H.BF16_MAX_ABS and ffi.device_status() == 0
        same = torch.equal(out, gathered)
        peer.out.fill_(float("nan"))
        dist.barrier()
        half = 384
        peer.fused_attention(ql[:, :half], kl[:, :half], vl[:, :half], hq, qs.start, start_pos=0, row0=0)
        peer.fused_attention(ql[:, half:], kl, vl, hq, qs.start, start_pos=half, row0=half)
        out2 = peer.sync()
        torch.cuda.synchronize()
        ok_chunks = float(np.abs(H.to_np(out2) - want).max()) <= H.BF16_MAX_ABS
        ret[rank] = (ok_two_step, ok_fused, bool(same), ok_chunks)
    finally:
        dist.destroy_process_group()


def test_fused_and_two_step_all_gather_match_unsharded():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert dict(ret) == {0: (True, True, True, True), 1: (True, True, True, True)}
