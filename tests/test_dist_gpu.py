"""Head-sharded attention on 2, 4 and 8 GPUs (as many as the box has): every form of the output
all-gather must reproduce the unsharded result on EVERY rank, as luma-dist checks its collectives on
every rank (luma-dist/src/backends/nccl/tests.rs:60-90):

* prefill, fused: the tensor-core kernel's epilogue stores into every rank's output over peer memory
  (head sizes 128 and 64), whole sequence and in two row chunks, with the log-sum-exp gathered too, and
  through an NVSwitch multicast address (one multimem.st per 16 bytes) where the box offers one;
* prefill, two-step: attention on the shard, then the all-gather along the head axis
  (torch.distributed's NCCL, and this library's own communicator: luma_comm_all_gather);
* decode, fused: the split-K merge kernel stores into every rank's output; and two-step.

One process per GPU over NCCL; skipped on a box with a single GPU."""
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


def _worker(rank, world, port, port2, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        from luma_b200 import comm as fcomm
        from luma_b200 import ffi, high
        from luma_b200.dist import HeadAllGather, PeerOutput, shard_heads
        from oracle import binding as ob
        from tests import helpers as H

        def close(a, want):
            return bool(np.isfinite(a).all() and np.abs(a - want).max() <= H.BF16_MAX_ABS)

        own = fcomm.init_process_group(rank, world, "127.0.0.1", port2, device=rank)
        for d in (128, 64):
            b, s, hq, hkv = 1, 640, 16, 8
            q = H.round_to(H.normal((b, s, hq, d), 1 + d), "bf16")
            k = H.round_to(H.normal((b, s, hkv, d), 2 + d), "bf16")
            v = H.round_to(H.normal((b, s, hkv, d), 3 + d), "bf16")
            want, lse_want = ob.attn_f64_batch(q, k, v, return_lse=True)
            qs, kvs = shard_heads(hq, hkv, world, rank)
            ql = H.to_dev(q[:, :, qs], "bf16", dev).contiguous()
            kl = H.to_dev(k[:, :, kvs], "bf16", dev).contiguous()
            vl = H.to_dev(v[:, :, kvs], "bf16", dev).contiguous()
            # two-step: attention on the shard, then the all-gather along the head axis
            o_local = high.flash_attn_func(ql, kl, vl)
            gathered = HeadAllGather(dist.group.WORLD, o_local.shape, o_local.dtype, dev)(o_local)
            torch.cuda.synchronize()
            res[f"two_step_d{d}"] = close(H.to_np(gathered), want)
            # the same through this library's own communicator
            mine = own.all_gather(o_local, 2)
            torch.cuda.synchronize()
            res[f"own_comm_d{d}"] = bool(torch.equal(mine, gathered))
            # fused: the kernel stores into every rank's output; whole sequence, then in two row chunks
            peer = PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev, with_lse=True)
            peer.out.fill_(float("nan"))
            peer.lse.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            peer.fused_attention(ql, kl, vl, hq, qs.start, gather_lse=True)
            out = peer.sync()
            torch.cuda.synchronize()
            res[f"fused_d{d}"] = close(H.to_np(out), want) and ffi.device_status() == 0
            res[f"fused_equals_two_step_d{d}"] = bool(torch.equal(out, gathered))
            res[f"fused_lse_d{d}"] = bool(np.abs(peer.lse.cpu().numpy() - lse_want).max() <= 1e-3)
            torch.cuda.synchronize()
            dist.barrier()
            peer.out.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            half = 384
            peer.fused_attention(ql[:, :half].contiguous(), kl[:, :half].contiguous(), vl[:, :half].contiguous(), hq, qs.start,
                                 start_pos=0, row0=0)
            peer.fused_attention(ql[:, half:].contiguous(), kl, vl, hq, qs.start, start_pos=half, row0=half)
            out2 = peer.sync()
            torch.cuda.synchronize()
            res[f"fused_chunks_d{d}"] = close(H.to_np(out2), want)
            peer.close()
            # the same through an NVSwitch multicast address, where the box offers one (else the peer-pointer path again)
            peer = PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev, multicast=True)
            peer.out.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            peer.fused_attention(ql, kl, vl, hq, qs.start)
            out3 = peer.sync()
            torch.cuda.synchronize()
            res[f"fused_multicast_d{d}"] = bool(torch.equal(out3, gathered)) and ffi.device_status() == 0
            res[f"multicast_used_d{d}"] = True      # informational: which path ran is printed, both are valid
            if rank == 0:
                print(f"world {world} d {d}: multicast address {'used' if peer.mc_ptr else 'not available'}", flush=True)
            peer.close()

        # more ranks than KV heads: the one KV head is replicated on every rank, its 8 query heads are split
        b, s, hq, hkv, d = 1, 384, 8, 1, 128
        q = H.round_to(H.normal((b, s, hq, d), 41), "bf16")
        k = H.round_to(H.normal((b, s, hkv, d), 42), "bf16")
        v = H.round_to(H.normal((b, s, hkv, d), 43), "bf16")
        want = ob.attn_f64_batch(q, k, v)
        qs, kvs = shard_heads(hq, hkv, world, rank)
        peer = PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev)
        peer.out.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        peer.fused_attention(H.to_dev(q[:, :, qs], "bf16", dev).contiguous(), H.to_dev(k[:, :, kvs], "bf16", dev).contiguous(),
                             H.to_dev(v[:, :, kvs], "bf16", dev).contiguous(), hq, qs.start)
        out = peer.sync()
        torch.cuda.synchronize()
        res["replicated_kv_head"] = close(H.to_np(out), want)
        peer.close()

        # decode: every rank holds the cache slice of its KV heads; tables and lengths are replicated
        d, hq, hkv, bs = 128, 16, 8, 16
        lens = [700, 33, 1, 1500, 129]
        kc, vc, table = H.make_paged_cache(lens, bs, hkv, d, seed=9)
        kc, vc = H.round_to(kc, "bf16"), H.round_to(vc, "bf16")
        qd = H.round_to(H.normal((len(lens), 1, hq, d), 10), "bf16")
        want = ob.attn_f64_kvcache(qd, kc, vc, lens, table)
        qs, kvs = shard_heads(hq, hkv, world, rank)
        ql = H.to_dev(qd[:, :, qs], "bf16", dev).contiguous()
        kcl = H.to_dev(kc[:, :, kvs], "bf16", dev).contiguous()
        vcl = H.to_dev(vc[:, :, kvs], "bf16", dev).contiguous()
        td, ld = torch.from_numpy(table).to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)
        o_local = high.flash_attn_with_kvcache(ql, kcl, vcl, ld, td)
        two = own.all_gather(o_local, 2)
        torch.cuda.synchronize()
        res["decode_two_step"] = close(H.to_np(two), want)
        peer = PeerOutput(dist.group.WORLD, (len(lens), 1, hq, d), torch.bfloat16, dev)
        peer.out.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        peer.fused_decode(ql, kcl, vcl, td, ld, hq, qs.start)
        out = peer.sync()
        torch.cuda.synchronize()
        res["decode_fused"] = close(H.to_np(out), want) and bool(torch.equal(out, two))
        peer.close()
        own.barrier()
        torch.cuda.synchronize()
        own.destroy()
        ret[rank] = res
    finally:
        dist.destroy_process_group()


def _run_world(world):
    import torch.multiprocessing as mp
    port, port2 = _free_port(), _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, port2, ret)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=420)
    finally:
        # a worker that stalled must not stay behind holding its GPU and its mappings
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
    assert [p.exitcode for p in procs] == [0] * world
    got = dict(ret)
    assert sorted(got) == list(range(world))
    for r in range(world):
        bad = [k for k, ok in got[r].items() if not ok]
        assert not bad, f"rank {r} of {world}: {bad}"
        assert len(got[r]) == 19


@pytest.mark.parametrize("world", [2, 4, 8])
def test_every_form_of_the_head_all_gather_matches_unsharded_on_every_rank(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_world(world)
