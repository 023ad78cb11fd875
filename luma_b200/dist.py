"""Head-sharded attention across the GPUs of one box, joined by ONE all-gather of the outputs.

Plays the role of luma-dist's `Comm::all_gather(&tensor, dim)` (luma-dist/src/base/comm.rs:212-214
-> backends/nccl/backend.rs:167-180 -> backends/nccl/mod.rs:56-64) for the attention output. The
reference has no sharded attention: its all-gather permutes `dim` to the front, materialises,
zero-fills the receive buffer, gathers, permutes back and materialises again
(luma-dist/src/utils.rs:12-37). Here each rank's (B, S, H_local, d) output goes through a single
ncclAllGather into a persistent (G, B*S, H_local*d) staging buffer and one strided copy into the
final (B, S, G*H_local, d) tensor — no memset, no input-side copy.

Partitioning (rank g of G): KV heads [g*Hkv/G, (g+1)*Hkv/G) and the Hq/Hkv query heads of each
when G divides Hkv; with G a multiple of Hkv every KV head is replicated on G/Hkv ranks and its query
heads are split among them. Block tables and context lengths are replicated.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_heads(n_q_heads: int, n_kv_heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Query-head and KV-head slices owned by `rank`. While the world divides the KV heads, whole KV
    groups stay together. With more ranks than KV heads (the world a multiple of them) every KV head is
    replicated on world / n_kv_heads ranks and its group of query heads is split evenly among them; the
    query slices still tile the head axis in rank order, so the all-gather along it is unchanged."""
    if n_q_heads % n_kv_heads != 0:
        raise ValueError("q heads must be a multiple of kv heads")
    group = n_q_heads // n_kv_heads
    if n_kv_heads % world == 0:
        kv_per = n_kv_heads // world
        kv = slice(rank * kv_per, (rank + 1) * kv_per)
        return slice(kv.start * group, kv.stop * group), kv
    if world % n_kv_heads == 0 and group % (world // n_kv_heads) == 0:
        replicas = world // n_kv_heads            # ranks that share one KV head
        per = group // replicas                   # query heads of that group per rank
        head = rank // replicas
        q0 = head * group + (rank % replicas) * per
        return slice(q0, q0 + per), slice(head, head + 1)
    raise ValueError(f"world size {world} must divide kv heads {n_kv_heads}, or be a multiple of them that divides "
                     f"the {group} query heads of a group")


class HeadAllGather:
    """all_gather of (B, S, H_local, d) along the head axis into a reused (B, S, G*H_local, d)."""

    def __init__(self, group, local_shape, dtype, device):
        self.group = group
        self.world = dist.get_world_size(group)
        b, s, h, d = local_shape
        self.local_shape = tuple(local_shape)
        self.staging = torch.empty((self.world * b * s, h * d), dtype=dtype, device=device)
        self.out = torch.empty((b, s, self.world * h, d), dtype=dtype, device=device)
        self.launches = 2  # the NCCL kernel and the interleaving copy

    def __call__(self, o_local: torch.Tensor) -> torch.Tensor:
        assert tuple(o_local.shape) == self.local_shape and o_local.is_contiguous()
        b, s, h, d = self.local_shape
        dist.all_gather_into_tensor(self.staging, o_local.view(b * s, h * d), group=self.group)
        # (G, B*S, H*d) -> (B*S, G, H*d): one pass over the gathered data
        self.out.view(b * s, self.world, h * d).copy_(self.staging.view(self.world, b * s, h * d).permute(1, 0, 2))
        return self.out


def all_gather_heads(o_local: torch.Tensor, group=None) -> torch.Tensor:
    """One-shot form of HeadAllGather (allocates its buffers); also runs on the gloo backend."""
    group = group if group is not None else dist.group.WORLD
    g = HeadAllGather(group, o_local.shape, o_local.dtype, o_local.device)
    return g(o_local.contiguous())


class PeerOutput:
    """The full attention output (B, S, Hq_total, d), allocated on every rank and mapped into every
    other rank of the group through CUDA IPC (luma_ipc_export / luma_ipc_open of the C ABI), so that
    a kernel on one GPU can store its heads straight into all copies (plain stores over NVLink;
    nothing here uses TMA or multicast). With `with_lse` a (B, Hq_total, S) f32 log-sum-exp tensor
    is shared the same way.

    With `multicast=True` the output is allocated as symmetric memory (torch.distributed._symmetric_memory:
    the same allocation on every rank, bound to one NVSwitch multicast object where the hardware and the
    driver offer it) and `fused_attention` stores through the multicast address: one `multimem.st` per 16
    bytes reaches every rank's copy, so a GPU sends its shard once instead of once per peer. Where
    multicast is not on offer (`self.mc_ptr == 0`, agreed across the group) the peer-pointer path is used.

    `fused_attention` runs the head-sharded prefill with the gather fused into its epilogue,
    `fused_decode` the head-sharded single-token decode with the gather fused into its merge kernel;
    `sync()` then synchronises the group, after which `self.out` (and `self.lse`) hold every rank's heads.
    """

    def __init__(self, group, shape, dtype, device, with_lse=False, multicast=False):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.lse = torch.empty((shape[0], shape[2], shape[1]), dtype=torch.float32, device=device) if with_lse else None
        self._opened = []        # mapped peer pointers, closed by close()
        self._symm = None
        self.mc_ptr = 0
        self.out = None
        if multicast:
            self._try_symmetric(shape, dtype, device)
        if self.out is None:
            self.out = torch.empty(shape, dtype=dtype, device=device)
            self.ptrs = self._exchange(self.out)
        self.lse_ptrs = self._exchange(self.lse) if with_lse else None
        self._flag = torch.zeros(1, device=device)
        dist.barrier(group=group)

    def _try_symmetric(self, shape, dtype, device):
        """Symmetric allocation + rendezvous; leaves self.out None when this build or box cannot do it."""
        try:
            import torch.distributed._symmetric_memory as symm
            out = symm.empty(tuple(shape), dtype=dtype, device=device)
            hdl = symm.rendezvous(out, self.group)
            off = int(getattr(hdl, "offset", 0))
            ptrs = [int(p) + off for p in hdl.buffer_ptrs]
            ok = ptrs[self.rank] == out.data_ptr()
            mc = int(hdl.multicast_ptr) if ok else 0
        except Exception:   # noqa: BLE001 - any failure means: no symmetric memory here
            out, hdl, ptrs, mc, off, ok = None, None, None, 0, 0, False
        # every rank must take the same path
        flag = torch.tensor([1 if ok else 0, 1 if mc else 0], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag[0]) == 1:
            self.out, self._symm, self.ptrs = out, hdl, ptrs
            self.mc_ptr = (mc + off) if int(flag[1]) == 1 else 0

    def _exchange(self, t):
        """Every rank's device pointer to its own copy of `t`, as seen from THIS process."""
        import ctypes
        from . import ffi
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_longlong(0)
        if ffi.lib.luma_ipc_export(t.data_ptr(), handle, ctypes.byref(offset)) != 0:
            raise RuntimeError(ffi.lib.luma_comm_last_error().decode())
        mine = (handle.raw, int(offset.value))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        ptrs = []
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            p = ctypes.c_void_p()
            if ffi.lib.luma_ipc_open(ctypes.c_char_p(h), off, ctypes.byref(p)) != 0:
                raise RuntimeError(ffi.lib.luma_comm_last_error().decode())
            self._opened.append(p.value)
            ptrs.append(p.value)
        return ptrs

    def fused_attention(self, q, k, v, q_heads_total, q_head_offset, start_pos=0, scale=None, row0=0, lse=None,
                        gather_lse=False):
        """q (B, Sq, Hq_local, d), k/v (B, Skv, Hkv_local, d): this rank's shard. Writes rows
        [row0, row0 + Sq) of every rank's output (and, with `gather_lse`, this rank's heads of every
        rank's LSE; whole sequences only). Call `sync()` before reading `self.out`."""
        from . import low
        b, sq, hq_l, d = q.shape
        skv, hkv_l = k.shape[1], k.shape[2]
        scale = float(scale) if scale is not None else 1.0 / (d ** 0.5)
        s_total = self.out.shape[1]
        assert b == self.out.shape[0] and (row0 == 0 or b == 1)
        esz = self.out.element_size()
        off = row0 * q_heads_total * d * esz
        # with row0 > 0 (b == 1) the call addresses a row range of the output; the kernel's batch
        # stride then never matters because batch == 1
        ptrs = [p + off for p in self.ptrs]
        assert sq + row0 <= s_total
        lse_ptrs = None
        if gather_lse:
            assert self.lse_ptrs is not None and row0 == 0 and sq == s_total
            lse_ptrs = self.lse_ptrs
        if self.mc_ptr and lse_ptrs is None:
            low.flash_attn_allgather_multicast(q, k, v, self.mc_ptr + off, q_heads_total, q_head_offset, b, sq, skv, hq_l,
                                               hkv_l, d, int(start_pos), scale, None, lse)
            return
        low.flash_attn_allgather(q, k, v, ptrs, q_heads_total, q_head_offset, b, sq, skv, hq_l, hkv_l, d,
                                 int(start_pos), scale, None, lse, lse_ptrs)

    def fused_decode(self, q, k_cache, v_cache, block_tables, context_lens, q_heads_total, q_head_offset, scale=None):
        """q (B, 1, Hq_local, d) and this rank's cache slice (num_blocks, page, Hkv_local, d): one
        decode step whose merge kernel writes this rank's heads into every rank's (B, 1, Hq_total, d)."""
        from . import low
        b, one, hq_l, d = q.shape
        assert one == 1 and tuple(self.out.shape) == (b, 1, q_heads_total, d)
        scale = float(scale) if scale is not None else 1.0 / (d ** 0.5)
        low.flash_attn_with_kvcache_allgather(q, k_cache, v_cache, self.ptrs, q_heads_total, q_head_offset, block_tables,
                                              context_lens, b, hq_l, k_cache.shape[2], d, k_cache.shape[1],
                                              block_tables.shape[1], scale)

    def sync(self):
        """Every rank's stores have landed everywhere once all ranks passed this point."""
        dist.all_reduce(self._flag, group=self.group)
        return self.out

    def close(self):
        """Drops the mappings of the peers' buffers. Collective: every rank calls it, after which no
        rank touches another rank's buffer again, so the owners may free them in any order."""
        from . import ffi
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self._opened:
            ffi.lib.luma_ipc_close(p)
        self._opened = []
        self._symm = None
        self.mc_ptr = 0
        self.ptrs = [self.out.data_ptr()]
        self.lse_ptrs = None
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
