"""The collective boundary of the head-sharded attention path; mirrors the part of luma-dist that
path uses, over the C ABI of include/luma_dist_comm.h (NCCL called directly, no torch.distributed).

* `Comm.all_gather(tensor, dim)`   <- Comm::all_gather, luma-dist/src/base/comm.rs:212-214
                                       (-> backends/nccl/backend.rs:167-180)
* `Comm.from_rank` / `Comm.from_devices` <- NcclBackend::from_rank / from_devices,
                                       luma-dist/src/backends/nccl/mod.rs:56-64,26-42
* `init_process_group(rank, world, addr, port, device)` <- luma-dist/src/backends/nccl/mod.rs:238-252:
                                       rank 0 makes the NCCL unique id and serves it over TCP
* `MultiThread.run(n, fn)`          <- luma-dist/src/scheme/multi_thread.rs:25-48: one host thread per
                                       rank in one process, each handed its own communicator
"""
from __future__ import annotations

import ctypes
import socket
import threading
import time
from typing import Callable, List, Sequence

import torch

from . import ffi

_UNIQUE_ID_BYTES = 128


class CommError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        msg = ffi.lib.luma_comm_last_error()
        raise CommError(msg.decode("utf-8", "replace") if msg else "luma_comm: unknown failure")


def unique_id() -> bytes:
    buf = ctypes.create_string_buffer(_UNIQUE_ID_BYTES)
    _check(ffi.lib.luma_comm_unique_id(buf))
    return buf.raw


def gather_extents(shape, dim: int, elem_bytes: int):
    """What luma_comm_all_gather takes for a dense tensor of `shape` gathered along `dim`:
    (outer, chunk_bytes) = (product of the dims before `dim`, bytes of one rank's slab per outer index)."""
    outer = 1
    for s in shape[:dim]:
        outer *= int(s)
    chunk = int(elem_bytes)
    for s in shape[dim:]:
        chunk *= int(s)
    return outer, chunk


class Comm:
    """One rank's communicator. `all_gather(t, dim)` concatenates every rank's `t` along `dim`."""

    def __init__(self, handle: int):
        self._h = ctypes.c_void_p(handle)

    @staticmethod
    def from_rank(world: int, uid: bytes, rank: int, device: int) -> "Comm":
        out = ctypes.c_void_p()
        _check(ffi.lib.luma_comm_from_rank(ctypes.byref(out), world, ctypes.c_char_p(uid), rank, device))
        return Comm(out.value)

    @staticmethod
    def from_devices(devices: Sequence[int]) -> List["Comm"]:
        n = len(devices)
        outs = (ctypes.c_void_p * n)()
        devs = (ctypes.c_int * n)(*[int(d) for d in devices])
        _check(ffi.lib.luma_comm_from_devices(outs, n, devs))
        return [Comm(outs[i]) for i in range(n)]

    @property
    def rank(self) -> int:
        return int(ffi.lib.luma_comm_rank(self._h))

    @property
    def world_size(self) -> int:
        return int(ffi.lib.luma_comm_world_size(self._h))

    @property
    def device(self) -> int:
        return int(ffi.lib.luma_comm_device(self._h))

    def all_gather(self, t: torch.Tensor, dim: int, out: torch.Tensor = None, stream=None) -> torch.Tensor:
        """Result shape = t's with `dim` multiplied by the world size; rank r's data at block r."""
        if not t.is_cuda or not t.is_contiguous():
            raise CommError("all_gather: the tensor must be a contiguous CUDA tensor")
        dim = dim % t.dim()
        shape = list(t.shape)
        outer, chunk = gather_extents(shape, dim, t.element_size())
        shape[dim] *= self.world_size
        if out is None:
            out = torch.empty(shape, dtype=t.dtype, device=t.device)
        elif list(out.shape) != shape or out.dtype != t.dtype or not out.is_contiguous():
            raise CommError("all_gather: out must be contiguous, typed like the input, with dim scaled by the world size")
        if t.numel() == 0:
            return out
        st = stream if stream is not None else torch.cuda.current_stream(t.device)
        _check(ffi.lib.luma_comm_all_gather(self._h, t.data_ptr(), out.data_ptr(), outer, chunk, int(st.cuda_stream)))
        return out

    def barrier(self, stream=None) -> None:
        dev = torch.device("cuda", self.device)
        st = stream if stream is not None else torch.cuda.current_stream(dev)
        _check(ffi.lib.luma_comm_barrier(self._h, int(st.cuda_stream)))

    def destroy(self) -> None:
        if self._h is not None and self._h.value:
            ffi.lib.luma_comm_destroy(self._h)
            self._h = None


def init_process_group(rank: int, world: int, addr: str = "127.0.0.1", port: int = 29555, device: int = None,
                       timeout_s: float = 60.0) -> Comm:
    """One communicator per process: rank 0 makes the unique id and serves it to the world - 1 other
    ranks over TCP, then everyone joins (backends/nccl/mod.rs:238-252)."""
    device = rank if device is None else device
    if rank == 0:
        uid = unique_id()
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as srv:
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port))
            srv.listen(world)
            srv.settimeout(timeout_s)
            for _ in range(world - 1):
                conn, _peer = srv.accept()
                with conn:
                    conn.sendall(uid)
    else:
        deadline = time.time() + timeout_s
        uid = b""
        while True:
            try:
                with socket.create_connection((addr, port), timeout=5.0) as c:
                    while len(uid) < _UNIQUE_ID_BYTES:
                        part = c.recv(_UNIQUE_ID_BYTES - len(uid))
                        if not part:
                            break
                        uid += part
                if len(uid) == _UNIQUE_ID_BYTES:
                    break
                raise ConnectionError("short unique id")
            except OSError:
                uid = b""
                if time.time() > deadline:
                    raise CommError(f"init_process_group: rank {rank} could not reach rank 0 at {addr}:{port}") from None
                time.sleep(0.05)
    return Comm.from_rank(world, uid, rank, device)


class MultiThread:
    """The thread-per-rank launch scheme: `run(devices, fn)` starts one host thread per device in
    this process and calls fn(comm) in each with that rank's communicator; returns the results in
    rank order and re-raises the first exception."""

    @staticmethod
    def run(devices: Sequence[int], fn: Callable[[Comm], object]) -> list:
        comms = Comm.from_devices(devices)
        results = [None] * len(comms)
        errors = [None] * len(comms)

        def work(i):
            try:
                torch.cuda.set_device(comms[i].device)
                results[i] = fn(comms[i])
            except BaseException as exc:  # noqa: BLE001 - reported to the caller below
                errors[i] = exc

        threads = [threading.Thread(target=work, args=(i,)) for i in range(len(comms))]
        for th in threads:
            th.start()
        for th in threads:
            th.join()
        for c in comms:
            c.destroy()
        for e in errors:
            if e is not None:
                raise e
        return results
