#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--only NAME]

Prints ONE JSON line. A "step" is one pass of the headline workload:

* one GPU: the GQA prefill the 60 %-of-peak target is quoted on — causal bf16, B=2, Hq=32, Hkv=8,
  S=8192, d=128 ("prefill_c3");
* N > 1 GPUs (torchrun, one rank per GPU): the head-sharded shape — Hq=64, Hkv=8, d=128, B=1,
  S=16384 ("prefill_c5"), total work fixed and split by KV-head groups over the ranks (strong
  scaling); every rank ends with the full output: the all-gather is fused into the kernel's epilogue
  (peer stores over NVLink) and sits inside the timed region.

The other configurations are measured as well and reported, compactly, under "workloads" (each
with its fraction of the measured and of the nominal peak); "--only NAME" restricts the run to one.
At every N the run also checks, outside the timed region, what the timed calls produced
("parity"): at N > 1 every rank recomputes, alone, the heads another rank owns and compares them
bit for bit with what arrived in its gathered output; at N = 1 a slice is recomputed on the library's
independent SIMT kernel.

Beside the CPU baseline the line carries "reference_cuda": the reference's own CUDA kernels (compiled
unmodified for sm_100a into oracle/_ref where the reference tree was mounted at build time), device-timed
on the S=8192 prefill and the batch-64 decode, outside the timed region, as a second stated baseline.

`--impl reference` times the CPU restatement of luma-cpu's math-path attention (oracle/) on the
host cores, on the same workload definition: the reference's own implementation of this path is
Rust and cannot be built with this image's toolchains.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0
NOMINAL_NVLINK_GBS = 900.0
# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from
# the ncu captures summarised under profiles/: the three prefill workloads were captured at full size
# (five metrics, one or two passes); a head-sharded run divides the figure by the number of GPUs (every
# GPU processes its share of the heads; q, k, v and o shard with them). The decode figure is the ratio
# measured on decode_c4_small (397.9 MB moved for 394.2 MB of algorithmic bytes, L2 hit rate 0.1 %:
# traffic grows in proportion to the cached tokens) applied to the run's own bytes.
NCU_TRAFFIC_BYTES = {"prefill_c2": 201_468_672 + 49_486_080, "prefill_c3": 202_012_928 + 101_843_968,
                     "prefill_c5": 666_307_840 + 230_259_968}
NCU_DECODE_TRAFFIC_RATIO = (394_186_496 + 3_808_768) / 394_223_184
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# name -> (batch, q heads, kv heads, sequence, head size, seed, input scale, with LSE)
PREFILL = {
    "prefill_c2": (4, 32, 32, 2048, 128, 2, 1.0, True),
    "prefill_c3": (2, 32, 8, 8192, 128, 3, 0.5, False),
    "prefill_c3_small": (1, 8, 2, 8192, 128, 3, 0.5, False),     # same kernel and head layout, short ncu capture
    "prefill_c5": (1, 64, 8, 16384, 128, 50, 1.0, False),
}
# name -> (sequences, q heads, kv heads, head size, page, shortest, longest context, pool pages, seed)
DECODE = {
    "decode_c4": (64, 32, 8, 128, 16, 512, 8192, 40000, 4),
    "decode_c4_small": (16, 32, 8, 128, 16, 512, 8192, 12000, 4),  # 0.8 GB of cache: same kernel, short ncu capture
    "decode_c5": (256, 64, 8, 128, 16, 1024, 32768, None, 51),
}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


def causal_flops(b, hq, sq, skv, d, start_pos=0):
    """4*d FLOPs per visible (query, key) pair; row i sees min(skv, start_pos + i + 1) keys."""
    i = np.arange(sq, dtype=np.int64)
    vis = np.minimum(skv, start_pos + i + 1).sum()
    return int(4 * d * b * hq * int(vis))


def prefill_config(name, world=1):
    b, hq, hkv, s, d, _seed, _sc, lse = PREFILL[name]
    cfg = {"workload": name, "batch": b, "q_heads": hq, "kv_heads": hkv, "seq_len": s, "head_dim": d, "causal": True,
           "lse": lse, "flops_per_step": causal_flops(b, hq, s, s, d), "l2": "inputs larger than L2"}
    if world > 1:
        cfg["parallelism"] = f"kv-head groups over {world} GPUs, fused all-gather of O"
    return cfg


# ------------------------------------------------------------------------------------------
# host placement: keep a rank's pinned buffers and threads on the NUMA node of its GPU
# ------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(torch, index):
    """Restricts this process to the CPUs that are local to GPU `index` (from sysfs), so that pinned
    staging buffers allocated afterwards come from that node. Returns the CPU list or None."""
    try:
        props = torch.cuda.get_device_properties(index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        text = Path(f"/sys/bus/pci/devices/{bus}/local_cpulist").read_text().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return text
    except Exception:
        pass
    return None


# ------------------------------------------------------------------------------------------
# clocks sampling
# ------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, torch=None, step=None, barrier=None, repeats=None):
        """Ends the sampling and summarises it. The timed region of a step is a few milliseconds,
        shorter than nvidia-smi's start-up: when `step` is given, the same step is first repeated,
        untimed, for about 0.35 s so that there are samples under this very load."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        if step is not None and torch is not None:
            # with several ranks the caller passes `repeats` (every rank must make the same number of
            # collective calls); alone the count comes from one timed call
            if repeats is None:
                t0 = time.time()
                step()
                torch.cuda.synchronize()
                repeats = int(0.35 / max(time.time() - t0, 1e-5))
            for _ in range(max(1, min(20000, int(repeats)))):
                step()
            torch.cuda.synchronize()
            if barrier is not None:
                barrier()
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


# ------------------------------------------------------------------------------------------
# inputs
# ------------------------------------------------------------------------------------------
def make_prefill(torch, dev, b, hq, hkv, s, d, seed, scale_in=1.0):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    q = (torch.randn(b, s, hq, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    k = (torch.randn(b, s, hkv, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    v = (torch.randn(b, s, hkv, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    return q, k, v


def make_decode(torch, dev, batch, hq, hkv, d, page, lo, hi, pool_pages, seed, q_seed=None):
    """Paged cache with a seeded permutation of physical pages; `q_seed` (default: seed) seeds the
    query rows alone, so that ranks sharing a cache seed still ask different questions."""
    rng = np.random.Generator(np.random.Philox(seed))
    lens = rng.integers(lo, hi + 1, size=batch).astype(np.int32)
    need = (lens.astype(np.int64) + page - 1) // page
    if pool_pages is None:
        pool_pages = int(need.sum() * 1.15) + 1
    assert need.sum() <= pool_pages
    perm = rng.permutation(pool_pages).astype(np.int32)
    max_blocks = int(math.ceil(hi / page))
    table = np.full((batch, max_blocks), -1, dtype=np.int32)
    pos = 0
    for s_, n in enumerate(need):
        table[s_, :n] = perm[pos:pos + n]
        pos += int(n)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    kc = torch.empty(pool_pages, page, hkv, d, device=dev, dtype=torch.bfloat16)
    vc = torch.empty_like(kc)
    step = 4096
    for i in range(0, pool_pages, step):
        n = min(step, pool_pages - i)
        kc[i:i + n] = torch.randn(n, page, hkv, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        vc[i:i + n] = torch.randn(n, page, hkv, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q = make_decode_q(torch, dev, batch, hq, d, seed if q_seed is None else q_seed)
    return q, kc, vc, torch.from_numpy(lens).to(dev), torch.from_numpy(table).to(dev), lens


def make_decode_q(torch, dev, batch, hq, d, q_seed):
    g = torch.Generator(device=dev)
    g.manual_seed(1_000_003 + q_seed)
    return torch.randn(batch, 1, hq, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)


def decode_bytes(lens, hq, hkv, d, page):
    """K and V rows of every cached token, q and o rows, block-table entries, the length."""
    lens = np.asarray(lens, dtype=np.int64)
    return int((2 * lens * hkv * d * 2).sum() + len(lens) * (2 * hq * d * 2) + (4 * ((lens + page - 1) // page)).sum() + 4 * len(lens))


def time_steps(torch, fn, steps, warmup, barrier=None):
    """W untimed + K timed calls; CUDA events on the current stream around the K calls."""
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / 1e3  # seconds for K steps


def _max_over_ranks(torch, dist, dev, sec):
    if dist is None:
        return sec
    t = torch.tensor([sec], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def tensor_roofline(tf, peaks, traffic=None):
    return {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
            "traffic": traffic, "peak_source": peaks["source"], "frac_nominal": tf / NOMINAL_TFLOPS}


def hbm_roofline(gbs, peaks, traffic=None):
    return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "traffic": traffic, "peak_source": peaks["source"], "frac_nominal": gbs / NOMINAL_HBM_GBS}


# ------------------------------------------------------------------------------------------
# single-GPU workloads
# ------------------------------------------------------------------------------------------
def run_prefill(torch, low, ffi, dev, name, steps, warmup, peaks):
    b, hq, hkv, s, d, seed, scale_in, want_lse = PREFILL[name]
    q, k, v = make_prefill(torch, dev, b, hq, hkv, s, d, seed, scale_in)
    o = torch.empty_like(q)
    lse = torch.empty(b, hq, s, device=dev, dtype=torch.float32) if want_lse else None
    scale = 1.0 / math.sqrt(d)

    def step():
        low.flash_attn(q, k, v, o, b, s, s, hq, hkv, d, 0, scale, None, None, lse)

    step()
    path, launches = ffi.last_path(), ffi.last_launches()
    sec = time_steps(torch, step, steps, warmup)
    flops = causal_flops(b, hq, s, s, d)
    tf = flops * steps / sec / 1e12
    res = {"metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
           "kernel_path": path, "launches_per_step": launches, "config": prefill_config(name),
           "roofline": tensor_roofline(tf, peaks, NCU_TRAFFIC_BYTES.get(name))}
    return res, (q, k, v, o, lse), step


def prefill_parity_single(torch, low, ffi, q, k, v, o):
    """One GPU: the timed kernel's output for one KV-head group of the last batch element, rows
    [0, 1024), against the library's SIMT tile kernel (f32 scalar arithmetic, no tensor cores, no TMA)
    on the same inputs. Untimed."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    group = hq // hkv
    rows = min(s, 1024)
    kvh = hkv - 1
    qs = q[b - 1:b, :rows, kvh * group:(kvh + 1) * group].contiguous()
    ks = k[b - 1:b, :rows, kvh:kvh + 1].contiguous()
    vs = v[b - 1:b, :rows, kvh:kvh + 1].contiguous()
    ref = torch.empty_like(qs)
    ffi.set_option("force_generic", 1)
    try:
        low.flash_attn(qs, ks, vs, ref, 1, rows, rows, group, 1, d, 0, 1.0 / math.sqrt(d))
        path = ffi.last_path()
    finally:
        ffi.set_option("force_generic", 0)
    torch.cuda.synchronize()
    got = o[b - 1:b, :rows, kvh * group:(kvh + 1) * group].float()
    err = (got - ref.float()).abs()
    ok = bool(torch.isfinite(got).all()) and float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3 and path == "tile_simt"
    return {"checked_ranks": 1, "ok": ok, "against": "tile_simt kernel, one KV-head group, 1024 rows",
            "max_abs_err": float(err.max())}


def run_decode(torch, low, ffi, dev, name, steps, warmup, peaks):
    batch, hq, hkv, d, page, lo, hi, pool, seed = DECODE[name]
    q, kc, vc, lens_d, table_d, lens = make_decode(torch, dev, batch, hq, hkv, d, page, lo, hi, pool, seed)
    o = torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    max_blocks = table_d.shape[1]

    def step():
        low.flash_attn_with_kvcache(q, kc, vc, o, table_d, lens_d, batch, 1, hq, hkv, d, page, max_blocks, scale)

    step()
    path, launches = ffi.last_path(), ffi.last_launches()
    sec = time_steps(torch, step, steps, warmup)
    nbytes = decode_bytes(lens, hq, hkv, d, page)
    gbs = nbytes * steps / sec / 1e9
    res = {"metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": sec / steps * 1e3,
           "kernel_path": path, "launches_per_step": launches,
           "config": {"workload": name, "batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "page_size": page,
                      "context": [int(lo), int(hi)], "tokens": int(lens.sum()), "pool_pages": int(kc.shape[0]),
                      "bytes_per_step": nbytes, "l2": "K/V touched per step larger than L2"},
           "roofline": hbm_roofline(gbs, peaks, int(nbytes * NCU_DECODE_TRAFFIC_RATIO))}
    return res


def run_paged_prefill(torch, low, ffi, dev, name, batch, sq, hq, hkv, d, page, lo, hi, steps, warmup, peaks, seed):
    """Chunked prefill: `sq` new tokens per sequence attend to a paged cache holding lo..hi tokens
    (the new ones included), bottom-right causal; K/V pages are gathered by TMA through the block table."""
    q1, kc, vc, lens_d, table_d, lens = make_decode(torch, dev, batch, hq, hkv, d, page, lo, hi, None, seed)
    g = torch.Generator(device=dev)
    g.manual_seed(seed + 1)
    q = torch.randn(batch, sq, hq, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    o = torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    max_blocks = table_d.shape[1]

    def step():
        low.flash_attn_with_kvcache(q, kc, vc, o, table_d, lens_d, batch, sq, hq, hkv, d, page, max_blocks, scale)

    step()
    path, launches = ffi.last_path(), ffi.last_launches()
    sec = time_steps(torch, step, steps, warmup)
    flops = sum(causal_flops(1, hq, sq, int(L), d, int(L) - sq) for L in lens)
    tf = flops * steps / sec / 1e12
    return {"metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
            "kernel_path": path, "launches_per_step": launches,
            "config": {"workload": name, "batch": batch, "chunk": sq, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                       "page_size": page, "context": [int(lo), int(hi)], "flops_per_step": flops},
            "roofline": tensor_roofline(tf, peaks)}


def run_varlen_prefill(torch, low, ffi, dev, name, num_seqs, lo, hi, hq, hkv, d, steps, warmup, peaks, seed):
    """Packed variable-length prefill (the serving shape of the batched config): `num_seqs` prompts of
    lo..hi tokens packed back to back, square causal per prompt, through the reference's flash_attn_varlen_bf16 symbol."""
    rng = np.random.Generator(np.random.Philox(seed))
    lens = rng.integers(lo, hi + 1, size=num_seqs).astype(np.int64)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    g = torch.Generator(device=dev)
    g.manual_seed(seed + 1)
    q = torch.randn(total, hq, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(total, hkv, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(total, hkv, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    o = torch.empty_like(q)
    cu_d = torch.from_numpy(cu).to(dev)
    scale = 1.0 / math.sqrt(d)
    max_len = int(lens.max())

    def step():
        low.flash_attn_varlen(q, k, v, o, cu_d, cu_d, num_seqs, max_len, max_len, hq, hkv, d, scale)

    step()
    path, launches = ffi.last_path(), ffi.last_launches()
    sec = time_steps(torch, step, steps, warmup)
    flops = sum(causal_flops(1, hq, int(L), int(L), d) for L in lens)
    tf = flops * steps / sec / 1e12
    return {"metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
            "kernel_path": path, "launches_per_step": launches,
            "config": {"workload": name, "num_seqs": num_seqs, "prompt_tokens": [int(lo), int(hi)], "total_tokens": total,
                       "q_heads": hq, "kv_heads": hkv, "head_dim": d, "flops_per_step": flops},
            "roofline": tensor_roofline(tf, peaks)}


def run_softmax(torch, low, ffi, dev, name, rows, n, dtype_name, steps, warmup, peaks, seed):
    """Row softmax of the math path on a (rows, n) score matrix: HBM-bound, one read and one write."""
    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype_name]
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = (torch.randn(rows, n, generator=g, device=dev, dtype=torch.float32) * 2.0).to(dt)
    y = torch.empty_like(x)

    def step():
        low.softmax_last_dim(x, out=y)

    step()
    path, launches = ffi.last_path(), ffi.last_launches()
    sec = time_steps(torch, step, steps, warmup)
    nbytes = 2 * rows * n * x.element_size()
    gbs = nbytes * steps / sec / 1e9
    return {"metric": "row-softmax HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": sec / steps * 1e3,
            "kernel_path": path, "launches_per_step": launches,
            "config": {"workload": name, "rows": rows, "row_size": n, "dtype": dtype_name, "bytes_per_step": nbytes},
            "roofline": hbm_roofline(gbs, peaks)}


# ------------------------------------------------------------------------------------------
# head-sharded workloads (strong scaling over the ranks; run at every N, N = 1 included)
# ------------------------------------------------------------------------------------------
def measure_peer_copy_gbs(torch, ffi, dist, dev, peer, rank, world, nbytes):
    """Peer bandwidth of this very run: every rank copies `nbytes` from its own memory into the
    next rank's shared output buffer (one cudaMemcpyAsync, all ranks at once, CUDA events, best of
    three); the slowest rank's figure is returned."""
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    src.zero_()
    dst = peer.ptrs[(rank + 1) % world]
    st = torch.cuda.current_stream(dev).cuda_stream
    best = float("inf")
    for it in range(4):
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if ffi.lib.luma_peer_copy(dst, src.data_ptr(), nbytes, st) != 0:
            raise RuntimeError(ffi.lib.luma_comm_last_error().decode())
        e1.record()
        torch.cuda.synchronize()
        if it > 0:
            best = min(best, e0.elapsed_time(e1) / 1e3)
    t = torch.tensor([best], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    return nbytes / float(t.item()) / 1e9


def args_no_multicast():
    """The fused all-gather stores to every peer with plain stores unless LUMA_B200_MULTICAST=1 asks for
    the NVSwitch multicast form (one multimem.st per 16 bytes). An all-gather is bound by what must ENTER
    each GPU, which multicast does not reduce (it adds the GPU's own shard to it): measured on 2 GPUs the
    NVLink-bound weak-scaled workload ran at 1083 TFLOP/s with multicast against 1283 with plain stores,
    the compute-bound strong-scaled one the same either way."""
    return os.environ.get("LUMA_B200_MULTICAST", "") in ("", "0")


def fused_roofline(flops_per_gpu, nvlink_out_bytes_per_gpu, sec_per_step, peaks, peer_gbs):
    """Roofline of the fused attention + all-gather kernel, per GPU: the target time is the slower of
    FLOPs / measured GEMM peak and bytes stored to peers over NVLink / the peer bandwidth measured in
    this run."""
    t_math = flops_per_gpu / (peaks["bf16_tflops"] * 1e12)
    t_link = nvlink_out_bytes_per_gpu / (peer_gbs * 1e9) if peer_gbs else 0.0
    if t_link > t_math:
        gbs = nvlink_out_bytes_per_gpu / sec_per_step / 1e9
        return {"bound": "nvlink", "achieved": gbs, "peak": peer_gbs, "unit": "GB/s", "frac": gbs / peer_gbs, "traffic": None,
                "peak_source": "peer copy measured in this run", "frac_nominal": gbs / NOMINAL_NVLINK_GBS,
                "target_ms": t_link * 1e3}
    tf = flops_per_gpu / sec_per_step / 1e12
    r = tensor_roofline(tf, peaks)
    r["target_ms"] = t_math * 1e3
    return r


def run_sharded_prefill(torch, low, ffi, dev, dist, world, rank, name, steps, warmup, peaks, sampler=None):
    """Strong scaling: the (b, s, hq, d) problem is split by KV-head groups over `world` ranks; every
    rank ends with the full O (the kernel stores its heads into every rank's output buffer). Rank r's
    inputs come from seed + r, so any rank can regenerate any other rank's shard for the parity check."""
    from luma_b200 import dist as fdist
    b, hq, hkv, s, d, seed, scale_in, _lse = PREFILL[name]
    qs, kvs = fdist.shard_heads(hq, hkv, world, rank)
    hq_l, hkv_l = qs.stop - qs.start, kvs.stop - kvs.start
    q, k, v = make_prefill(torch, dev, b, hq_l, hkv_l, s, d, seed + rank, scale_in)
    scale = 1.0 / math.sqrt(d)
    launches = [0]
    peer_gbs = None
    if world > 1:
        # plain peer stores by default; LUMA_B200_MULTICAST=1: symmetric allocation and, where the box offers
        # an NVSwitch multicast address, stores through it
        peer = fdist.PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev, multicast=not args_no_multicast())
        gather = "multimem.st through an NVSwitch multicast address" if peer.mc_ptr else "plain stores to every peer"
        peer_gbs = measure_peer_copy_gbs(torch, ffi, dist, dev, peer, rank, world, min(256 << 20, peer.out.numel() * 2))
        out = peer.out

        def step():
            peer.fused_attention(q, k, v, hq, qs.start, scale=scale)
            peer.sync()
            launches[0] = 2
    else:
        out = torch.empty_like(q)

        def step():
            low.flash_attn(q, k, v, out, b, s, s, hq_l, hkv_l, d, 0, scale)
            launches[0] = ffi.last_launches()

    step()
    path = ffi.last_path()
    barrier = (lambda: dist.barrier()) if dist is not None else None
    if sampler is not None:
        sampler.start()
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, step, steps, warmup, barrier))
    clocks = sampler.stop(torch, step, barrier, repeats=(0.35 / max(sec / steps, 1e-6)) if world > 1 else None) if sampler is not None else None

    # ---- parity, untimed: what is in `out` after the timed steps -------------------------------
    if world > 1:
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        step()
        torch.cuda.synchronize()
        dist.barrier()
        other = (rank + 1) % world
        oq, okv = fdist.shard_heads(hq, hkv, world, other)
        q2, k2, v2 = make_prefill(torch, dev, b, hq_l, hkv_l, s, d, seed + other, scale_in)
        ref = torch.empty_like(q2)
        low.flash_attn(q2, k2, v2, ref, b, s, s, hq_l, hkv_l, d, 0, scale)
        torch.cuda.synchronize()
        ok = bool(torch.equal(out[:, :, oq], ref)) and bool(torch.isfinite(out.float()).all())
        mine = torch.empty_like(q)
        low.flash_attn(q, k, v, mine, b, s, s, hq_l, hkv_l, d, 0, scale)
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(out[:, :, qs], mine))
        t = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        parity = {"checked_ranks": world, "ok": bool(t.item() == 1.0),
                  "against": "every rank recomputes the next rank's heads and its own alone; bit-exact with the gathered output"}
        del q2, k2, v2, ref, mine
        peer.close()
    else:
        parity = prefill_parity_single(torch, low, ffi, q, k, v, out)
    flops = causal_flops(b, hq, s, s, d)
    tf = flops * steps / sec / 1e12
    res = {"metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "per_gpu": tf / world,
           "ms_per_step": sec / steps * 1e3, "scaling": "strong", "n_gpus": world, "kernel_path": path,
           "launches_per_step": launches[0], "config": prefill_config(name, world), "parity": parity,
           "roofline": fused_roofline(flops / world, q.numel() * 2 * (world - 1), sec / steps, peaks, peer_gbs) if world > 1   # bytes that must enter every GPU
           else tensor_roofline(tf, peaks, NCU_TRAFFIC_BYTES.get(name))}
    if world > 1 and NCU_TRAFFIC_BYTES.get(name):
        res["roofline"]["traffic"] = NCU_TRAFFIC_BYTES[name] // world   # this GPU's share of the one-GPU capture
    if peer_gbs is not None:
        res["peer_copy_gbs"] = peer_gbs
        res["gather"] = gather
    return res, clocks, (q, k, v)


def run_sharded_decode(torch, low, ffi, dev, dist, world, rank, name, steps, warmup, peaks):
    """Strong scaling of paged decode: every rank holds the cache slice of its KV heads
    (num_blocks, page, hkv/world, d); block tables and lengths are replicated; the merge kernel stores
    its heads into every rank's (batch, 1, hq, d) output. All ranks build their cache slice from the
    same seed and differ in their query rows, so a rank can recompute another rank's heads alone."""
    from luma_b200 import dist as fdist
    batch, hq, hkv, d, page, lo, hi, pool, seed = DECODE[name]
    qs, kvs = fdist.shard_heads(hq, hkv, world, rank)
    hq_l, hkv_l = qs.stop - qs.start, kvs.stop - kvs.start
    q, kc, vc, lens_d, table_d, lens = make_decode(torch, dev, batch, hq_l, hkv_l, d, page, lo, hi, pool, seed, q_seed=seed + rank)
    scale = 1.0 / math.sqrt(d)
    max_blocks = table_d.shape[1]
    if world > 1:
        peer = fdist.PeerOutput(dist.group.WORLD, (batch, 1, hq, d), torch.bfloat16, dev)
        out = peer.out

        def step():
            peer.fused_decode(q, kc, vc, table_d, lens_d, hq, qs.start, scale)
            peer.sync()
    else:
        out = torch.empty_like(q)

        def step():
            low.flash_attn_with_kvcache(q, kc, vc, out, table_d, lens_d, batch, 1, hq_l, hkv_l, d, page, max_blocks, scale)

    step()
    path, launches = ffi.last_path(), ffi.last_launches() + (1 if world > 1 else 0)
    barrier = (lambda: dist.barrier()) if dist is not None else None
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, step, steps, warmup, barrier))
    parity = None
    if world > 1:
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        step()
        torch.cuda.synchronize()
        dist.barrier()
        other = (rank + 1) % world
        oq, _ = fdist.shard_heads(hq, hkv, world, other)
        q2 = make_decode_q(torch, dev, batch, hq_l, d, seed + other)
        ref = torch.empty_like(q2)
        low.flash_attn_with_kvcache(q2, kc, vc, ref, table_d, lens_d, batch, 1, hq_l, hkv_l, d, page, max_blocks, scale)
        torch.cuda.synchronize()
        ok = bool(torch.equal(out[:, :, oq], ref)) and bool(torch.isfinite(out.float()).all())
        t = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        parity = {"checked_ranks": world, "ok": bool(t.item() == 1.0)}
        peer.close()
    nbytes = decode_bytes(lens, hq, hkv, d, page)   # whole job: all KV heads
    gbs = nbytes * steps / sec / 1e9
    r = hbm_roofline(gbs / world, peaks)
    return {"metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "per_gpu": gbs / world,
            "ms_per_step": sec / steps * 1e3, "scaling": "strong", "n_gpus": world, "kernel_path": path,
            "launches_per_step": launches, "parity": parity,
            "config": {"workload": name, "batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                       "page_size": page, "context": [int(lo), int(hi)], "tokens": int(lens.sum()),
                       "pool_pages": int(kc.shape[0]), "bytes_per_step": nbytes},
            "roofline": r}


def run_weak_prefill(torch, low, ffi, dev, dist, world, rank, name, steps, warmup, peaks):
    """Weak scaling: every rank owns the heads of one whole `name` problem of a world-times-wider layer
    and stores them into every rank's output (NVLink-bound by construction at larger N)."""
    from luma_b200 import dist as fdist
    b, hq, hkv, s, d, seed, scale_in, _lse = PREFILL[name]
    q, k, v = make_prefill(torch, dev, b, hq, hkv, s, d, seed + rank, scale_in)
    peer = fdist.PeerOutput(dist.group.WORLD, (b, s, hq * world, d), torch.bfloat16, dev, multicast=not args_no_multicast())

    def step():
        peer.fused_attention(q, k, v, hq * world, hq * rank)
        peer.sync()

    step()
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, step, steps, warmup, lambda: dist.barrier()))
    peer.close()
    flops = causal_flops(b, hq, s, s, d) * world
    tf = flops * steps / sec / 1e12
    return {"metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "per_gpu": tf / world, "ms_per_step": sec / steps * 1e3,
            "scaling": "weak", "n_gpus": world, "config": {"workload": name + "_weak", "q_heads": hq * world},
            "roofline": {"bound": "nvlink", "achieved": q.numel() * 2 * (world - 1) / (sec / steps) / 1e9, "unit": "GB/s"}}


# ------------------------------------------------------------------------------------------
# end to end through the host-tensor API
# ------------------------------------------------------------------------------------------
def run_e2e(torch, dev, dist, q, k, v, flops_total, steps):
    """Same metric through luma_b200.high.flash_attn_func_host: this rank's q/k/v in pinned HOST
    memory -> device, kernel, output -> pinned host, every step. Max over ranks."""
    from luma_b200 import high
    hq_h, hk_h, hv_h = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        high.flash_attn_func_host(hq_h, hk_h, hv_h, ho, None, True, 0, dev)

    barrier = (lambda: dist.barrier()) if dist is not None else None
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, e2e_step, steps, 2, barrier))
    ok = bool(torch.isfinite(ho.float()).all())
    h2d_bytes, d2h_bytes = int((q.numel() + k.numel() + v.numel()) * 2), int(q.numel() * 2)

    # What the host link gives while every rank uses it at once, both directions together: the same
    # bytes as plain copies on two streams, no kernel. The e2e step cannot be shorter than this.
    dq, dk, dv = (torch.empty_like(t) for t in (q, k, v))
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def link_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            dq.copy_(hq_h, non_blocking=True)
            dk.copy_(hk_h, non_blocking=True)
            dv.copy_(hv_h, non_blocking=True)
        with torch.cuda.stream(s_out):
            ho.copy_(q, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    link_sec = _max_over_ranks(torch, dist, dev, time_steps(torch, link_step, 3, 1, barrier)) / 3
    del dq, dk, dv
    return {"value": flops_total * steps / sec / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
            "steps": steps, "ms_per_step": sec / steps * 1e3, "finite": ok,
            "host_link": {"copies_only_ms": link_sec * 1e3, "gbs_per_gpu": (h2d_bytes + d2h_bytes) / link_sec / 1e9,
                          "frac": link_sec / (sec / steps)},
            "api": "high.flash_attn_func_host -> flash_attn_host_bf16 (pinned host buffers, row chunks pipelined); bytes per GPU"}


# ------------------------------------------------------------------------------------------
# CPU baseline (oracle port of luma-cpu's math path) — bounded sample of the headline workload
# ------------------------------------------------------------------------------------------
def cpu_sample_inputs(name, n_heads, seed=0):
    """One batch element, one KV head and `n_heads` of its query heads, full sequence length."""
    _b, _hq, _hkv, s, d, _seed, scale_in, _lse = PREFILL[name]
    rng = np.random.Generator(np.random.Philox(seed))
    q = rng.standard_normal((1, s, n_heads, d), dtype=np.float32) * np.float32(scale_in)
    k = rng.standard_normal((1, s, 1, d), dtype=np.float32) * np.float32(scale_in)
    v = rng.standard_normal((1, s, 1, d), dtype=np.float32) * np.float32(scale_in)
    return q, k, v


def cpu_sample_text(name, n_heads):
    b, hq, hkv, s, _d, _seed, _sc, _lse = PREFILL[name]
    return (f"1 of {b} batch elements x 1 of {hkv} KV heads x {n_heads} of its {hq // hkv} query heads, full S={s}; "
            "f32 math path (oracle port of luma-cpu), causal FLOPs counted")


def cpu_baseline_prefill(name, budget_s=12.0):
    from oracle import binding as ob
    cores = ob.hardware_threads()
    _b, hq, hkv, s, d, _seed, _sc, _lse = PREFILL[name]
    group = hq // hkv
    q, k, v = cpu_sample_inputs(name, 1)
    t0 = time.perf_counter()
    ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    probe = time.perf_counter() - t0
    nh = int(max(1, min(group, budget_s / max(probe, 1e-3))))
    if nh > 1:
        q, k, v = cpu_sample_inputs(name, nh)
        t0 = time.perf_counter()
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
        sec = time.perf_counter() - t0
    else:
        sec = probe
    flops = causal_flops(1, nh, s, s, d)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": cpu_sample_text(name, nh) + f"; {sec:.2f} s"}


def reference_cuda_baseline(torch, low, ffi, dev):
    """The reference's own CUDA kernels (luma-flash-attn/kernels/*.cu, compiled unmodified for sm_100a
    into oracle/_ref by oracle/Makefile's `ref` target) on the S=8192 GQA prefill and the batch-64 paged
    decode, device-timed, with their outputs compared with this library's. Part of the baseline leg: a
    second stated baseline beside the CPU one, not a measured product path. None where the file was not
    built (the reference tree is not mounted everywhere)."""
    import ctypes
    path = ROOT / "oracle" / "_ref" / "libflash_attn_ref.so"
    if not path.exists():
        return None
    ref = ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)
    ref.flash_attn_bf16.argtypes = ffi._BATCH_ARGS
    ref.flash_attn_with_kvcache_bf16.argtypes = ffi._KVCACHE_ARGS
    st = torch.cuda.current_stream().cuda_stream

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3 / reps

    out = {"kind": "reference CUDA kernels compiled for sm_100a"}
    b, hq, hkv, s, d, seed, scale_in, _lse = PREFILL["prefill_c3"]
    q, k, v = make_prefill(torch, dev, b, hq, hkv, s, d, seed, scale_in)
    theirs, mine = torch.empty_like(q), torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)

    def ref_prefill():
        rc = ref.flash_attn_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), theirs.data_ptr(), b, s, s, hq, hkv, d, 0, scale, None, st)
        if rc != 0:
            raise RuntimeError(f"reference flash_attn_bf16 returned {rc}")
    sec = timed(ref_prefill, 2)
    low.flash_attn(q, k, v, mine, b, s, s, hq, hkv, d, 0, scale)
    torch.cuda.synchronize()
    diff = float((mine.float() - theirs.float()).abs().max())
    out["prefill_c3"] = {"value": causal_flops(b, hq, s, s, d) / sec / 1e12, "unit": "TFLOP/s", "ms": sec * 1e3, "max_abs_diff_vs_ours": diff}
    del q, k, v, theirs, mine
    torch.cuda.empty_cache()

    batch, hq, hkv, d, page, lo, hi, pool, seed = DECODE["decode_c4"]
    q, kc, vc, lens_d, table_d, lens = make_decode(torch, dev, batch, hq, hkv, d, page, lo, hi, pool, seed)
    theirs, mine = torch.empty_like(q), torch.empty_like(q)

    def ref_decode():
        rc = ref.flash_attn_with_kvcache_bf16(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), theirs.data_ptr(), table_d.data_ptr(),
                                              lens_d.data_ptr(), batch, 1, hq, hkv, d, page, table_d.shape[1], scale, st)
        if rc != 0:
            raise RuntimeError(f"reference flash_attn_with_kvcache_bf16 returned {rc}")
    sec = timed(ref_decode, 3)
    low.flash_attn_with_kvcache(q, kc, vc, mine, table_d, lens_d, batch, 1, hq, hkv, d, page, table_d.shape[1], scale)
    torch.cuda.synchronize()
    diff = float((mine.float() - theirs.float()).abs().max())
    out["decode_c4"] = {"value": decode_bytes(lens, hq, hkv, d, page) / sec / 1e9, "unit": "GB/s", "ms": sec * 1e3, "max_abs_diff_vs_ours": diff}
    del q, kc, vc, theirs, mine
    torch.cuda.empty_cache()
    return out


def reference_arm(args):
    """`--impl reference`: the CPU path on the host cores, K timed steps after W warm-up steps as
    given, each step a bounded sample of the same headline workload as the GPU arm at this N."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, int(os.environ.get("WORLD_SIZE", str(args.gpus))))
    name = "prefill_c3" if world == 1 else "prefill_c5"
    from oracle import binding as ob
    cores = ob.hardware_threads()
    _b, hq, hkv, s, d, _seed, _sc, _lse = PREFILL[name]
    group = hq // hkv
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # size the sample so that the whole run stays within about two and a half minutes
    q, k, v = cpu_sample_inputs(name, 1)
    t0 = time.perf_counter()
    ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    probe = time.perf_counter() - t0
    nh = int(max(1, min(group, 150.0 / max(probe * (steps + warmup), 1e-3))))
    if nh > 1:
        q, k, v = cpu_sample_inputs(name, nh)
    for _ in range(warmup):
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    sec = time.perf_counter() - t0
    flops = causal_flops(1, nh, s, s, d)
    tf = flops * steps / sec / 1e12
    print(json.dumps({
        "impl": "reference", "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": sec / steps * 1e3,
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": prefill_config(name, world),
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": cpu_sample_text(name, nh)},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def _short_floats(x):
    """Six significant digits for every float of the printed line (it has to survive in a log tail)."""
    if isinstance(x, float):
        return float(f"{x:.6g}")
    if isinstance(x, dict):
        return {k: _short_floats(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_short_floats(v) for v in x]
    return x


def compact(res):
    """A workload's entry under "workloads": the figures, not the prose."""
    out = {"value": round(res["value"], 1), "unit": res["unit"], "ms": round(res["ms_per_step"], 4),
           "frac": round(res["roofline"].get("frac", 0.0), 4) if res["roofline"].get("frac") is not None else None,
           "frac_nominal": round(res["roofline"]["frac_nominal"], 4) if res["roofline"].get("frac_nominal") is not None else None,
           "bound": res["roofline"]["bound"]}
    for key in ("per_gpu", "scaling", "peer_copy_gbs"):
        if key in res:
            out[key] = round(res[key], 1) if isinstance(res[key], float) else res[key]
    if res.get("parity") is not None:
        out["parity_ok"] = res["parity"]["ok"]
    return out


# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, help="headline plus just one other workload: prefill_c2, decode_c4, paged_prefill, "
                                                  "varlen_prefill, softmax_scores, prefill_c5, decode_c5, none")
    ap.add_argument("--profile", default=None,
                    help="run ONE workload and nothing else (for ncu): prefill_c2, prefill_c3, prefill_c3_small, prefill_c5, "
                         "decode_c4, decode_c4_small, decode_c5, varlen_prefill, softmax_<dtype>_<rows>x<row_size>")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return
    args.warmup = max(args.warmup, 3) if not args.profile else args.warmup

    import torch
    from luma_b200 import ffi, low
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the measured path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(torch, local_rank)
    peaks = load_peaks()
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    if args.profile:
        # one workload, nothing else: the command line the ncu summaries under profiles/ were made with
        name = args.profile
        if name in PREFILL:
            res, _bufs, _step = run_prefill(torch, low, ffi, dev, name, args.steps, args.warmup, peaks)
        elif name in DECODE:
            res = run_decode(torch, low, ffi, dev, name, args.steps, args.warmup, peaks)
        elif name == "varlen_prefill":
            res = run_varlen_prefill(torch, low, ffi, dev, name, 32, 1024, 8192, 32, 8, 128, args.steps, args.warmup, peaks, seed=7)
        elif name.startswith("softmax_"):   # softmax_<dtype>_<rows>x<row_size>, e.g. softmax_bf16_131072x4096
            _, dtn, shp = name.split("_")
            r_, n_ = (int(t) for t in shp.split("x"))
            res = run_softmax(torch, low, ffi, dev, name, r_, n_, dtn, args.steps, args.warmup, peaks, seed=8)
        else:
            raise SystemExit(f"unknown --profile {name}")
        print(json.dumps(res))
        return

    sampler = ClockSampler(local_rank)
    workloads = {}
    only = args.only
    K, W = args.steps, args.warmup
    extra_steps = max(3, min(K, 10))

    # ---- headline ---------------------------------------------------------------------------
    if world == 1:
        sampler.start()
        primary, bufs, step = run_prefill(torch, low, ffi, dev, "prefill_c3", K, W, peaks)
        clocks = sampler.stop(torch, step)
        q, k, v, o, _lse = bufs
        primary["parity"] = prefill_parity_single(torch, low, ffi, q, k, v, o)
        primary["scaling"] = "weak"
        del o, bufs, step
    else:
        primary, clocks, (q, k, v) = run_sharded_prefill(torch, low, ffi, dev, dist, world, rank, "prefill_c5", K, W, peaks, sampler)

    # ---- end to end through the host API with HOST buffers ------------------------------------
    e2e = run_e2e(torch, dev, dist, q, k, v, primary["config"]["flops_per_step"], max(3, min(K, 10)))
    del q, k, v
    torch.cuda.empty_cache()

    # ---- the other configurations -----------------------------------------------------------
    if world == 1:
        if only in (None, "prefill_c2"):
            res, _b, _s = run_prefill(torch, low, ffi, dev, "prefill_c2", K, W, peaks)
            workloads["prefill_c2"] = compact(res)
            del _b, _s
            torch.cuda.empty_cache()
        if only in (None, "decode_c4"):
            workloads["decode_c4"] = compact(run_decode(torch, low, ffi, dev, "decode_c4", max(K, 20), 5, peaks))
            torch.cuda.empty_cache()
        if only in (None, "paged_prefill"):
            # the step before decode: 1024-token chunks over paged contexts of 1024..8192 tokens, page 16
            workloads["paged_prefill"] = compact(run_paged_prefill(torch, low, ffi, dev, "paged_prefill", 16, 1024, 32, 8, 128, 16,
                                                                   1024, 8192, extra_steps, 3, peaks, seed=6))
            torch.cuda.empty_cache()
        if only in (None, "varlen_prefill"):
            # 32 prompts of 1024..8192 tokens packed, GQA 32/8
            workloads["varlen_prefill"] = compact(run_varlen_prefill(torch, low, ffi, dev, "varlen_prefill", 32, 1024, 8192, 32, 8, 128,
                                                                     extra_steps, 3, peaks, seed=7))
            torch.cuda.empty_cache()
        if only in (None, "softmax_scores"):
            # the scores of one head group of the GQA prefill on the math path, bf16
            workloads["softmax_scores"] = compact(run_softmax(torch, low, ffi, dev, "softmax_scores", 131072, 4096, "bf16",
                                                              extra_steps, 3, peaks, seed=8))
            torch.cuda.empty_cache()
        if only in (None, "prefill_c5"):
            res, _c, _bufs = run_sharded_prefill(torch, low, ffi, dev, None, 1, 0, "prefill_c5", extra_steps, 3, peaks)
            workloads["prefill_c5"] = compact(res)
            del _bufs
            torch.cuda.empty_cache()
    else:
        if only in (None, "prefill_c2"):
            workloads["prefill_c2_weak"] = compact_weak(run_weak_prefill(torch, low, ffi, dev, dist, world, rank, "prefill_c2",
                                                                          extra_steps, 3, peaks))
            torch.cuda.empty_cache()
    if only in (None, "decode_c5"):
        workloads["decode_c5"] = compact(run_sharded_decode(torch, low, ffi, dev, dist, world, rank, "decode_c5",
                                                            max(extra_steps, 10), 3, peaks))
        torch.cuda.empty_cache()

    # ---- CPU baseline, rank 0, N == 1 only -----------------------------------------------------
    cpu = None
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline_prefill("prefill_c3")
        ref_cuda = reference_cuda_baseline(torch, low, ffi, dev)

    if rank == 0:
        line = {
            "metric": primary["metric"], "value": primary["value"], "unit": primary["unit"],
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": primary["ms_per_step"],
            "higher_is_better": True, "scaling": primary["scaling"], "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": primary["config"], "roofline": primary["roofline"],
            "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "parity": primary["parity"],
            "gpu_launches": int(primary["launches_per_step"]) * K, "kernel_path": primary["kernel_path"],
            "workloads": workloads,
        }
        if "peer_copy_gbs" in primary:
            line["peer_copy_gbs"] = primary["peer_copy_gbs"]
            line["gather"] = primary["gather"]
        if "per_gpu" in primary:
            line["per_gpu"] = primary["per_gpu"]
        if ref_cuda is not None:
            line["reference_cuda"] = ref_cuda
        if numa:
            line["host_cpus"] = numa
        print(json.dumps(_short_floats(line)))
    ok = primary["parity"]["ok"] and all(w.get("parity_ok", True) for w in workloads.values())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed: the gathered output differs from a local recomputation")


def compact_weak(res):
    return {"value": round(res["value"], 1), "unit": res["unit"], "per_gpu": round(res["per_gpu"], 1), "ms": round(res["ms_per_step"], 4),
            "scaling": "weak", "bound": "nvlink", "nvlink_out_gbs_per_gpu": round(res["roofline"]["achieved"], 1)}


if __name__ == "__main__":
    main()
