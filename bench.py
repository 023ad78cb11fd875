#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--only NAME]

Prints ONE JSON line. A "step" is one pass of the primary workload (BASELINE.json configs[1]:
causal bf16 prefill B=4, Hq=Hkv=32, S=2048, d=128 with fp32 LSE). With N > 1 (torchrun, one rank
per GPU) every rank owns 32 query/KV heads of a 32*N-head layer (weak scaling), runs the same
kernel on its shard and the outputs are joined by one all-gather along the head axis, inside the
timed region. The other BASELINE.json configs are measured as well and reported under
"workloads" (each with its own roofline object); "--only NAME" restricts the run to one of them.

`--impl reference` times the CPU restatement of luma-cpu's math-path attention (oracle/) on the
host cores: the reference's own implementation of this path is Rust and cannot be built with
this image's toolchains.
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
# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from
# the ncu captures summarised under profiles/. prefill_c2 was captured at full size; the decode
# figure is the ratio measured on decode_c4_small (399.9 MB moved for 394.2 MB of algorithmic bytes,
# L2 hit rate 0.4 %: traffic grows in proportion to the cached tokens) applied to the run's own bytes.
NCU_TRAFFIC_BYTES = {"prefill_c2": 512_585_728 + 51_621_632}
NCU_DECODE_TRAFFIC_RATIO = (394_139_648 + 4_231_680) / 394_223_184
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


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
            if step is not None:
                out["note"] = "sampled from the start of the timed region through an untimed ~0.35 s repeat of the same step"
        return out


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------
def make_prefill(torch, dev, b, hq, hkv, s, d, seed, scale_in=1.0):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    q = (torch.randn(b, s, hq, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    k = (torch.randn(b, s, hkv, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    v = (torch.randn(b, s, hkv, d, generator=g, device=dev, dtype=torch.float32) * scale_in).to(torch.bfloat16)
    return q, k, v


def make_decode(torch, dev, batch, hq, hkv, d, page, lo, hi, pool_pages, seed):
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
    q = torch.randn(batch, 1, hq, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    return q, kc, vc, torch.from_numpy(lens).to(dev), torch.from_numpy(table).to(dev), lens


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


def run_prefill(torch, low, ffi, dev, name, b, hq, hkv, s, d, steps, warmup, peaks, seed, scale_in=1.0, want_lse=True):
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
    peak = peaks["bf16_tflops"]
    res = {
        "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
        "kernel_path": path, "launches_per_step": launches,
        "config": {"workload": name, "batch": b, "q_heads": hq, "kv_heads": hkv, "seq_len": s, "head_dim": d,
                   "causal": True, "lse": want_lse, "flops_per_step": flops,
                   "l2_policy": "inputs larger than L2 (q+k+v+o = %d MiB)" % ((q.numel() * 2 + k.numel() * 4) * 2 // 2 ** 20 // 1)},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)",
                     "frac_of_nominal_2250": tf / NOMINAL_TFLOPS},
    }
    return res, (q, k, v, o, lse)


def run_decode(torch, low, ffi, dev, name, batch, hq, hkv, d, page, lo, hi, pool, steps, warmup, peaks, seed):
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
    peak = peaks["hbm_gbs"]
    res = {
        "metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": sec / steps * 1e3,
        "kernel_path": path, "launches_per_step": launches,
        "config": {"workload": name, "batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d, "page_size": page,
                   "context": [int(lo), int(hi)], "tokens": int(lens.sum()), "pool_pages": int(kc.shape[0]),
                   "bytes_per_step": nbytes, "l2_policy": "K/V touched per step (%d MiB) larger than L2" % (nbytes // 2 ** 20)},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "traffic": int(nbytes * NCU_DECODE_TRAFFIC_RATIO),
                     "peak_source": f"of {peaks['source']} (copy bandwidth)",
                     "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS},
    }
    return res, (q, kc, vc, o, lens_d, table_d)


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
    peak = peaks["bf16_tflops"]
    return {
        "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
        "kernel_path": path, "launches_per_step": launches,
        "config": {"workload": name, "batch": batch, "chunk": sq, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "page_size": page, "context": [int(lo), int(hi)], "flops_per_step": flops},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                     "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)", "frac_of_nominal_2250": tf / NOMINAL_TFLOPS},
    }


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
    peak = peaks["bf16_tflops"]
    return {
        "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / steps * 1e3,
        "kernel_path": path, "launches_per_step": launches,
        "config": {"workload": name, "num_seqs": num_seqs, "prompt_tokens": [int(lo), int(hi)], "total_tokens": total,
                   "q_heads": hq, "kv_heads": hkv, "head_dim": d, "flops_per_step": flops,
                   "l2_policy": "inputs larger than L2"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                     "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)", "frac_of_nominal_2250": tf / NOMINAL_TFLOPS},
    }


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
    return {
        "metric": "row-softmax HBM GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": sec / steps * 1e3,
        "kernel_path": path, "launches_per_step": launches,
        "config": {"workload": name, "rows": rows, "row_size": n, "dtype": dtype_name, "bytes_per_step": nbytes,
                   "l2_policy": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "traffic": None, "peak_source": f"of {peaks['source']} (copy bandwidth)",
                     "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS},
    }


NVLINK_PEER_GBS = 770.0   # measured peer-copy bandwidth per direction on this pool (nominal 900)


def fused_roofline(flops_per_gpu, nvlink_out_bytes_per_gpu, sec_per_step, peaks):
    """Roofline of the fused attention + all-gather kernel, per GPU: the target time is the slower of
    FLOPs / measured GEMM peak and bytes stored to peers over NVLink / measured peer bandwidth."""
    t_math = flops_per_gpu / (peaks["bf16_tflops"] * 1e12)
    t_link = nvlink_out_bytes_per_gpu / (NVLINK_PEER_GBS * 1e9)
    if t_link > t_math:
        gbs = nvlink_out_bytes_per_gpu / sec_per_step / 1e9
        return {"bound": "nvlink", "achieved": gbs, "peak": NVLINK_PEER_GBS, "unit": "GB/s", "frac": gbs / NVLINK_PEER_GBS,
                "traffic": None, "peak_source": "measured peer copy, per direction per GPU; bytes = this GPU's O shard "
                                                "stored to every peer", "target_ms": t_link * 1e3}
    tf = flops_per_gpu / sec_per_step / 1e12
    return {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": tf / peaks["bf16_tflops"], "traffic": None,
            "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst); per GPU, all-gather included",
            "frac_of_nominal_2250": tf / NOMINAL_TFLOPS, "target_ms": t_math * 1e3}


def _max_over_ranks(torch, dist, dev, sec):
    if dist is None:
        return sec
    t = torch.tensor([sec], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_sharded_prefill(torch, low, ffi, dev, dist, world, rank, b, hq, hkv, s, d, steps, warmup, peaks, seed, chunks=4):
    """Strong scaling: the (b, s, hq, d) problem is split by KV-head groups over `world` ranks; every
    rank ends with the full O (the kernel stores its heads into every rank's output buffer)."""
    from luma_b200 import dist as fdist
    qs, kvs = fdist.shard_heads(hq, hkv, world, rank)
    hq_l, hkv_l = qs.stop - qs.start, kvs.stop - kvs.start
    q, k, v = make_prefill(torch, dev, b, hq_l, hkv_l, s, d, seed + rank)
    scale = 1.0 / math.sqrt(d)
    launches = [0]
    if world > 1:
        peer = fdist.PeerOutput(dist.group.WORLD, (b, s, hq, d), torch.bfloat16, dev)

        def step():
            peer.fused_attention(q, k, v, hq, qs.start, scale=scale)
            peer.sync()
            launches[0] = 2
    else:
        o_local = torch.empty_like(q)

        def step():
            low.flash_attn(q, k, v, o_local, b, s, s, hq_l, hkv_l, d, 0, scale)
            launches[0] = ffi.last_launches()

    step()
    path = ffi.last_path()
    barrier = (lambda: dist.barrier()) if dist is not None else None
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, step, steps, warmup, barrier))
    if world > 1:
        peer.close()
    flops = causal_flops(b, hq, s, s, d)
    tf = flops * steps / sec / 1e12
    peak = peaks["bf16_tflops"]
    return {
        "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "per_gpu": tf / world,
        "ms_per_step": sec / steps * 1e3, "scaling": "strong", "n_gpus": world, "kernel_path": path,
        "launches_per_step": launches[0],
        "config": {"workload": "prefill_c5", "batch": b, "q_heads": hq, "kv_heads": hkv, "seq_len": s, "head_dim": d,
                   "causal": True, "flops_per_step": flops,
                   "parallelism": f"KV-head groups over {world} GPU(s); all-gather of O fused into the kernel epilogue "
                                  "(peer stores over NVLink) + one 4-byte all-reduce"},
        "roofline": fused_roofline(flops / world, q.numel() * 2 * (world - 1), sec / steps, peaks),
    }


def run_sharded_decode(torch, low, ffi, dev, dist, world, rank, batch, hq, hkv, d, page, lo, hi, steps, warmup, peaks, seed):
    """Strong scaling of paged decode: every rank holds the cache slice of its KV heads
    (num_blocks, page, hkv/world, d); block tables and lengths are replicated; O is all-gathered."""
    from luma_b200 import dist as fdist
    qs, kvs = fdist.shard_heads(hq, hkv, world, rank)
    hq_l, hkv_l = qs.stop - qs.start, kvs.stop - kvs.start
    q, kc, vc, lens_d, table_d, lens = make_decode(torch, dev, batch, hq_l, hkv_l, d, page, lo, hi, None, seed)
    o_local = torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    max_blocks = table_d.shape[1]
    gather = fdist.HeadAllGather(dist.group.WORLD, (batch, 1, hq_l, d), torch.bfloat16, dev) if world > 1 else None

    def step():
        low.flash_attn_with_kvcache(q, kc, vc, o_local, table_d, lens_d, batch, 1, hq_l, hkv_l, d, page, max_blocks, scale)
        if gather is not None:
            gather(o_local)

    step()
    path, launches = ffi.last_path(), ffi.last_launches() + (2 if gather is not None else 0)
    barrier = (lambda: dist.barrier()) if dist is not None else None
    sec = _max_over_ranks(torch, dist, dev, time_steps(torch, step, steps, warmup, barrier))
    nbytes = decode_bytes(lens, hq, hkv, d, page)   # whole job: all KV heads
    gbs = nbytes * steps / sec / 1e9
    peak = peaks["hbm_gbs"]
    return {
        "metric": "paged-decode HBM GB/s", "value": gbs, "unit": "GB/s", "per_gpu": gbs / world,
        "ms_per_step": sec / steps * 1e3, "scaling": "strong", "n_gpus": world, "kernel_path": path,
        "launches_per_step": launches,
        "config": {"workload": "decode_c5", "batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "page_size": page, "context": [int(lo), int(hi)], "tokens": int(lens.sum()),
                   "pool_pages": int(kc.shape[0]), "bytes_per_step": nbytes,
                   "parallelism": f"KV heads over {world} GPU(s), all-gather of O"},
        "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                     "traffic": None, "peak_source": f"of {peaks['source']} (copy bandwidth); per GPU, all-gather included",
                     "frac_of_nominal_8000": gbs / world / NOMINAL_HBM_GBS},
    }


# ------------------------------------------------------------------------------------------
# CPU baseline (oracle port of luma-cpu's math path) — bounded sample of the primary workload
# ------------------------------------------------------------------------------------------
def cpu_baseline_prefill(b, hq, hkv, s, d, budget_s=12.0, seed=0):
    from oracle import binding as ob
    cores = ob.hardware_threads()
    group = hq // hkv
    rng = np.random.Generator(np.random.Philox(seed))

    def make(nh_kv):
        q = rng.standard_normal((1, s, nh_kv * group, d), dtype=np.float32)
        k = rng.standard_normal((1, s, nh_kv, d), dtype=np.float32)
        v = rng.standard_normal((1, s, nh_kv, d), dtype=np.float32)
        return q, k, v

    # probe with one KV head (and its query heads) of one batch element
    q, k, v = make(1)
    t0 = time.perf_counter()
    ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    probe = time.perf_counter() - t0
    nh = int(max(1, min(hkv, budget_s / max(probe, 1e-3))))
    if nh > 1:
        q, k, v = make(nh)
        t0 = time.perf_counter()
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
        sec = time.perf_counter() - t0
    else:
        sec = probe
    flops = causal_flops(1, nh * group, s, s, d)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"1 of {b} batch elements x {nh * group} of {hq} query heads ({nh} KV heads), full S={s}, "
                      f"f32 math path over the full key range, {sec:.2f} s; rate counts causal FLOPs only"}, sec


def reference_arm(args):
    """`--impl reference`: the CPU path, timed per step on a bounded sample of the primary workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b, hq, hkv, s, d = 4, 32, 32, 2048, 128
    from oracle import binding as ob
    cores = ob.hardware_threads()
    rng = np.random.Generator(np.random.Philox(0))
    nh = 2
    q = rng.standard_normal((1, s, nh, d), dtype=np.float32)
    k = rng.standard_normal((1, s, nh, d), dtype=np.float32)
    v = rng.standard_normal((1, s, nh, d), dtype=np.float32)
    for _ in range(min(args.warmup, 2)):
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        ob.sdpa_math_f32(q, k, v, causal=True, nthreads=cores)
    sec = time.perf_counter() - t0
    flops = causal_flops(1, nh, s, s, d)
    tf = flops * steps / sec / 1e12
    sample = f"1 of {b} batch elements x {nh} of {hq} heads per step, full S={s}; f32 math path (oracle port of luma-cpu)"
    print(json.dumps({
        "impl": "reference", "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": sec / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "prefill_c2", "batch": b, "q_heads": hq, "kv_heads": hkv, "seq_len": s, "head_dim": d,
                   "causal": True},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, help="run just one workload: prefill_c2, prefill_c3, decode_c4, prefill_c5, decode_c5")
    ap.add_argument("--profile", default=None,
                    help="run ONE workload and nothing else (for ncu): prefill_c2, prefill_c3, prefill_c3_small, "
                         "decode_c4, decode_c4_small, decode_c5")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--small", action="store_true", help="shrink every workload (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.small and not args.profile else args.warmup

    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    from luma_b200 import ffi, low
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the measured path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = load_peaks()
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    if args.profile:
        # one workload, nothing else: the command line the ncu summaries under profiles/ were made with
        name = args.profile
        if name == "prefill_c2":
            res, _ = run_prefill(torch, low, ffi, dev, name, 4, 32, 32, 2048, 128, args.steps, args.warmup, peaks, seed=2)
        elif name == "prefill_c3":
            res, _ = run_prefill(torch, low, ffi, dev, name, 2, 32, 8, 8192, 128, args.steps, args.warmup, peaks, seed=3,
                                 scale_in=0.5, want_lse=False)
        elif name == "prefill_c3_small":   # one batch element, 8 of 32 heads: same kernel, short capture
            res, _ = run_prefill(torch, low, ffi, dev, name, 1, 8, 2, 8192, 128, args.steps, args.warmup, peaks, seed=3,
                                 scale_in=0.5, want_lse=False)
        elif name == "varlen_prefill":
            res = run_varlen_prefill(torch, low, ffi, dev, name, 32, 1024, 8192, 32, 8, 128, args.steps, args.warmup, peaks, seed=7)
        elif name.startswith("softmax_"):   # softmax_<dtype>_<rows>x<row_size>, e.g. softmax_bf16_131072x4096
            _, dtn, shp = name.split("_")
            r_, n_ = (int(t) for t in shp.split("x"))
            res = run_softmax(torch, low, ffi, dev, name, r_, n_, dtn, args.steps, args.warmup, peaks, seed=8)
        elif name == "decode_c4":
            res, _ = run_decode(torch, low, ffi, dev, name, 64, 32, 8, 128, 16, 512, 8192, 40000, args.steps, args.warmup,
                                peaks, seed=4)
        elif name == "decode_c4_small":    # 16 sequences, 12k-page pool (0.8 GB of cache): same kernel
            res, _ = run_decode(torch, low, ffi, dev, name, 16, 32, 8, 128, 16, 512, 8192, 12000, args.steps, args.warmup,
                                peaks, seed=4)
        elif name == "decode_c5":
            res, _ = run_decode(torch, low, ffi, dev, name, 256, 64, 8, 128, 16, 1024, 32768, None, args.steps, args.warmup,
                                peaks, seed=5)
        else:
            raise SystemExit(f"unknown --profile {name}")
        print(json.dumps(res))
        return

    sampler = ClockSampler(local_rank)
    workloads = {}
    only = args.only
    K, W = args.steps, args.warmup

    # ---- primary: BASELINE.json configs[1] --------------------------------------------------
    b, hq, hkv, s, d = (4, 32, 32, 2048, 128) if not args.small else (1, 8, 8, 2048, 128)
    if world == 1:
        sampler.start()
        primary, bufs = run_prefill(torch, low, ffi, dev, "prefill_c2", b, hq, hkv, s, d, K, W, peaks, seed=2)
        q, k, v, o, lse = bufs
        clocks = sampler.stop(torch, lambda: low.flash_attn(q, k, v, o, b, s, s, hq, hkv, d, 0, 1.0 / math.sqrt(d), None, None, lse))
        scaling_note = "single GPU"
    else:
        from luma_b200 import dist as fdist
        q, k, v = make_prefill(torch, dev, b, hq, hkv, s, d, seed=2 + rank)
        lse = torch.empty(b, hq, s, device=dev, dtype=torch.float32)
        # the kernel's epilogue stores this rank's heads into every rank's full output (peer memory
        # over NVLink); one tiny all-reduce then tells everyone that all stores have landed
        peer = fdist.PeerOutput(dist.group.WORLD, (b, s, hq * world, d), torch.bfloat16, dev)
        o_local = peer.out

        def step():
            peer.fused_attention(q, k, v, hq * world, hq * rank, lse=lse)
            peer.sync()

        step()
        path, launches = ffi.last_path(), ffi.last_launches() + 1
        sampler.start()
        sec = time_steps(torch, step, K, W, barrier)
        t = torch.tensor([sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
        clocks = sampler.stop(torch, step, barrier, repeats=0.35 / max(sec / K, 1e-6))
        flops = causal_flops(b, hq, s, s, d) * world
        tf = flops * K / sec / 1e12
        primary = {
            "metric": "prefill attn TFLOP/s", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec / K * 1e3,
            "kernel_path": path, "launches_per_step": launches,
            "config": {"workload": "prefill_c2", "batch": b, "q_heads": hq * world, "kv_heads": hkv * world,
                       "seq_len": s, "head_dim": d, "causal": True, "lse": True, "flops_per_step": flops,
                       "parallelism": f"head-sharded x{world} (32 heads per GPU); the all-gather of O along heads is fused "
                                      "into the kernel epilogue (peer stores over NVLink) + one 4-byte all-reduce",
                       "l2_policy": "inputs larger than L2"},
            "roofline": fused_roofline(flops / world, q.numel() * 2 * (world - 1), sec / K, peaks),
        }
        o = o_local
        scaling_note = "weak: 32 heads per GPU"

    # ---- end to end through the host API with HOST buffers ------------------------------------
    from luma_b200 import high
    hq_h, hk_h, hv_h = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        # the library's host-tensor call: batch elements pipelined over copy-in / kernel / copy-out streams
        high.flash_attn_func_host(hq_h, hk_h, hv_h, ho, None, True, 0, dev)

    e2e_steps = max(3, min(K, 10))
    sec_e2e = time_steps(torch, e2e_step, e2e_steps, 2, barrier)
    if dist is not None:
        t = torch.tensor([sec_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec_e2e = float(t.item())
    e2e_flops = causal_flops(b, hq, s, s, d) * world
    e2e = {"value": e2e_flops * e2e_steps / sec_e2e / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": int((q.numel() + k.numel() + v.numel()) * 2),
           "d2h_bytes_per_step": int(q.numel() * 2), "steps": e2e_steps,
           "note": "luma_b200.high.flash_attn_func_host: pinned host q/k/v -> device, kernel, output -> pinned host, one batch "
                   "element at a time over three streams (both directions of the host link busy), per step, per GPU"}
    del hq_h, hk_h, hv_h, ho

    # ---- the other BASELINE.json configs ------------------------------------------------------
    if world > 1:
        peer.close()
    del q, k, v, o, lse
    torch.cuda.empty_cache()
    if world == 1 and not args.small:
        extra_steps = max(3, min(K, 10))
        if only in (None, "prefill_c3"):
            workloads["prefill_c3"], _b = run_prefill(torch, low, ffi, dev, "prefill_c3", 2, 32, 8, 8192, 128,
                                                      extra_steps, 3, peaks, seed=3, scale_in=0.5, want_lse=False)
            del _b
            torch.cuda.empty_cache()
        if only in (None, "paged_prefill"):
            # the step before decode (not a BASELINE config): 1024-token chunks over paged contexts
            workloads["paged_prefill"] = run_paged_prefill(torch, low, ffi, dev, "paged_prefill", 16, 1024, 32, 8, 128, 16,
                                                           1024, 8192, extra_steps, 3, peaks, seed=6)
            torch.cuda.empty_cache()
        if only in (None, "varlen_prefill"):
            # not a BASELINE config: 32 prompts of 1024..8192 tokens packed, GQA 32/8 (q+k+v+o = 230 MB at the mean)
            workloads["varlen_prefill"] = run_varlen_prefill(torch, low, ffi, dev, "varlen_prefill", 32, 1024, 8192, 32, 8, 128,
                                                             extra_steps, 3, peaks, seed=7)
            torch.cuda.empty_cache()
        if only in (None, "softmax_scores"):
            # not a BASELINE config: the scores of one configs[2]-sized head group on the math path, bf16
            workloads["softmax_scores"] = run_softmax(torch, low, ffi, dev, "softmax_scores", 131072, 4096, "bf16",
                                                      extra_steps, 3, peaks, seed=8)
            torch.cuda.empty_cache()
        if only in (None, "decode_c4"):
            workloads["decode_c4"], _b = run_decode(torch, low, ffi, dev, "decode_c4", 64, 32, 8, 128, 16, 512, 8192,
                                                    40000, max(K, 20), 5, peaks, seed=4)
            del _b
            torch.cuda.empty_cache()

    # ---- BASELINE.json configs[4]: the head-sharded shape, total work fixed, split over N GPUs ----
    if not args.small and only in (None, "prefill_c5", "decode_c5", "c5"):
        extra_steps = max(3, min(K, 10))
        if only in (None, "prefill_c5", "c5"):
            workloads["prefill_c5"] = run_sharded_prefill(torch, low, ffi, dev, dist, world, rank, 1, 64, 8, 16384, 128,
                                                          extra_steps, 3, peaks, seed=50, chunks=4)
            torch.cuda.empty_cache()
        if only in (None, "decode_c5", "c5"):
            workloads["decode_c5"] = run_sharded_decode(torch, low, ffi, dev, dist, world, rank, 256, 64, 8, 128, 16,
                                                        1024, 32768, max(extra_steps, 10), 3, peaks, seed=51)
            torch.cuda.empty_cache()

    # ---- CPU baseline, rank 0, N == 1 only -----------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and not args.small:
        cpu, _ = cpu_baseline_prefill(4, 32, 32, 2048, 128)

    if rank == 0:
        line = {
            "metric": primary["metric"], "value": primary["value"], "unit": primary["unit"],
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": primary["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": primary["config"], "roofline": primary["roofline"],
            "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": int(primary["launches_per_step"]) * K, "kernel_path": primary["kernel_path"],
            "scaling_note": scaling_note, "workloads": workloads,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
