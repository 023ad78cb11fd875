"""Builds the attention library for sm_100a with nvcc, in-tree (luma_b200/lib/): the static archive
libflash_attn.a the reference crate links (`static=flash_attn`, luma-flash-attn/build.rs:147-148)
and libflash_attn.so for ctypes.

Mirrors what luma-flash-attn/build.rs:47-253 does for the reference crate — find nvcc
(CUDA_HOME / CUDA_PATH / CUDA_ROOT, then PATH), compile every kernels translation unit, `ar rcs`
the objects, link cudart and stdc++ — with two deliberate differences: the architecture is pinned
to compute_100a/sm_100a, and there is no stub: without nvcc the build fails.

`python -m luma_b200.build [--force] [-v] [--trace]`; `--trace` adds -DFA_TRACE (the prefill
kernel's timeline instrumentation, compiled out of the default build).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libflash_attn.so"

ARCHIVE_PATH = LIB_DIR / "libflash_attn.a"

SOURCES = ["api.cu", "tile_simt.cu", "decode_splitk.cu", "prefill_tcgen05.cu", "kv_append.cu", "softmax_lastdim.cu", "comm.cu", "host_pipe.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    for var in ("CUDA_HOME", "CUDA_PATH", "CUDA_ROOT"):
        base = os.environ.get(var)
        if base and (Path(base) / "bin" / "nvcc").exists():
            return str(Path(base) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    if Path("/usr/local/cuda/bin/nvcc").exists():
        return "/usr/local/cuda/bin/nvcc"
    raise RuntimeError("nvcc not found: set CUDA_HOME; this library has no CPU stub")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> Path:
    nvcc = find_nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT.parent / "include").glob("*.h"))
    flag_file = obj_dir / "flags.txt"
    flags = "trace" if trace else "default"
    if not flag_file.exists() or flag_file.read_text() != flags:
        force = True
        flag_file.write_text(flags)
    objs = []
    procs = []
    for name in SOURCES:
        src = CSRC / name
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC",
                   *(["-DFA_TRACE"] if trace else []),
                   "-Xptxas", "-v" if verbose else "-O3", "-c", str(src), "-o", str(obj)]
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {name} ---\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(ARCHIVE_PATH, objs):
        # the archive the reference's build script makes (build.rs:196-208); consumers add cudart and stdc++
        if ARCHIVE_PATH.exists():
            ARCHIVE_PATH.unlink()
        subprocess.run(["ar", "rcs", str(ARCHIVE_PATH), *map(str, objs)], check=True)
    if force or procs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(LIB_PATH), *map(str, objs), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv)
    print(path)
