"""Compiled-code tests over include/*.h (built by `make -C tests/cpp`):

* the C++ host mirror (include/luma_flash_attn.hpp) running the reference's low-level suite
  (luma-flash-attn/tests/low.rs: eleven numeric cases, seven error cases), linked against the shared
  library and — the way the reference crate links its kernels, luma-flash-attn/build.rs:147-150 —
  against the static archive libflash_attn.a;
* thread-per-rank use of the C ABI (luma-dist/src/scheme/multi_thread.rs:25-48): concurrent calls
  from two host threads, thread-local last-error, and on two or more GPUs the head-sharded prefill
  with luma_comm_from_devices in one process.
"""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CPP = ROOT / "tests" / "cpp"
BINARIES = ("low_cases", "low_cases_static", "thread_per_rank")


def _ensure_built():
    if not all((CPP / b).exists() for b in BINARIES):
        subprocess.run(["make", "-C", str(CPP), "-s"], check=True)


def test_cpp_programs_are_built():
    # built by __graft_entry__.build() (make -C tests/cpp)
    _ensure_built()
    assert all((CPP / b).exists() for b in BINARIES)
    assert (ROOT / "luma_b200" / "lib" / "libflash_attn.a").exists()


@pytest.mark.gpu
@pytest.mark.parametrize("binary", ["low_cases", "low_cases_static"])
def test_cpp_low_suite_passes_on_gpu(binary):
    _ensure_built()
    out = subprocess.run([str(CPP / binary)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-1000:]
    assert out.stdout.count("ok   ") == 18 and "PASSED" in out.stdout


@pytest.mark.gpu
def test_thread_per_rank_calls_on_gpu():
    _ensure_built()
    out = subprocess.run([str(CPP / "thread_per_rank")], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-1000:]
    assert "PASSED" in out.stdout and "FAIL" not in out.stdout
