"""The C++ host mirror (include/luma_flash_attn.hpp) running the reference's low-level suite
(luma-flash-attn/tests/low.rs: eleven numeric cases, seven error cases) as compiled code."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "tests" / "cpp" / "low_cases"


def test_cpp_host_mirror_is_built():
    # built by __graft_entry__.build() (make -C tests/cpp); header-only mirror + test driver
    if not BIN.exists():
        subprocess.run(["make", "-C", str(BIN.parent), "-s"], check=True)
    assert BIN.exists()


@pytest.mark.gpu
def test_cpp_low_suite_passes_on_gpu():
    if not BIN.exists():
        subprocess.run(["make", "-C", str(BIN.parent), "-s"], check=True)
    out = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-1000:]
    assert out.stdout.count("ok   ") == 18 and "PASSED" in out.stdout
