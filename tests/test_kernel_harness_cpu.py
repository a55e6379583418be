"""The collective kernel bodies on the CPU under ThreadSanitizer: every CUDA thread a host thread, flags as atomics
with the PTX's memory order, data accesses plain (csrc/kernels/host_shim.h, tests/cpu_harness/kernel_harness.cc).
A missing flag, fence or barrier - or a block row reading bytes another row staged - shows as a data race; a protocol
that cannot progress ends in the bounded wait's failure record.  AddressSanitizer checks the same run for bounds."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(flag: str, out: Path) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    src = ROOT / "tests" / "cpu_harness" / "kernel_harness.cc"
    deps = [src, ROOT / "tests" / "cpu_harness" / "harness_ext.inc", *(ROOT / "csrc" / "kernels").glob("*.cuh"), *(ROOT / "csrc" / "kernels").glob("*.h")]
    if out.exists() and out.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return
    cmd = ["g++", "-std=c++17", "-O1", "-g", flag, "-Wno-attributes", "-DHCCL_HOST_SHIM", f"-I{ROOT / 'csrc'}", f"-I{ROOT / 'csrc' / 'include'}",
           f"-I{CUDA_HOME}/include", str(src), "-o", str(out), "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


@pytest.mark.skipif(shutil.which("g++") is None or not Path(CUDA_HOME, "include", "cuda_runtime.h").exists(), reason="needs g++ and the CUDA headers")
@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_kernel_bodies_on_cpu_threads(sanitizer):
    exe = ROOT / "build" / f"kernel_harness_{sanitizer}"
    _build(f"-fsanitize={sanitizer}", exe)
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 second_deadlock_stack=1", ASAN_OPTIONS="detect_leaks=0")
    r = subprocess.run([str(exe), "--quick"], capture_output=True, text=True, env=env, timeout=1500)
    assert "ThreadSanitizer" not in r.stderr and "AddressSanitizer" not in r.stderr, r.stderr[-6000:]
    assert r.returncode == 0 and "all checks passed" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


@pytest.mark.skipif(shutil.which("g++") is None or not Path(CUDA_HOME, "include", "cuda_runtime.h").exists(), reason="needs g++ and the CUDA headers")
def test_small_sizes_around_vector_and_slice_boundaries():
    """1 ... 257 elements on 2 and 3 ranks for the bodies whose slicing rounds to 16 bytes (short and empty slices, block
    rows with nothing to do, tails shorter than a vector), under AddressSanitizer; `--edges-all` runs every size, also
    on 5 ranks (several minutes)."""
    exe = ROOT / "build" / "kernel_harness_address"
    _build("-fsanitize=address", exe)
    r = subprocess.run([str(exe), "--edges"], capture_output=True, text=True, env=dict(os.environ, ASAN_OPTIONS="detect_leaks=0"), timeout=1500)
    assert "AddressSanitizer" not in r.stderr, r.stderr[-6000:]
    assert r.returncode == 0 and "all checks passed" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
