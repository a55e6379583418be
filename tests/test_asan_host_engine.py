"""Host code under AddressSanitizer: the library's host objects (API, selector, host engine, verifier, bootstrap) are
built with -fsanitize=address and a slice of the host-engine tests runs against that build in a child interpreter.
Any heap overflow, use after free or stack overflow in host code ends the child with a sanitizer report."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _libasan():
    try:
        path = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True, check=True).stdout.strip()
    except (OSError, subprocess.CalledProcessError):
        return None
    return path if os.path.isabs(path) and os.path.exists(path) else None


@pytest.mark.skipif(_libasan() is None, reason="libasan not installed")
def test_host_engine_slice_is_clean_under_asan():
    build = subprocess.run([sys.executable, str(ROOT / "hccl_b200" / "build.py"), "--asan"], capture_output=True, text=True, cwd=ROOT)
    assert build.returncode == 0, build.stderr[-3000:]
    lib = build.stdout.strip().splitlines()[-1]
    env = dict(os.environ)
    env.update({"HCCL_B200_LIB": lib, "LD_PRELOAD": _libasan(), "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=0:exitcode=66",
                "PYTHONMALLOC": "malloc"})
    select = "test_allreduce_algorithms_and_rank_counts and (3-ring or 5-rhd or 7-nhr or 8-mesh or 4-oneshot) or test_rooted_and_alltoall_ops or test_v_variants_host"
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", "tests/test_host_engine.py", "tests/test_host_executors.py",
                        "tests/test_verifier_selftests.py", "tests/test_host_retry.py", "-k",
                        select + " or test_tree_executor or test_hierarchical_alltoall or test_pipeline_executors or test_semantic_defects or test_dropped_notify"
                        " or test_serial_windowed_all_to_all or (test_three_level_pipeline_all_reduce and 8)"
                        " or (test_concurrent_executors and 5) or (test_all_reduce_over_two_link_sets and 5)"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert "AddressSanitizer" not in r.stdout + r.stderr, tail
    assert r.returncode == 0, tail
    assert " passed" in r.stdout, tail
