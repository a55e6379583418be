"""CPU-side checks of the Python layers that need no GPU: backend registration, reduce-op mapping, and the PyTorch
expressions the fused element-wise kernels fall back to (and are compared against on the GPU)."""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from hccl_b200.ops import fused


def test_torch_backend_is_registered_and_maps_reduce_ops():
    import hccl_b200.torch_backend as tb
    from hccl_b200.types import ReduceOp

    assert "HCCL" in dist.Backend._plugins
    tb.register()                                   # idempotent
    assert tb._red(dist.ReduceOp.SUM) == ReduceOp.SUM
    assert tb._red(dist.ReduceOp.PRODUCT) == ReduceOp.PROD
    assert tb._red(dist.ReduceOp.MAX) == ReduceOp.MAX
    assert tb._red(dist.ReduceOp.MIN) == ReduceOp.MIN
    try:
        tb._red(dist.ReduceOp.BAND)
        raised = False
    except NotImplementedError:
        raised = True
    assert raised


def test_fused_ops_take_the_reference_path_on_cpu_tensors():
    torch.manual_seed(0)
    x, d, w = torch.randn(6, 32), torch.randn(6, 32), torch.rand(32) + 0.5
    x_out, h = fused.add_rms_norm(x, d, w, 1e-5)
    assert torch.equal(x_out, x + d)
    torch.testing.assert_close(h, F.rms_norm(x + d, (32,), w, 1e-5))
    x2, h2 = fused.add_rms_norm(x, None, w, 1e-5)
    assert x2 is x
    torch.testing.assert_close(h2, F.rms_norm(x, (32,), w, 1e-5))
    gu = torch.randn(5, 16)
    torch.testing.assert_close(fused.swiglu(gu), F.silu(gu[:, :8]) * gu[:, 8:])
    q = torch.randn(7, 2, 8)
    ang = torch.rand(7, 4)
    out = fused.rope(q, ang.cos(), ang.sin())
    # a rotation preserves the norm of every (i, i + d/2) pair
    torch.testing.assert_close(out[..., :4] ** 2 + out[..., 4:] ** 2, q[..., :4] ** 2 + q[..., 4:] ** 2)


def test_decoder_stack_runs_on_cpu_with_reference_ops():
    """World size 1, CPU tensors: the model code path (residual stream + pending delta) against a plain restatement."""
    from hccl_b200.models.llama import rope_tables

    torch.manual_seed(1)
    s, hdim, heads, d = 16, 32, 2, 16
    x = torch.randn(s, hdim)
    w = torch.ones(hdim)
    cos, sin = rope_tables(s, d, 10000.0, x.device)
    x1, h1 = fused.add_rms_norm(x, None, w, 1e-5, use_kernels=False)
    x2, h2 = fused.add_rms_norm(x1, h1, w, 1e-5, use_kernels=False)
    torch.testing.assert_close(x2, x + F.rms_norm(x, (hdim,), w, 1e-5))
    q = fused.rope(h2.view(s, heads, d), cos, sin, use_kernels=False)
    assert q.shape == (s, heads, d)


def test_python_wrapper_overhead_over_raw_ctypes():
    """The Python method adds little over the raw ctypes call of the same operator (the reference budgets 10 us for its
    wrapper: 20 warm-up calls, 100 timed, count 8).  A single-rank communicator takes the local-copy shortcut, so the
    time is entry code only.  The bound here is loose because the CPU this runs on is shared."""
    import ctypes
    import time

    import numpy as np

    import hccl_b200 as hb
    from hccl_b200._lib import lib
    from hccl_b200.types import DataType, ReduceOp

    comm = hb.Communicator.host_sim(1)[0]
    x, y = np.arange(8, dtype=np.float32), np.zeros(8, np.float32)
    px, py = x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p)

    def best(fn):
        for _ in range(20):
            fn()
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            for _ in range(100):
                fn()
            times.append((time.perf_counter() - t0) / 100)
        return min(times) * 1e6

    raw = best(lambda: lib.HcclAllReduce(px, py, 8, int(DataType.FP32), int(ReduceOp.SUM), comm.handle, None))
    wrapped = best(lambda: comm.all_reduce(x, y))
    assert np.array_equal(y, x)
    assert wrapped - raw < 50.0, (raw, wrapped)
    comm.destroy()


def test_hccl_test_command_line_on_the_host_engine():
    """The hccl_test-style tool prints one row per size with a passing result check."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for op, extra in (("all_reduce", ["-o", "max", "-d", "int32"]), ("reduce_scatter", ["-d", "fp16"]), ("alltoall", ["-d", "int64"])):
        r = subprocess.run([sys.executable, str(root / "bench" / "hccl_test.py"), "--op", op, "-b", "1K", "-e", "16K", "-f", "4", "-p", "3", "-n", "2", "-w", "1",
                            "--host-sim", *extra], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        rows = [l.split() for l in r.stdout.splitlines() if l.strip() and not l.startswith("#") and not l.strip().startswith("data_size")]
        assert [int(x[0]) for x in rows] == [1024, 4096, 16384], r.stdout
        assert all(x[3] == "success" for x in rows), r.stdout
