"""One process per GPU over the real transport (VMM or IPC peer mappings,
NVLS when the box has it).  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
WORKER = str(Path(__file__).resolve().parent / "_mp_device_worker.py")


def _run(world, scenario, env_extra=None, timeout=600):
    env = dict(os.environ)
    env.update(env_extra or {})
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "root_info")
        procs = [subprocess.Popen([sys.executable, WORKER, str(r), str(world), path, scenario], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n[killed after timeout]"
            outs.append(out)
        return [p.returncode for p in procs], outs


def _world():
    return min(torch.cuda.device_count(), 8)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_collectives_multiprocess():
    codes, outs = _run(_world(), "collectives")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_collectives_multiprocess_p2p_only():
    codes, outs = _run(_world(), "collectives", {"HCCL_NVLS_ENABLE": "0"})
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("nvls", ["0", "1"])
def test_ranks_out_of_step_and_buffers_that_differ_per_rank(nvls):
    codes, outs = _run(_world(), "skew", {"HCCL_NVLS_ENABLE": nvls})
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_switch_allgather_scatter_broadcast_and_cast_reductions():
    codes, outs = _run(_world(), "switch_forms")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_peer_exit_is_detected():
    # NVLS off and plain peer loads: a rank that dies while bound to a multicast object can fault its peers
    codes, outs = _run(min(_world(), 4), "peer_exit", {"HCCL_NVLS_ENABLE": "0", "NCCL_NVLS_ENABLE": "0"}, timeout=120)
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_mc2_fused_multiprocess():
    codes, outs = _run(_world(), "mc2")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_mc2_fused_multiprocess_peer_to_peer_reduce_scatter():
    # Matmul->ReduceScatter without the switch reduction: partial tiles pushed to the owner, reduced by worker CTAs
    codes, outs = _run(_world(), "mc2", {"HCCL_MC2_RS_P2P": "1"})
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_mc2_fused_multiprocess_with_copy_worker_ctas():
    # AllGather->Matmul push form with dedicated copy CTAs instead of the epilogue warps
    codes, outs = _run(_world(), "mc2", {"HCCL_MC2_AG_WORKERS": "16"})
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_cuda_graph_capture_and_replay():
    codes, outs = _run(_world(), "graph")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_torch_distributed_backend():
    codes, outs = _run(_world(), "torch_backend")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_tp_model_gradients_match_nccl_arm():
    codes, outs = _run(_world(), "model")
    assert all(c == 0 for c in codes), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_registered_user_buffers_are_used_in_place():
    codes, outs = _run(_world(), "register")
    assert all(c == 0 for c in codes), "\n".join(outs)
