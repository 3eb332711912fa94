"""Multi-GPU checks of the peer-memory (NVLink) kernels.  Each test launches worker processes with
``torch.distributed.run`` (one per GPU, rendezvous on 127.0.0.1) and is skipped on boxes with one GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(script: str, nproc: int, timeout: int = 600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", "29671", os.path.join(HERE, "multigpu", script)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_fused_comm_kernels():
    res = _launch("worker_fused_comm.py", min(_gpus(), 8))
    sys.stdout.write(res.stdout[-3000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "FUSED_COMM_RESULTS" in res.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_channel_gather_fused_into_mlp():
    res = _launch("worker_channel_gather.py", 2)
    sys.stdout.write(res.stdout[-2000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "CHANNEL_GATHER_RESULTS" in res.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_branch_parallel_all_to_all():
    res = _launch("worker_branch_a2a.py", 2)
    sys.stdout.write(res.stdout[-2000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "BRANCH_A2A_RESULTS" in res.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_model_parallel_render_merge():
    res = _launch("worker_mp_render.py", 2)
    sys.stdout.write(res.stdout[-2000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "MP_RENDER_RESULTS" in res.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_engine_block_model_parallel_render():
    res = _launch("worker_engine_block_mp.py", 2)
    sys.stdout.write(res.stdout[-2000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "ENGINE_BLOCK_MP_RESULTS" in res.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_dynamic_loading_nvlink_fanout():
    res = _launch("worker_offload_fanout.py", 2)
    sys.stdout.write(res.stdout[-2000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "OFFLOAD_FANOUT_RESULTS" in res.stdout
