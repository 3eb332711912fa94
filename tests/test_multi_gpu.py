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


def _worlds():
    """Rank counts to exercise: 2, 4 and 8, as far as the box has GPUs (one entry that skips on a single-GPU box)."""
    have = [w for w in (2, 4, 8) if w <= _gpus()]
    return have or [pytest.param(2, marks=pytest.mark.skip(reason="needs at least 2 GPUs"))]


def _run_worker(script: str, world: int, marker: str, tail: int = 3000):
    res = _launch(script, world)
    sys.stdout.write(res.stdout[-tail:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert marker in res.stdout


@pytest.mark.parametrize("world", _worlds())
def test_fused_comm_kernels(world):
    _run_worker("worker_fused_comm.py", world, "FUSED_COMM_RESULTS")


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_channel_gather_fused_into_mlp():
    _run_worker("worker_channel_gather.py", 2, "CHANNEL_GATHER_RESULTS", 2000)


@pytest.mark.parametrize("world", _worlds())
def test_branch_parallel_all_to_all(world):
    _run_worker("worker_branch_a2a.py", world, "BRANCH_A2A_RESULTS", 2000)


@pytest.mark.parametrize("world", _worlds())
def test_model_parallel_render_merge(world):
    _run_worker("worker_mp_render.py", world, "MP_RENDER_RESULTS", 2000)


@pytest.mark.parametrize("world", _worlds())
def test_engine_block_model_parallel_render(world):
    _run_worker("worker_engine_block_mp.py", world, "ENGINE_BLOCK_MP_RESULTS", 2000)


@pytest.mark.parametrize("world", _worlds())
def test_dynamic_loading_nvlink_fanout(world):
    _run_worker("worker_offload_fanout.py", world, "OFFLOAD_FANOUT_RESULTS", 2000)


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
def test_partitioned_optimizer_resumes_from_per_rank_shards():
    _run_worker("worker_zero_resume.py", 2, "ZERO_RESUME_RESULTS", 2000)
