"""Peer-memory collectives and tensor-parallel inference on 2, 4 and 8 GPUs (spawned as one process per GPU), with
the arena on NVLink-switch multicast memory (in-switch reductions) and on plain CUDA-IPC memory (peer loads / stores)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(script: str, n: int, timeout: int = 420, env_extra=None):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", **(env_extra or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29541 + n), os.path.join(ROOT, "tests", script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-6000:], r.stderr[-1500:])
    return r.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


WORLDS = [pytest.param(w, marks=pytest.mark.skipif(_ngpu() < w, reason=f"needs {w} GPUs")) for w in (2, 4, 8)]
ARENAS = [pytest.param({}, id="multicast"), pytest.param({"VELO_NO_MULTIMEM": "1", "NCCL_NVLS_ENABLE": "0"}, id="ipc")]


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("env", ARENAS)
def test_collectives(world, env):
    out = _spawn("mp_comm_worker.py", world, env_extra=env)
    assert "COMM_OK" in out


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("env", ARENAS)
def test_tensor_parallel_model_matches_single_gpu(world, env):
    out = _spawn("mp_tp_worker.py", world, env_extra=env)
    assert "TP_OK" in out
