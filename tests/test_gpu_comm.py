"""Peer-memory collectives and tensor-parallel inference on 2+ GPUs (spawned as one process per GPU).
NVLS is switched off in the library used for bootstrap; the kernels under test use plain peer loads/stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(script: str, n: int, timeout: int = 300):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    return r.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_collectives_two_ranks():
    out = _spawn("mp_comm_worker.py", 2)
    assert "COMM_OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_model_matches_single_gpu():
    out = _spawn("mp_tp_worker.py", 2)
    assert "TP_OK" in out
