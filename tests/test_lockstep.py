"""Multi-process lockstep scheduling on CPU ranks (gloo), including the divergence drill."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(env_extra, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1", **env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_lockstep_worker.py")]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)


def test_mirror_replays_head_and_streams_agree():
    r = _run({}, 29551)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    assert r.stdout.count("LOCKSTEP_OK") == 2


def test_divergence_drill_trips_the_guard():
    r = _run({"VELO_TP_AGREE_DRILL": "2"}, 29552)
    assert r.returncode != 0
    assert "DIVERGED" in r.stdout and "LOCKSTEP_OK" not in r.stdout


def test_rank_leaving_between_steps_surfaces_as_divergence():
    """A rank that stops answering (it exits between two steps, nothing of it in flight) must end the survivors
    with DivergenceError through the control group's timeout, never hang them."""
    r = _run({"LOCKSTEP_MODE": "leave"}, 29553)
    assert r.returncode != 0
    assert "DIVERGED rank 0" in r.stdout and "UNEXPECTED_END" not in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


def test_device_failure_on_one_rank_stops_every_rank():
    """One rank's health probe reports a kernel failure: the flag travels in the per-step agreement and both
    ranks raise in the same step."""
    r = _run({"LOCKSTEP_MODE": "fault"}, 29554)
    assert r.returncode != 0
    assert r.stdout.count("DIVERGED") == 2 and "device failure" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
