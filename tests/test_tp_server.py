"""The multi-process server and the one-shot generate mode, started the way a user starts them (one process per rank,
rank 0 owns the HTTP port, the others mirror its schedule): requests are served, the same greedy request gives the same
text twice, and a SIGINT to rank 0 ends every rank cleanly through the lockstep stop message. Runs on CPU ranks (gloo,
oracle backend) everywhere and on two GPUs under ``-m gpu`` (CUDA-IPC arena, NVLS off: ranks leave at the end)."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(args, world, extra_env):
    master = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(master), **extra_env)
        procs.append(subprocess.Popen([sys.executable, "-m", "velogb10_b200"] + args, env=env, cwd=ROOT,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    return procs


def _reap(procs, timeout):
    outs = []
    for p in procs:
        try:
            o, e = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()                                    # the exact process this test started
            o, e = p.communicate()
            e += "\n[test] killed after timeout"
        outs.append((p.returncode, o, e))
    return outs


def _post(port, body, timeout=120):
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return r.read().decode()


def _serve_and_generate(backend_args, extra_env, boot_timeout):
    port = _free_port()
    procs = _launch(["--server", "--synthetic", "tiny", "--tp", "2", "--port", str(port), "--host", "127.0.0.1",
                     "--max-batch", "4", "--mtp", "off", "--max-seq-len", "256"] + backend_args, 2, extra_env)
    try:
        t0 = time.time()
        while True:
            if any(p.poll() is not None for p in procs):
                raise AssertionError([(p.returncode, p.stderr.read()[-3000:]) for p in procs if p.poll() is not None])
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                pass
            assert time.time() - t0 < boot_timeout, "server did not come up"
            time.sleep(0.5)
        body = {"model": "m", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 12, "temperature": 0}
        a = json.loads(_post(port, body))
        b = json.loads(_post(port, body))
        assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
        assert a["usage"]["completion_tokens"] >= 1
        s = _post(port, dict(body, stream=True))
        assert "data: [DONE]" in s and "chat.completion.chunk" in s
    finally:
        procs[0].send_signal(signal.SIGINT)             # rank 0 shuts down; its stop message releases the mirror
        outs = _reap(procs, 90)
    assert outs[1][0] == 0, outs[1][2][-3000:]
    assert "killed after timeout" not in outs[0][2] and "killed after timeout" not in outs[1][2]
    # one-shot generation over the same ranks: rank 0 prints the token ids
    gen = _reap(_launch(["--generate", "--synthetic", "tiny", "--tp", "2", "--prompt-ids", "5,6,7,8", "--max-new", "8",
                         "--max-seq-len", "128"] + backend_args, 2, extra_env), 240)
    assert all(rc == 0 for rc, _, _ in gen), [g[2][-2000:] for g in gen]
    assert gen[0][1].strip(), gen[0][2][-2000:]


def test_two_rank_server_and_generate_cpu():
    _serve_and_generate(["--cpu"], {}, 420)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_server_and_generate_gpu():
    _serve_and_generate([], {"VELO_NO_MULTIMEM": "1", "NCCL_NVLS_ENABLE": "0"}, 300)
