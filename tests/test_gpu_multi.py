"""Multi-GPU tests (skipped on a single-GPU box): the peer-memory self test and a data-parallel bench
step, each launched as one process per GPU with a loopback rendezvous."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, port, *args, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), *args]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def _last_json(text):
    for line in reversed(text.strip().splitlines()):
        line = line.strip()
        if line.startswith("{"):
            return json.loads(line)
    raise AssertionError("no JSON line in output:\n" + text[-2000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_selftest_two_ranks():
    r = _torchrun(2, 29561, "-m", "rpeg_b200.parallel.selftest")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = _last_json(r.stdout)
    assert rep["ok"] and rep["fused_adam_ok"] and rep["weights_identical_after_grpo"], rep


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_tiny_two_ranks():
    r = _torchrun(2, 29562, "bench.py", "--config", "grpo_tiny", "--gpus", "2", "--steps", "2", "--warmup", "3")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["gpu_launches"] > 0 and line["e2e"]["value"] > 0
