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


def _torchrun(n, port, *args, timeout=300):
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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runtime_graph_on_two_ranks_with_the_engine_backend(tmp_path):
    """Plan a tiny GRPO job for the engine backend on two GPUs (data-parallel plan family), execute the run file with
    one process per GPU and check rank 0's verified trace, the summary and the other rank's own trace."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "grpo-2gpu", "policy": {"algorithm": "grpo"}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 2},
           "models": {"actor": tiny, "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 2, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 2}, "optimizer": {"k_eval": 2}, "runtime_hardware": {"worker_overhead_bytes": 0},
           "runtime": {"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    r = _torchrun(2, 29563, "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    events = read_trace(tmp_path / "out/traces/run.jsonl")
    train = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
    assert len(train) == 2 and all(e["status"] == "ok" and e["counters"]["kernel_launches"] > 0 for e in train)
    summary = json.loads((tmp_path / "out/metrics/summary.json").read_text())
    assert summary["nodes_failed"] == 0 and summary["logical_steps"] == 2 and summary["nonfinite_losses"] == 0
    other = read_trace(tmp_path / "out/traces/run.rank1.jsonl")
    assert sum(1 for e in other if e["event"] == "finish" and e["node_id"].startswith("t_pi@")) == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_tiny_async_two_ranks():
    """Generation and training on disjoint ranks with one step of staleness, through bench.py's own loop."""
    r = _torchrun(2, 29564, "bench.py", "--config", "grpo_tiny_async", "--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["config"]["algorithm"] == "grpo_async"
    assert line["config"]["parallelism"].startswith("gen1+train1")
