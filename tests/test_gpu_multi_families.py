"""Multi-GPU tests of the engine plan families (pipeline-parallel training, disjoint generation and training GPUs)
and of PPO on two ranks; skipped on a single-GPU box. The launch helpers are those of ``test_gpu_multi.py``."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from test_gpu_multi import ROOT, _last_json, _torchrun  # noqa: E402


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runtime_graph_with_pipeline_parallel_training_on_two_ranks(tmp_path):
    """The ``pipeline_train`` plan family through the engine backend: generation and the reference pass data parallel,
    the policy update 1F1B over the two ranks as stages, weights switched back to the replicated layout in the
    training node; both ranks' traces carry the pipeline counters and the losses are finite."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "grpo-2gpu-pp", "policy": {"algorithm": "grpo"}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 2},
           "models": {"actor": tiny, "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 2, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 2}, "optimizer": {"k_eval": 2, "plan_family": "pipeline_train"},
           "data": {"synthetic_response_lengths": "quantiles"},     # rows of a group end at different lengths: the rule reward differs
          
           "runtime_hardware": {"worker_overhead_bytes": 0},
           "runtime": {"default_backend": "engine", "gen_slots": 8, "micro_tokens": 256}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    r = _torchrun(2, 29565, "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for trace in ("run.jsonl", "run.rank1.jsonl"):
        events = read_trace(tmp_path / "out/traces" / trace)
        train = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
        assert len(train) == 2 and all(e["status"] == "ok" for e in train)
        for e in train:
            c = e["counters"]
            assert c["pipeline_stages"] == 2 and c["pipeline_p2p_calls"] > 0 and c["layout_switch_bytes"] > 0
            assert c["loss"] == c["loss"] and c["grad_norm"] > 0
    summary = json.loads((tmp_path / "out/metrics/summary.json").read_text())
    assert summary["nodes_failed"] == 0 and summary["logical_steps"] == 2 and summary["nonfinite_losses"] == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runtime_graph_with_generation_and_training_on_disjoint_gpus(tmp_path):
    """The ``disaggregated`` plan family with one step of staleness through the engine backend: rank 0 generates, rank 1
    trains; each side's trace shows its own work (consumed versions 0, 0, 1 on the generation side, published versions
    1, 2, 3 on the training side) and both verify."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "grpo-2gpu-async", "policy": {"algorithm": "grpo", "tau": {"actor": 1}}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 2},
           "models": {"actor": tiny, "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 2, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 3}, "optimizer": {"k_eval": 3, "plan_family": "disaggregated"},
           "data": {"synthetic_response_lengths": "quantiles"},
          
           "runtime_hardware": {"worker_overhead_bytes": 0}, "checkpoints": {"interval_steps": 100, "save_final": False},
           "runtime": {"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024, "node_timeout_s": 120}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29566", "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"])]
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    gen = [e for e in read_trace(tmp_path / "out/traces/run.jsonl") if e["event"] == "finish" and e["node_id"].startswith("g_pi@")
           and "generated_tokens" in e["counters"]]
    assert [e["counters"]["weight_version"] for e in gen] == [0, 0, 1] and all(e["counters"]["generated_tokens"] > 0 for e in gen)
    train = [e for e in read_trace(tmp_path / "out/traces/run.rank1.jsonl") if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
    assert [e["counters"]["published_version"] for e in train] == [1.0, 2.0, 3.0]
    assert all(e["counters"]["loss"] == e["counters"]["loss"] and e["counters"]["grad_norm"] > 0 for e in train)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_tiny_pipeline_trained_two_ranks():
    """Data-parallel generation with a pipeline-parallel policy update, through bench.py's own loop."""
    r = _torchrun(2, 29567, "bench.py", "--config", "grpo_tiny_pp", "--gpus", "2", "--steps", "1", "--warmup", "3")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = _last_json(r.stdout)
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["config"]["parallelism"] == "generation dp2, training pp2"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runtime_graph_ppo_on_two_ranks(tmp_path):
    """PPO (actor, critic, reward, reference) through the engine backend on two data-parallel ranks: both optimizers run
    their fused data-parallel step (the critic's through a cloned context with its own barrier slots)."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "ppo-2gpu", "policy": {"algorithm": "ppo"}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 2},
           "models": {"actor": tiny, "critic": dict(tiny), "reward": dict(tiny), "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 1, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 2}, "optimizer": {"k_eval": 2}, "runtime_hardware": {"worker_overhead_bytes": 0},
           "runtime": {"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    r = _torchrun(2, 29568, "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    events = read_trace(tmp_path / "out/traces/run.jsonl")
    for prefix, key in (("t_pi@", "grad_norm"), ("t_V@", "critic_grad_norm")):
        fin = [e for e in events if e["event"] == "finish" and e["node_id"].startswith(prefix)]
        assert len(fin) == 2 and all(e["status"] == "ok" and e["counters"][key] > 0 for e in fin)
    summary = json.loads((tmp_path / "out/metrics/summary.json").read_text())
    assert summary["nodes_failed"] == 0 and summary["nonfinite_losses"] == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_runtime_graph_with_tensor_parallel_generation_on_two_ranks(tmp_path):
    """The ``tp_generation`` plan family through the engine backend: the generation vertex runs tensor parallel over both
    ranks (every rank decodes all rows on its weight shard), the RESHARD node of the publication edge re-slices the
    updated weights and reports its device time, the other vertices run data parallel."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "grpo-2gpu-tpgen", "policy": {"algorithm": "grpo"}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 2},
           "models": {"actor": tiny, "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 2, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 2}, "optimizer": {"k_eval": 2, "plan_family": "tp_generation"},
           "data": {"synthetic_response_lengths": "quantiles"}, "runtime_hardware": {"worker_overhead_bytes": 0},
           "runtime": {"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    r = _torchrun(2, 29569, "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for trace in ("run.jsonl", "run.rank1.jsonl"):
        events = read_trace(tmp_path / "out/traces" / trace)
        gen = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("g_pi@") and "generated_tokens" in e["counters"]]
        assert len(gen) == 2 and all(e["counters"]["generated_tokens"] > 0 for e in gen)
        train = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
        assert len(train) == 2 and all(e["status"] == "ok" and e["counters"]["grad_norm"] > 0 for e in train)
        switches = [e for e in events if e["event"] == "finish" and e["counters"].get("transport") == "layout_switch"]
        assert switches and all(e["counters"]["reshard_us"] > 0 and e["counters"]["transferred_bytes"] > 0 for e in switches)
    summary = json.loads((tmp_path / "out/metrics/summary.json").read_text())
    assert summary["nodes_failed"] == 0 and summary["logical_steps"] == 2 and summary["nonfinite_losses"] == 0


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_runtime_graph_with_generation_in_two_tensor_parallel_groups_on_four_ranks(tmp_path):
    """``optimizer.generation_tp: 2`` on four ranks: generation layout (2, 1, 2). Each group of two ranks decodes the rows of
    its own prompts tensor parallel; every rank then trains on its slice and the gradients are reduced over all four."""
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import plan_runtime_job
    from rpeg_b200.runtime.trace import read_trace
    tiny = {"layers": 2, "hidden_dim": 256, "ffn_dim": 512, "vocab_size": 512, "head_dim": 128}
    cfg = {"run_id": "grpo-4gpu-tpgroups", "policy": {"algorithm": "grpo"}, "hardware": {"preset": "b200_nvswitch"},
           "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4},
           "models": {"actor": tiny, "reference": {"source": "actor"}},
           "workload": {"batch_size": 8, "samples_per_prompt": 2, "context_length": 32, "generation_length": 48,
                        "gen_quantiles": [[0.5, 16], [1.0, 48]]},
           "training": {"max_steps": 2}, "optimizer": {"k_eval": 2, "plan_family": "tp_generation", "generation_tp": 2},
           "data": {"synthetic_response_lengths": "quantiles"}, "runtime_hardware": {"worker_overhead_bytes": 0},
           "runtime": {"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024}, "outputs": {"seed": 3}}
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    assert tuple(res["compiled"].config.plan.pi["g_pi"]) == (2, 1, 2)
    r = _torchrun(4, 29576, "-m", "rpeg_b200.runtime.run", "--config", str(res["run_file"]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for trace in ("run.jsonl", "run.rank1.jsonl", "run.rank2.jsonl", "run.rank3.jsonl"):
        events = read_trace(tmp_path / "out/traces" / trace)
        gen = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("g_pi@") and "generated_tokens" in e["counters"]]
        assert len(gen) == 2 and all(e["counters"]["generated_tokens"] > 0 for e in gen)
        train = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("t_pi@")]
        assert len(train) == 2 and all(e["status"] == "ok" and e["counters"]["grad_norm"] > 0 for e in train)
    summary = json.loads((tmp_path / "out/metrics/summary.json").read_text())
    assert summary["nodes_failed"] == 0 and summary["logical_steps"] == 2 and summary["nonfinite_losses"] == 0
