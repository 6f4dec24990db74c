"""CPU tests of the auxiliary tools: generation profile, cost calibration, environment check,
distributed validation over gloo, suite report, calibrate.py fits."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from rpeg_b200.runtime.compiler import compile_runtime_plan
from rpeg_b200.runtime.cost_calibration import calibrate_costs, fit_scale
from rpeg_b200.runtime.environment_check import run_checks
from rpeg_b200.runtime.generation_profile import build_profile, quantiles_from_lengths
from rpeg_b200.runtime.suite_report import aggregate
from rpeg_b200.analytic.cost import NodeCostModel
from rpeg_b200.analytic.hardware import b200_nvswitch
from test_runtime_metadata import spread_job

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_generation_profile_quantiles():
    lengths = [10] * 50 + [300] * 40 + [2048] * 10
    q = quantiles_from_lengths(lengths, 2048)
    assert q == [[0.5, 64], [0.9, 320], [1.0, 2048]]
    assert quantiles_from_lengths([5, 5, 5, 5], 128) == [[0.5, 64], [1.0, 128]]       # degenerate phases merge
    prof = build_profile(lengths, 2048)
    assert prof["schema_version"] == "rpeg.generation_profile.v1" and prof["truncated_fraction"] == 0.1
    with pytest.raises(ValueError):
        quantiles_from_lengths([], 10)


def test_job_planner_ingests_generation_profile(tmp_path):
    from rpeg_b200.runtime.io import dump_mapping
    from rpeg_b200.runtime.job_plan import job_workload
    prof = build_profile([10] * 50 + [100] * 50, 256)
    (tmp_path / "p.json").write_text(json.dumps(prof))
    cfg = {"workload": {"batch_size": 8, "context_length": 16, "generation_length": 256}, "generation_profile": {"path": "p.json"}}
    wl = job_workload(cfg, tmp_path)
    assert wl.gen_quantiles == ((0.5, 64), (0.9, 128), (1.0, 256))
    cfg["workload"]["generation_length"] = 512
    from rpeg_b200.runtime.errors import RuntimeConfigError
    with pytest.raises(RuntimeConfigError, match="max_new_tokens"):
        job_workload(cfg, tmp_path)


def test_cost_calibration_recovers_scales(tmp_path):
    compiled = compile_runtime_plan(spread_job(tmp_path, "ppo", steps=2, width=1))
    hw = b200_nvswitch(mem=float(compiled.run_config.hardware.memory_per_gpu_bytes))
    cost = NodeCostModel(hw, compiled.model_suite, compiled.workload, optimizer_stage=1, activation_checkpointing=True)
    events, t = [], 0.0
    factor = {"GEN": 1.5, "INF": 0.8, "TRAIN": 2.0}
    for n in compiled.lowered.nodes:
        f = factor[n.role.value] if n.role is not None and n.op is not None else 1.25
        d = cost.time(n) * f
        events.append({"node_id": n.id, "event": "start", "status": "ok", "timestamp": t, "counters": {}})
        events.append({"node_id": n.id, "event": "finish", "status": "ok", "timestamp": t + d, "counters": {"duration_s": d}})
        t += d
    rep = calibrate_costs(compiled, events, hw)
    assert rep["matched_nodes"] == len(compiled.lowered.nodes)
    assert rep["hardware"]["op_generation_scale"] == pytest.approx(1.5, rel=1e-6)
    assert rep["hardware"]["op_inference_scale"] == pytest.approx(0.8, rel=1e-6)
    assert rep["hardware"]["op_training_scale"] == pytest.approx(2.0, rel=1e-6)
    assert fit_scale([(1.0, 2.0), (2.0, 4.0)]) == pytest.approx(2.0) and fit_scale([]) is None


def test_environment_check_and_suite_report(tmp_path):
    rep = run_checks(need_gpu=False)
    assert rep["schema_version"] == "rpeg.environment_check.v1" and rep["ok"]
    names = {c["name"] for c in rep["checks"]}
    assert {"package:torch", "kernels:built", "kernels:abi"} <= names
    (tmp_path / "env.json").write_text(json.dumps(rep))
    (tmp_path / "bench.json").write_text(json.dumps({"metric": "m", "value": 1.0, "gpu_launches": 5}))
    (tmp_path / "ref.json").write_text(json.dumps({"impl": "reference", "unavailable": "x"}))
    (tmp_path / "bad.json").write_text(json.dumps({"schema_version": "rpeg.runtime_alerts.v1", "status": "critical", "alerts": [1]}))
    good = aggregate([str(tmp_path / "env.json"), str(tmp_path / "bench.json"), str(tmp_path / "ref.json")])
    assert good["ok"] and [i["kind"] for i in good["items"]] == ["environment_check", "bench", "bench_reference"]
    from rpeg_b200.runtime.suite_report import classify
    assert classify({"schema_version": "rpeg.engine_validate.v1", "ok": False, "world": 8, "checks": [{"name": "train_step", "ok": False}]}) == \
        {"kind": "engine_validate", "ok": False, "detail": {"world": 8, "failed": ["train_step"], "error": None}}
    assert classify({"schema_version": "rpeg.cluster_contract.v1", "performance_comparable": True, "nodes": 2})["ok"] is True
    from rpeg_b200.runtime.collective_benchmark import large_message_gate
    rows = [{"bytes": 10 ** 6, "nccl_all_reduce_busbw_gbs": 40.0}, {"bytes": 10 ** 9, "nccl_all_reduce_busbw_gbs": 550.0}]
    assert large_message_gate(rows, 300.0) == {"ok": True, "min_large_message_gbps": 300.0, "measured_gbps": 550.0, "bytes": 10 ** 9}
    assert not large_message_gate(rows, 600.0)["ok"] and not large_message_gate([], 0.0)["ok"] and large_message_gate(rows, 0.0)["ok"]
    slow = {"schema_version": "rpeg.collective_benchmark.v1", "world": 8, "rows": rows, "gate": large_message_gate(rows, 600.0)}
    assert classify(slow)["ok"] is False and classify(dict(slow, gate=large_message_gate(rows, 300.0)))["ok"] is True
    bad = aggregate([str(tmp_path / "env.json"), str(tmp_path / "bad.json"), str(tmp_path / "missing.json")])
    assert not bad["ok"] and len(bad["failed"]) == 2


def test_distributed_validate_over_gloo(tmp_path):
    out = tmp_path / "dist.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), "-m", "rpeg_b200.runtime.distributed_validate", "--backend", "gloo",
           "--output", str(out)]
    r = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rep = json.loads(out.read_text())
    assert rep["ok"] and rep["world"] == 2 and rep["all_reduce_sum"] == rep["expected_sum"] and len(rep["ranks"]) == 2


def test_calibrate_fits():
    sys.path.insert(0, ROOT)
    import calibrate as c
    a, b = c.fit_alpha_beta([1e5, 2e5, 1e6, 1e7, 1e8], [2e-5 + s * 1.3e-12 for s in (1e5, 2e5, 1e6, 1e7, 1e8)])
    assert a == pytest.approx(2e-5, rel=1e-3) and b == pytest.approx(1.3e-12, rel=1e-6)
    assert c.fit_gemm_m_half([128, 1024, 8192], [128 / 224, 1024 / 1120, 8192 / 8288]) == pytest.approx(96.0)


def test_model_registry_and_hf_helpers(tmp_path):
    import struct
    from rpeg_b200.models.registry import config_from_hf, hf_config_dict
    from rpeg_b200.runtime.errors import RuntimeConfigError
    from rpeg_b200.runtime.hf import (model_spec_from_hf_config, require_pinned_revision, resolve_model_path, safetensors_header,
                                      safetensors_parameter_count)
    llama3 = {"model_type": "llama", "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "num_hidden_layers": 32,
              "intermediate_size": 14336, "vocab_size": 128256, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
              "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192}}
    c = config_from_hf(llama3, max_pos=4096)
    assert (c.n_kv_heads, c.rope_scaling_factor, c.qk_norm, c.family, c.max_pos) == (8, 8.0, False, "llama", 4096)
    q = config_from_hf({"model_type": "qwen3", "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                        "num_hidden_layers": 36, "intermediate_size": 12288, "vocab_size": 151936, "tie_word_embeddings": False})
    assert q.qk_norm and q.rms_eps == 1e-6 and q.rope_theta == 1e6
    assert config_from_hf(hf_config_dict(q)) == q
    for bad in ({**llama3, "model_type": "mixtral"}, {**llama3, "attention_bias": True}, {**llama3, "hidden_size": 4096, "num_attention_heads": 64},
                {**llama3, "rope_scaling": {"rope_type": "yarn", "factor": 4.0}}):
        with pytest.raises(RuntimeConfigError):
            config_from_hf(bad)
    spec = model_spec_from_hf_config(llama3)
    assert (spec.L, spec.d, spec.d_ff, spec.V) == (32, 4096, 14336, 128256)
    with pytest.raises(RuntimeConfigError):
        require_pinned_revision("org/model", "main")
    assert require_pinned_revision("org/model", "a" * 40) == "a" * 40
    with pytest.raises(RuntimeConfigError):
        resolve_model_path("hf", "org/model", None, "a" * 40)
    # header-only parameter count on a hand-written safetensors file
    header = json.dumps({"a": {"dtype": "BF16", "shape": [3, 4], "data_offsets": [0, 24]},
                         "b": {"dtype": "BF16", "shape": [5], "data_offsets": [24, 34]}, "__metadata__": {"format": "pt"}}).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 34)
    assert set(safetensors_header(tmp_path / "m.safetensors")) == {"a", "b", "__metadata__"}
    assert safetensors_parameter_count(tmp_path) == 17


def test_hf_weight_roundtrip_on_cpu(tmp_path):
    import torch
    from rpeg_b200.models.llama import LlamaConfig, ParamLayout
    from rpeg_b200.runtime.hf import load_hf_weights, save_hf_weights

    class Flat:                     # the part of LlamaModel the import/export touches, on the CPU
        def __init__(self, cfg, fill):
            self.cfg, self.layout = cfg, ParamLayout(cfg)
            self.w = torch.zeros(self.layout.total, dtype=torch.bfloat16)
            if fill:
                self.w.copy_(torch.randn(self.layout.total).bfloat16())
            self.p = {n: self.layout.view(self.w, n) for n in self.layout.entries}

    cfg = LlamaConfig.tiny(n_heads=4, n_kv_heads=2, d_model=512, qk_norm=True, family="qwen3")
    a, b = Flat(cfg, True), Flat(cfg, False)
    save_hf_weights(a, tmp_path / "ckpt", shard_bytes=1 << 20)
    assert len(list((tmp_path / "ckpt").glob("*.safetensors"))) > 1
    n = load_hf_weights(b, tmp_path / "ckpt")
    assert n == sum(int(v.numel()) for v in a.p.values())
    for name in a.p:
        assert torch.equal(a.p[name], b.p[name]), name
    from rpeg_b200.models.registry import config_from_hf_path
    assert config_from_hf_path(tmp_path / "ckpt", max_pos=cfg.max_pos) == cfg


def test_experiment_generators_and_optimizer_bench(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "experiments"))
    import gen_ablation_configs as ab
    import gen_scaling_configs as sc
    import optimizer_bench as ob
    from rpeg_b200.planner.pipeline import load_yaml, validate_config
    assert sc.generate(tmp_path / "scaling") == 108
    cfg = load_yaml(str(tmp_path / "scaling/both/128gpu_t896_tau2.yaml"))
    validate_config(cfg)
    assert cfg["hardware"]["racks"] * cfg["hardware"]["nodes_per_rack"] * cfg["hardware"]["gpus_per_node"] == 128
    assert cfg["workload"]["gen_quantiles"] == [[0.5, 224], [0.85, 448], [1.0, 896]]
    assert cfg["optimizer"]["staleness_candidates"] == {"actor": [2], "critic": [1]}
    assert ab.generate(tmp_path / "ablation", ("tight",)) == 50
    a1 = load_yaml(str(tmp_path / "ablation/A1_no_gen_inf_overlap/tight_16gpu_s3.yaml"))
    base = load_yaml(str(tmp_path / "ablation/baseline/tight_16gpu_s3.yaml"))
    assert "gen_quantiles" not in a1["workload"] and "gen_quantiles" in base["workload"] and a1["output"]["seed"] == 3
    a1["workload"]["gen_quantiles"] = base["workload"]["gen_quantiles"]
    a1["output"]["log_file"] = base["output"]["log_file"]
    assert a1 == base                                     # nothing but the ablated knob differs
    row = ob.bench_instance("micro2", seeds=2, evals=200)
    assert row["space_size"] == 625 and row["worst_gap"] <= 0.03 and 0 < row["coverage"] <= 1


def test_dataset_and_minibatch_indices():
    from rpeg_b200.runtime.data import dataset_batch_indices, minibatch_indices
    assert dataset_batch_indices(10, 4, 1) == [0, 1, 2, 3]
    assert dataset_batch_indices(10, 4, 3) == [8, 9, 0, 1]                      # windows wrap around
    a = dataset_batch_indices(10, 4, 2, seed=5, shuffle=True)
    assert a == dataset_batch_indices(10, 4, 2, seed=5, shuffle=True) and len(set(a)) == 4
    seen = sorted(i for s in (1, 2, 3) for i in dataset_batch_indices(12, 4, s, seed=1, shuffle=True))
    assert seen == list(range(12))                                              # one pass visits every row once
    mbs = minibatch_indices(10, 4, epochs=2, seed=3)
    assert [len(m) for m in mbs] == [4, 4, 2, 4, 4, 2]
    assert sorted(i for m in mbs[:3] for i in m) == list(range(10)) == sorted(i for m in mbs[3:] for i in m)
    assert mbs[:3] != mbs[3:]                                                   # a fresh order every epoch
    assert minibatch_indices(6, None, epochs=2) == [list(range(6))] * 2
    assert [len(m) for m in minibatch_indices(10, 4, drop_last=True)] == [4, 4]
    with pytest.raises(ValueError):
        minibatch_indices(0, 4)


def test_quantile_lengths_follow_the_workload_phases():
    from rpeg_b200.runtime.data import quantile_lengths
    from rpeg_b200.runtime.errors import RuntimeConfigError
    from rpeg_b200.runtime.schema import DataConfig, _build
    q = ((0.5, 128), (0.85, 256), (1.0, 512))
    lens = quantile_lengths(4000, q, seed=7)
    assert lens == quantile_lengths(4000, q, seed=7) != quantile_lengths(4000, q, seed=8)
    assert min(lens) >= 1 and max(lens) <= 512
    frac = [sum(1 for l in lens if l <= b) / len(lens) for _, b in q]
    assert frac[0] == pytest.approx(0.5, abs=0.03) and frac[1] == pytest.approx(0.85, abs=0.03) and frac[2] == 1.0
    mean = 0.5 * 64.5 + 0.35 * 192.5 + 0.15 * 384.5
    assert sum(lens) / len(lens) == pytest.approx(mean, rel=0.05)
    assert quantile_lengths(0, q) == []
    assert _build(DataConfig, {"synthetic_response_lengths": "quantiles"}, "data").synthetic_response_lengths == "quantiles"
    assert _build(DataConfig, {}, "data").synthetic_response_lengths == "cap"
    with pytest.raises(RuntimeConfigError):
        _build(DataConfig, {"synthetic_response_lengths": "short"}, "data")


def test_dot_writers_cover_template_unrolled_and_lowered_graphs(tmp_path):
    from rpeg_b200.analytic.models import ModelSpec, ModelSuite
    from rpeg_b200.analytic.workload import Workload
    from rpeg_b200.core.types import Allocation, Model
    from rpeg_b200.ir.plan import ExecutionPlan
    from rpeg_b200.ir.templates import build_PPO_RPEG
    from rpeg_b200.passes.lower import lower
    from rpeg_b200.passes.unroll import unroll
    from rpeg_b200.utils.visualize import exec_to_dot, rpeg_to_dot, unrolled_to_dot
    spec = ModelSpec(8, 1024, 2816, 32000)
    suite = ModelSuite({m: spec for m in Model})
    wl = Workload(16, 1, 64, 128, ((0.5, 32), (1.0, 128)))
    r = build_PPO_RPEG(suite, wl, tau={Model.ACTOR: 1, Model.CRITIC: 0})
    un = unroll(r, 3)
    plan = ExecutionPlan()
    for i, v in enumerate(r.vertices):
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, i % 4), (1, 1, 1)), (1, 1, 1), 1
    low = lower(r, un, plan, suite, 3, workload=wl)
    t1, t2, t3 = rpeg_to_dot(r, str(tmp_path / "a.dot")), unrolled_to_dot(un, str(tmp_path / "b.dot")), exec_to_dot(low, str(tmp_path / "c.dot"))
    assert t1.startswith("digraph") and all(v.id in t1 for v in r.vertices)
    assert t2.count("subgraph cluster_") == 3 and '"t_pi@0" -> "g_pi@2"' in t2 and "style=dashed" in t2   # staleness 1: weights of step 0 serve step 2
    assert all(n.id in t3 for n in low.nodes)
    assert (tmp_path / "b.dot").read_text() == t2


def test_cost_model_validation_statistics_and_chart(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("pcv", os.path.join(ROOT, "experiments", "plot_cost_model_validation.py"))
    pcv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(pcv)
    st = pcv.validation_stats([(1.0, 1.0), (2.2, 2.0), (0.5, 1.0)])
    assert st["n"] == 3 and st["mape"] == pytest.approx((0 + 0.1 + 0.5) / 3) and st["within_25pct"] == pytest.approx(2 / 3)
    assert pcv.validation_stats([(3.0, 3.0), (9.0, 9.0)])["log_r2"] == pytest.approx(1.0)
    rep = {"nodes": [{"class": "GEN", "predicted_s": 10.0, "measured_s": 11.0}, {"class": "TRAIN", "predicted_s": 5.0, "measured_s": 4.0},
                     {"class": "INF", "predicted_s": 0.001, "measured_s": 0.002}]}
    (tmp_path / "r.json").write_text(json.dumps(rep))
    assert pcv.main([str(tmp_path / "r.json"), "--output", str(tmp_path / "v.svg")]) == 0
    svg = (tmp_path / "v.svg").read_text()
    assert svg.startswith("<svg") and svg.count("<circle") == 2          # the 2 ms node is below --min-seconds


def test_slurm_inventory_from_the_environment():
    from rpeg_b200.core.types import Allocation, DeviceSpace
    from rpeg_b200.runtime.cluster import expand_nodelist, slurm_inventory
    from rpeg_b200.runtime.errors import RuntimeConfigError
    assert expand_nodelist("gpu[01-03,07],login1") == ("gpu01", "gpu02", "gpu03", "gpu07", "login1")
    assert expand_nodelist("nid005") == ("nid005",)
    space = DeviceSpace(1, 2, 4)
    inv = slurm_inventory(space, {"SLURM_JOB_NODELIST": "b200-[10-11]"})
    refs = inv.resolve_allocation(Allocation((0, 1, 2), (1, 1, 2)))
    assert [(r.hostname, r.local_cuda_index, r.global_rank) for r in refs] == [("b200-11", 2, 6), ("b200-11", 3, 7)]
    with pytest.raises(RuntimeConfigError):
        slurm_inventory(space, {"SLURM_JOB_NODELIST": "b200-10"})
    with pytest.raises(RuntimeConfigError):
        slurm_inventory(space, {})


def test_scaling_sweep_script_writes_csv_and_chart(tmp_path):
    gen = subprocess.run([sys.executable, os.path.join(ROOT, "experiments", "gen_scaling_configs.py"), "--out", str(tmp_path / "cfg")],
                         capture_output=True, text=True, cwd=ROOT)
    assert gen.returncode == 0, gen.stderr[-2000:]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "experiments", "run_scaling.py"), str(tmp_path / "cfg"), "--match", "actor/16gpu_t128_sync",
                        "--time", "1", "--csv", str(tmp_path / "s.csv"), "--plot", str(tmp_path / "s.svg")], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rows = (tmp_path / "s.csv").read_text().strip().splitlines()
    assert len(rows) == 2 and "optimized_tokens_per_s" in rows[0] and rows[1].startswith("16gpu_t128_sync.yaml,16,")
    assert (tmp_path / "s.svg").read_text().startswith("<svg")


def test_slurm_preflight_node_health_and_cluster_contract(tmp_path, capsys):
    """Node health from injected probes (no GPU needed) and the contract over several nodes' lines."""
    from rpeg_b200.runtime import slurm_preflight as sp
    from rpeg_b200.runtime.errors import RuntimeConfigError

    def torch_probe(n=8, mem=183 * 2 ** 30, cap="10.0", name="NVIDIA B200"):
        return lambda: {"available": n > 0, "count": n, "names": [name] * n, "memory": [mem] * n, "capabilities": [cap] * n,
                        "torch_version": "2.11.0", "cuda_version": "12.8", "nccl_version": "2.28.9"}

    def smi(n=8, driver="580.159"):
        return lambda: {"count": n, "driver": driver}

    good = sp.check_node(8, torch_probe=torch_probe(), smi_probe=smi(), nic_probe=lambda: ["mlx5_0:28.39"], hostname="n0",
                         clock_ns=lambda: 1_000_000_000, min_memory_bytes=150 * 2 ** 30, require_capability="10.0")
    assert good.ok and good.message == "ok" and good.to_dict()["min_total_memory_bytes"] == 183 * 2 ** 30
    few = sp.check_node(8, torch_probe=torch_probe(7), smi_probe=smi(8), nic_probe=list, hostname="n1")
    assert not few.ok and "expected 8" in few.message and "nvidia-smi lists 8" in few.message
    old = sp.check_node(8, torch_probe=torch_probe(cap="9.0"), smi_probe=smi(), nic_probe=list, hostname="n2", require_capability="10.0")
    assert not old.ok and "compute capability 10.0" in old.message
    small = sp.check_node(8, torch_probe=torch_probe(mem=80 * 2 ** 30), smi_probe=smi(), nic_probe=list, min_memory_bytes=150 * 2 ** 30)
    assert not small.ok and "less than" in small.message
    none = sp.check_node(8, torch_probe=torch_probe(0), smi_probe=lambda: {"count": None, "driver": None}, nic_probe=list)
    assert not none.ok and "no CUDA device" in none.message
    # the real probes run anywhere and never raise
    here = sp.check_node(0, nic_probe=lambda: sp.probe_nic_firmware(str(tmp_path / "absent")))
    assert here.hostname and here.torch_version and isinstance(here.to_dict()["wall_time_ns"], int)

    rows = [sp.check_node(8, torch_probe=torch_probe(), smi_probe=smi(), nic_probe=lambda: ["mlx5_0:28.39"], hostname=f"n{i}",
                          clock_ns=lambda i=i: 10 ** 9 + i * 10 ** 8).to_dict() for i in range(3)]
    c = sp.cluster_contract(rows, expected_nodes=3)
    assert c["schema_version"] == "rpeg.cluster_contract.v1" and c["performance_comparable"] and c["nodes"] == 3
    assert c["clock_skew_s"] == pytest.approx(0.2) and c["gpus_per_node"] == [8] and c["min_gpu_memory_bytes"] == 183 * 2 ** 30
    odd = dict(rows[2], driver_version="570.00", wall_time_ns=rows[2]["wall_time_ns"] + 3 * 10 ** 9, nic_firmware=["mlx5_0:20.1"])
    c2 = sp.cluster_contract([rows[0], rows[1], odd, few.to_dict()], expected_nodes=3)
    text = " | ".join(c2["non_comparable_reasons"])
    assert not c2["performance_comparable"]
    for piece in ("driver versions", "NIC firmware", "clock skew", "unhealthy nodes: ['n1']", "reported more than once", "expected 3"):
        assert piece in text, piece
    assert sp.hardware_from_preflight(rows, expected_nodes=3) == ("NVIDIA B200", 183 * 2 ** 30)
    with pytest.raises(RuntimeConfigError, match="2 of 3"):
        sp.hardware_from_preflight(rows[:2], expected_nodes=3)
    assert sp.hardware_from_preflight(None, expected_nodes=1, explicit_memory_bytes=10, explicit_gpu_type="B200") == ("B200", 10)
    with pytest.raises(RuntimeConfigError):
        sp.hardware_from_preflight(None, expected_nodes=1)
    # CLI: contract from a file of lines; --strict turns "not comparable" into exit code 2
    lines = tmp_path / "preflight.jsonl"
    lines.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    from rpeg_b200.runtime.job_plan import job_hardware
    job = {"hardware": {"preset": "b200_nvswitch", "preflight": "preflight.jsonl"}, "device_space": {"racks": 1, "nodes_per_rack": 3, "gpus_per_node": 8}}
    assert job_hardware(job, tmp_path).memory_per_gpu == 183 * 2 ** 30       # the smallest GPU the nodes reported
    job["hardware"]["memory_per_gpu"] = 1e11
    assert job_hardware(job, tmp_path).memory_per_gpu == 1e11                 # an explicit value wins
    assert sp.main(["--contract-from", str(lines), "--contract-output", str(tmp_path / "c.json"), "--expected-nodes", "3", "--strict"]) == 0
    assert json.loads((tmp_path / "c.json").read_text())["performance_comparable"]
    lines.write_text(json.dumps(rows[0]) + "\n" + json.dumps(odd) + "\n")
    assert sp.main(["--contract-from", str(lines), "--strict"]) == 2
    assert sp.main(["--contract-from", str(lines)]) == 0
    lines.write_text("not json\n")
    assert sp.main(["--contract-from", str(lines)]) == 2
    capsys.readouterr()


def test_operator_breakdown_and_strong_scaling_scripts(tmp_path, capsys):
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "experiments"))
    import plot_operator_breakdown as pob
    import plot_strong_scaling as pss
    rep = {"run_id": "demo", "input": {"seconds_by_vertex": {"g_pi": 4.0, "i_ref": 0.5, "t_pi": 2.0}, "seconds_by_kind": {"GEN": 4.0, "INF": 0.5, "TRAIN": 2.0}},
           "output": {"seconds_by_vertex": {"g_pi": 3.0, "i_ref": 0.5, "t_pi": 1.5, "x_new": 0.1}, "seconds_by_kind": {"GEN": 3.0, "INF": 0.5, "TRAIN": 1.5, "comm": 0.2}}}
    a = tmp_path / "a.json"
    a.write_text(json.dumps(rep))
    trace = tmp_path / "run.jsonl"
    trace.write_text("\n".join(json.dumps(e) for e in [
        {"event": "start", "node_id": "g_pi@0"}, {"event": "finish", "node_id": "g_pi@0", "counters": {"duration_s": 3.2}},
        {"event": "finish", "node_id": "g_pi@1", "counters": {"duration_s": 3.3}}, {"event": "finish", "node_id": "t_pi@0", "duration_s": 1.4}]) + "\n")
    groups = pob.breakdown_groups([str(a)], "vertex", str(trace))
    assert [g[0] for g in groups] == ["actor\ngen.", "ref.\ninf.", "actor\ntrain", "x_new"]
    assert groups[0][1] == [("input plan", 4.0), ("optimized plan", 3.0), ("measured", 6.5)]
    assert groups[2][1][2] == ("measured", 1.4)
    assert pob.main([str(a), "--output", str(tmp_path / "b.svg")]) == 0 and "<rect" in (tmp_path / "b.svg").read_text()
    assert pob.main([str(a), str(a), "--by", "kind", "--output", str(tmp_path / "k.svg")]) == 0
    assert len(pob.breakdown_groups([str(a), str(a)], "kind")) == 4
    old = tmp_path / "old.json"
    old.write_text(json.dumps({"input": {}, "output": {}}))
    with pytest.raises(SystemExit):
        pob.breakdown_groups([str(old)])
    # strong scaling: JSON lines mixed with log text, a JSON list, two series
    (tmp_path / "n.log").write_text('warm-up\n{"n_gpus": 1, "value": 6.4, "impl": "ours"}\n{"n_gpus": 8, "value": 19.2, "impl": "ours"}\nnot json {\n')
    (tmp_path / "r.json").write_text(json.dumps([{"n_gpus": 1, "value": 3.0, "impl": "reference"}, {"n_gpus": 8, "value": 12.0, "impl": "reference"},
                                                 {"impl": "reference", "unavailable": "x"}]))
    pts = pss.read_points([str(tmp_path / "n.log"), str(tmp_path / "r.json")], series_key="impl")
    assert pts == {"ours": [(1, 6.4), (8, 19.2)], "reference": [(1, 3.0), (8, 12.0)]}
    rows = pss.scaling_table(pts["ours"])
    assert rows[1]["speedup"] == pytest.approx(3.0) and rows[1]["efficiency"] == pytest.approx(0.375)
    assert pss.scaling_table([(2, 10.0), (4, 6.0)], higher_is_better=False)[1]["efficiency"] == pytest.approx(10 / 6 / 2)
    assert pss.main([str(tmp_path / "n.log"), str(tmp_path / "r.json"), "--series-key", "impl", "--output", str(tmp_path / "s.svg")]) == 0
    assert "ideal" in (tmp_path / "s.svg").read_text()
    (tmp_path / "empty.json").write_text("")
    assert pss.main([str(tmp_path / "empty.json")]) == 2
    capsys.readouterr()


def test_engine_validate_cli_without_a_gpu(capsys):
    """On a machine without a GPU the smoke worker says so and exits 2; its model arguments are validated."""
    import torch

    from rpeg_b200.runtime import engine_validate as ev
    args = ev.build_parser().parse_args(["--layers", "4", "--hidden", "1024", "--ffn", "2816", "--kv-heads", "2"])
    cfg = ev.model_config(args)
    assert (cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff) == (4, 1024, 8, 2, 2816)
    with pytest.raises(SystemExit):
        ev.model_config(ev.build_parser().parse_args(["--hidden", "200"]))
    if not torch.cuda.is_available():
        assert ev.main(["--json"]) == 2
        assert json.loads(capsys.readouterr().out)["error"] == "no CUDA device visible"


def test_published_results_reader_and_charts(tmp_path):
    """The published measurements' layout (``<GPUs>-<model>/metrics_report.json`` in a directory or a tar archive): rows
    per run with both schedules, the speed-up, and one SVG chart per metric; a schedule without numbers stays empty."""
    import importlib.util
    import tarfile
    spec = importlib.util.spec_from_file_location("plot_published_results", os.path.join(ROOT, "experiments", "plot_published_results.py"))
    ppr = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ppr)
    def report(a, b):
        run = lambda t: None if t is None else {"runtime": {"benchmark_wall_time_s": t, "tokens_per_s": 98304 / t,
                                                            "hardware_utilization": {"avg_utilization_pct": 90.0}}}
        return {"schedules": {k: v for k, v in (("pardistrlm", run(a)), ("native", run(b))) if v is not None}}
    src = tmp_path / "athena_results"
    for name, (a, b) in {"8-7": (300.0, 390.0), "16-7": (200.0, 210.0), "16-32": (600.0, None)}.items():
        (src / name).mkdir(parents=True)
        (src / name / "metrics_report.json").write_text(json.dumps(report(a, b)))
    rows = ppr.load(src)
    assert [(r["model_b"], r["gpus"]) for r in rows] == [(7, 8), (7, 16), (32, 16)]
    assert abs(rows[0]["speedup"] - 1.3) < 1e-9 and rows[2]["speedup"] is None and rows[2]["native.iteration_s"] is None
    with tarfile.open(tmp_path / "r.tar.bz2", "w:bz2") as tar:
        tar.add(src, arcname="athena_results")
    assert ppr.load(tmp_path / "r.tar.bz2") == rows
    assert "1.30" in ppr.table(rows)
    written = ppr.charts(rows, tmp_path / "fig")
    assert len(written) == 3 and all(p.read_text().startswith("<svg") for p in written)
    (tmp_path / "nothing_here").mkdir()
    assert ppr.main(["--results", str(tmp_path / "nothing_here")]) == 1


def test_bench_clock_sampler_reads_every_gpu_of_the_job():
    """``bench.py``'s sampler parses ``nvidia-smi`` lines of several GPUs: overall median, per-GPU medians (the slowest GPU
    sets the pace of a multi-GPU step), the union of the throttle reasons; malformed lines are skipped."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class Done:
        def terminate(self):
            pass

    s = bench.ClockSampler([0, 1])
    s.proc = Done()
    s.lines = ["0, 1965, 1965, 800.1, Not Active, Not Active, Not Active, Active",
               "1, 1500, 1965, 900.0, Not Active, Not Active, Not Active, Active",
               "0, 1900, 1965, 810.3, Not Active, Not Active, Not Active, Not Active",
               "1, 1410, 1965, 905.0, Not Active, Not Active, Active, Active",
               "garbage line", "1, [N/A], 1965, x, -, -, -, -"]
    out = s.stop()
    assert out["samples"] == 4 and out["sm_max_mhz"] == 1965.0
    assert out["sm_mhz_per_gpu"] == {"0": 1965.0, "1": 1500.0}
    assert out["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]
    one = bench.ClockSampler(0)
    one.proc, one.lines = Done(), ["0, 1800, 1965, 700, Not Active, Not Active, Not Active, Not Active"]
    assert one.stop() == {"sm_mhz": 1800.0, "sm_max_mhz": 1965.0, "reasons": [], "samples": 1}
