"""CPU tests of the runtime layer with the metadata backend: job planning, strict run/plan schema,
compilation, graph resources, asynchronous execution, the trace verifier and host-side failure
injection. Nothing here touches a GPU."""
import json

import pytest

from rpeg_b200.analytic.cost import NodeCostModel
from rpeg_b200.analytic.memory import MemoryPolicy
from rpeg_b200.core.types import Allocation, DeviceSpace, Model, TransferResourcePolicy
from rpeg_b200.ir.plan import ExecutionPlan
from rpeg_b200.ir.serialize import execution_schedule_to_dict, optimized_plan_to_dict
from rpeg_b200.ir.templates import build_rpeg
from rpeg_b200.passes.lower import ExecNodeType, lower
from rpeg_b200.passes.unroll import unroll
from rpeg_b200.runtime.compiler import compile_runtime_plan
from rpeg_b200.runtime.errors import RuntimeConfigError, RuntimeExecutionError
from rpeg_b200.runtime.executor import MetadataOnlyOperationHandler, RuntimeExecutor
from rpeg_b200.runtime.graph import build_runtime_graph
from rpeg_b200.runtime.io import dump_mapping, load_mapping
from rpeg_b200.runtime.job_plan import job_hardware, job_suite, plan_runtime_job, run_config_mapping
from rpeg_b200.runtime.schema import OptimizedPlan, RuntimeRunConfig
from rpeg_b200.runtime.trace import RuntimeTraceWriter, read_trace
from rpeg_b200.runtime.verification import verify_runtime_trace
from rpeg_b200.analytic.workload import Workload
from rpeg_b200.schedule.scheduler import schedule
from rpeg_b200.search.evaluate import Configuration

MODEL = {"layers": 8, "hidden_dim": 1024, "ffn_dim": 2816, "vocab_size": 32000, "head_dim": 128}
SPACE = DeviceSpace(1, 1, 8)


def job_mapping(algorithm="ppo", steps=3, quantiles=True, **extra):
    models = {"actor": dict(MODEL), "reference": {"source": "actor"}}
    if algorithm == "ppo":
        models.update(critic=dict(MODEL), reward=dict(MODEL))
    cfg = {
        "run_id": f"{algorithm}-test", "policy": {"algorithm": algorithm}, "hardware": {"preset": "b200_nvswitch"},
        "device_space": {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 8}, "models": models,
        "workload": {"batch_size": 64, "samples_per_prompt": 2 if algorithm == "grpo" else 1, "context_length": 128,
                     "generation_length": 256, "gen_quantiles": [[0.5, 64], [0.9, 128], [1.0, 256]] if quantiles else None},
        "training": {"max_steps": steps},
        "optimizer": {"k_eval": 2, "k_x": 2, "e_max": 40, "e_struct": 20, "workers": 1},
        "runtime_hardware": {"worker_overhead_bytes": 1 << 30}, "outputs": {"seed": 3},
    }
    cfg.update(extra)
    return cfg


def spread_job(tmp_path, algorithm="ppo", steps=3, ac_share=False, tau=None, width=2, space=SPACE, colocate=False, model=None,
               workload=None, **extra):
    """A plan/run pair with every vertex on its own GPUs (so the graph has COMM and RESHARD nodes),
    built by hand instead of searched."""
    cfg = job_mapping(algorithm, steps, **extra)
    cfg["device_space"] = {"racks": space.R, "nodes_per_rack": space.N, "gpus_per_node": space.G}
    if model is not None:
        for name, m in cfg["models"].items():
            if "layers" in m:
                cfg["models"][name] = dict(model)
    if workload is not None:
        cfg["workload"].update(workload)
    suite, hw = job_suite(cfg), job_hardware(cfg)
    w = cfg["workload"]
    q = w["gen_quantiles"]
    wl = Workload(w["batch_size"], w["samples_per_prompt"], w["context_length"], w["generation_length"],
                  tuple((float(a), int(b)) for a, b in q) if q else None)
    tau_m = None
    if tau is not None:
        tau_m = {Model.ACTOR: tau, Model.CRITIC: 0} if algorithm == "ppo" else {Model.ACTOR: tau}
    rpeg = build_rpeg("ac_share" if ac_share else algorithm, suite, wl, tau=tau_m)
    plan = ExecutionPlan()
    for i, v in enumerate(rpeg.vertices):
        if colocate:        # every vertex data parallel over all GPUs
            plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, 0), (1, 1, space.G)), (space.G, 1, 1), 1
        else:
            g0 = (i * width) % space.G
            plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, g0), (1, 1, width)), (1, 1, width), 1
    conf = Configuration(rpeg, plan, space, False, TransferResourcePolicy("both_endpoints", "both_endpoints"))
    lowered = lower(rpeg, unroll(rpeg, steps), plan, suite, steps, workload=wl)
    trace = schedule(lowered, NodeCostModel(hw, suite, wl, optimizer_stage=1), space,
                     transfer_resource_policy=conf.transfer_resource_policy)
    d = optimized_plan_to_dict(conf, algorithm, wl, None, execution_schedule_to_dict(trace, horizon=steps))
    dump_mapping(d, tmp_path / "optimized_plan.yaml")
    run = run_config_mapping(cfg, run_id=cfg["run_id"], algorithm=algorithm, workload=wl, space=space, hw=hw,
                             policy=MemoryPolicy(1, True, 0.10, float(1 << 30)), plan_file="optimized_plan.yaml",
                             plan_hash=d["plan_hash"], fusion=False)
    dump_mapping(run, tmp_path / "run.yaml")
    return tmp_path / "run.yaml"


def execute(compiled, tmp_path, handler=None, name="trace.jsonl", **kw):
    graph = compiled.runtime_graph()
    tw = RuntimeTraceWriter(tmp_path / name, run_id=compiled.run_config.run_id)
    ex = RuntimeExecutor(graph, run_id=compiled.run_config.run_id, handler=handler or MetadataOnlyOperationHandler(compiled),
                         trace=tw, **kw)
    try:
        ctx = ex.run()
    finally:
        tw.close()
    return graph, ctx, read_trace(tmp_path / name)


def test_engine_jobs_get_the_data_parallel_plan_family(tmp_path):
    """A job for the engine backend on several GPUs is planned as the one family that backend executes:
    every vertex (G, 1, 1) on the whole node; the pair compiles and passes the backend's own plan check."""
    from rpeg_b200.runtime.engine_backend import validate_engine_plan
    cfg = job_mapping("grpo", steps=2, runtime={"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    job = tmp_path / "job.yaml"
    dump_mapping(cfg, job)
    res = plan_runtime_job(job, tmp_path / "out", quiet=True)
    compiled = res["compiled"]
    assert {tuple(pi) for pi in compiled.config.plan.pi.values()} == {(4, 1, 1)}
    assert validate_engine_plan(compiled) == "data_parallel"
    assert res["comparison"]["evaluations"] == 0                      # nothing was searched
    compiled.run_config.algorithm.entropy_coef = 0.01                 # an entropy bonus is part of the PPO / GRPO objective ...
    assert validate_engine_plan(compiled) == "data_parallel"
    compiled.run_config.algorithm.name = "dpo"                        # ... and meaningless for DPO
    with pytest.raises(RuntimeConfigError, match="entropy_coef"):
        validate_engine_plan(compiled)
    compiled.run_config.algorithm.name, compiled.run_config.algorithm.entropy_coef = "grpo", 0.0
    cfg["optimizer"]["plan_family"] = "bogus"
    dump_mapping(cfg, job)
    with pytest.raises(RuntimeConfigError):
        plan_runtime_job(job, tmp_path / "out2", quiet=True)


def test_engine_jobs_can_ask_for_pipeline_parallel_training(tmp_path):
    """``optimizer.plan_family: pipeline_train``: generation / inference vertices stay (G, 1, 1), training vertices become
    (1, G, 1) with at least G microbatches; the pair compiles, the engine backend recognises the family (GRPO only), and
    the graph (now with real layout switches on the publication edges) executes and verifies with the metadata backend."""
    from rpeg_b200.runtime.engine_backend import validate_engine_plan
    cfg = job_mapping("grpo", steps=2, runtime={"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    cfg["optimizer"]["plan_family"] = "pipeline_train"
    job = tmp_path / "job.yaml"
    dump_mapping(cfg, job)
    res = plan_runtime_job(job, tmp_path / "out", quiet=True)
    compiled = res["compiled"]
    pi, mb = compiled.config.plan.pi, compiled.config.plan.mb
    assert tuple(pi["t_pi"]) == (1, 4, 1) and mb["t_pi"] >= 4
    assert {tuple(pi[v]) for v in pi if v != "t_pi"} == {(4, 1, 1)}
    assert validate_engine_plan(compiled) == "pipeline_train"
    assert any(n.kind.value == "reshard" for n in compiled.lowered.nodes)
    graph, ctx, events = execute(compile_runtime_plan(res["run_file"]), tmp_path)
    assert verify_runtime_trace(compiled, graph, events)["ok"]
    cfg["optimizer"]["plan_family"] = "engine"                        # the better of the two executable families
    dump_mapping(cfg, job)
    auto = plan_runtime_job(job, tmp_path / "out3", quiet=True)
    fam = validate_engine_plan(auto["compiled"])
    both = {"pipeline_train": res["comparison"]["output"]["makespan_s"]}
    cfg["optimizer"]["plan_family"] = "data_parallel"
    dump_mapping(cfg, job)
    both["data_parallel"] = plan_runtime_job(job, tmp_path / "out4", quiet=True)["comparison"]["output"]["makespan_s"]
    assert fam == min(both, key=both.get) and auto["comparison"]["output"]["makespan_s"] == pytest.approx(min(both.values()))
    ppo = job_mapping("ppo", steps=1, runtime={"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024})
    ppo["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    ppo["optimizer"]["plan_family"] = "pipeline_train"
    dump_mapping(ppo, job)
    with pytest.raises(RuntimeConfigError, match="GRPO only"):
        plan_runtime_job(job, tmp_path / "out2", quiet=True)
    compiled.run_config.algorithm.name = "ppo"                        # the backend checks the same on its side
    with pytest.raises(RuntimeConfigError, match="GRPO only"):
        validate_engine_plan(compiled)
    compiled.run_config.algorithm.name = "grpo"


def test_engine_jobs_can_ask_for_tensor_parallel_generation(tmp_path):
    """``optimizer.plan_family: tp_generation``: the generation vertex ``(1, 1, G)``, everything else ``(G, 1, 1)``. The pair
    compiles, the publication edge from the data-parallel training vertex becomes a RESHARD node (the layout switch the
    engine backend executes), the backend recognises the family and the graph verifies with the metadata backend."""
    from rpeg_b200.runtime.engine_backend import validate_engine_plan
    cfg = job_mapping("grpo", steps=2, runtime={"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    cfg["optimizer"].update(plan_family="tp_generation")
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    compiled = res["compiled"]
    assert validate_engine_plan(compiled) == "tp_generation"
    assert tuple(compiled.config.plan.pi["g_pi"]) == (1, 1, 4) and tuple(compiled.config.plan.pi["t_pi"]) == (4, 1, 1)
    assert any(n.kind is ExecNodeType.RESHARD for n in compiled.lowered.nodes)
    graph, ctx, events = execute(compile_runtime_plan(res["run_file"]), tmp_path)
    assert verify_runtime_trace(compiled, graph, events)["ok"]
    compiled.run_config.algorithm.name = "ppo"
    with pytest.raises(RuntimeConfigError, match="GRPO only"):
        validate_engine_plan(compiled)
    compiled.run_config.algorithm.name = "grpo"
    ppo = job_mapping("ppo", steps=2, runtime={"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024})
    ppo["device_space"] = cfg["device_space"]
    ppo["optimizer"].update(plan_family="tp_generation")
    dump_mapping(ppo, tmp_path / "job2.yaml")
    with pytest.raises(RuntimeConfigError, match="GRPO only"):
        plan_runtime_job(tmp_path / "job2.yaml", tmp_path / "out2", quiet=True)


def test_tensor_parallel_generation_in_groups_of_ranks(tmp_path):
    """``optimizer.generation_tp: t``: the generation vertex ``(G / t, 1, t)`` (groups of t GPUs decode the rows of their own
    prompts); ``auto`` lets the cost model choose among the divisors of G; anything else is refused."""
    from rpeg_b200.runtime.engine_backend import validate_engine_plan
    cfg = job_mapping("grpo", steps=2, runtime={"default_backend": "engine", "gen_slots": 16, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    cfg["optimizer"].update(plan_family="tp_generation", generation_tp=2)
    dump_mapping(cfg, tmp_path / "job.yaml")
    res = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)
    compiled = res["compiled"]
    assert tuple(compiled.config.plan.pi["g_pi"]) == (2, 1, 2) and tuple(compiled.config.plan.pi["t_pi"]) == (4, 1, 1)
    assert validate_engine_plan(compiled) == "tp_generation"
    assert any(n.kind is ExecNodeType.RESHARD for n in compiled.lowered.nodes)
    graph, ctx, events = execute(compile_runtime_plan(res["run_file"]), tmp_path)
    assert verify_runtime_trace(compiled, graph, events)["ok"]
    cfg["optimizer"]["generation_tp"] = "auto"
    dump_mapping(cfg, tmp_path / "job.yaml")
    auto = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out2", quiet=True)["compiled"]
    dp, pp, tp = auto.config.plan.pi["g_pi"]
    assert pp == 1 and tp in (2, 4) and dp * tp == 4 and validate_engine_plan(auto) == "tp_generation"
    cfg["optimizer"]["generation_tp"] = 3
    dump_mapping(cfg, tmp_path / "job.yaml")
    with pytest.raises(RuntimeConfigError, match="divisor"):
        plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out3", quiet=True)


def test_engine_family_chooses_the_generation_layout_of_the_flagship_job(tmp_path):
    """``plan_family: engine`` on the flagship GRPO job (Llama-7B, 32 prompts x 8 samples, lengths by quantiles) with the
    measured hardware file: at 2 GPUs tensor-parallel and data-parallel generation are predicted within 2 % of each other
    (either may win), at 8 GPUs generation runs tensor parallel in groups (the decode step's per-row work and all-reduce
    launches grow with the rows a group decodes, the weight stream with the GPUs that share it); everything else is data
    parallel."""
    from rpeg_b200.analytic.predict import bench_job_mapping
    spec = dict(algo="grpo", model="llama7b", prompts=32, k=8, prompt_len=512, max_new=2048,
                quantiles=((0.5, 512), (0.9, 1024), (1.0, 2048)))
    chosen = {}
    for n in (2, 8):
        cfg = bench_job_mapping(spec, n, recompute_fraction=0.0)
        cfg["optimizer"]["plan_family"] = "engine"
        cfg["training"] = {"max_steps": 1}
        dump_mapping(cfg, tmp_path / f"job{n}.yaml")
        res = plan_runtime_job(tmp_path / f"job{n}.yaml", tmp_path / f"out{n}", quiet=True)
        pi = res["compiled"].config.plan.pi
        chosen[n] = tuple(pi["g_pi"])
        assert tuple(pi["t_pi"]) == (n, 1, 1) and tuple(pi["i_ref"]) == (n, 1, 1)
    assert chosen[2] in ((1, 1, 2), (2, 1, 1))
    assert chosen[8][1] == 1 and chosen[8][2] >= 2 and chosen[8][0] * chosen[8][2] == 8


@pytest.mark.parametrize("tau", [0, 1])
def test_engine_jobs_can_put_generation_and_training_on_disjoint_gpus(tmp_path, tau):
    """``optimizer.plan_family: disaggregated``: generation data parallel on ``gen_gpus`` GPUs, the rest on the others; with
    ``policy.tau`` the graph carries stale weight versions. The pair compiles, the engine backend recognises the family and
    its rank split, and the graph executes and verifies with the metadata backend."""
    from rpeg_b200.runtime.engine_backend import disaggregated_ranks, validate_engine_plan
    cfg = job_mapping("grpo", steps=3, runtime={"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    cfg["optimizer"].update(plan_family="disaggregated")          # default: half of the GPUs generate
    if tau:
        cfg["policy"]["tau"] = {"actor": tau}
    job = tmp_path / "job.yaml"
    dump_mapping(cfg, job)
    res = plan_runtime_job(job, tmp_path / "out", quiet=True)
    compiled = res["compiled"]
    assert disaggregated_ranks(compiled) == ([0, 1], [2, 3])
    assert validate_engine_plan(compiled) == "disaggregated"
    assert tuple(compiled.config.plan.pi["g_pi"]) == (2, 1, 1) and tuple(compiled.config.plan.pi["t_pi"]) == (2, 1, 1)
    graph, ctx, events = execute(compile_runtime_plan(res["run_file"]), tmp_path)
    assert verify_runtime_trace(compiled, graph, events)["ok"]
    compiled.run_config.algorithm.name = "ppo"
    with pytest.raises(RuntimeConfigError, match="GRPO only"):
        validate_engine_plan(compiled)
    compiled.run_config.algorithm.name = "grpo"
    if tau:                                   # the same staleness on shared GPUs is refused by the planner: nothing could overlap
        cfg["optimizer"].update(plan_family="data_parallel")
        dump_mapping(cfg, job)
        with pytest.raises(RuntimeConfigError):
            plan_runtime_job(job, tmp_path / "out2", quiet=True)
    bad = dict(cfg, optimizer=dict(cfg["optimizer"], plan_family="disaggregated", gen_gpus=4))
    dump_mapping(bad, job)
    with pytest.raises(RuntimeConfigError, match="gen_gpus"):
        plan_runtime_job(job, tmp_path / "out3", quiet=True)


def test_job_planner_emits_a_compilable_pair(tmp_path):
    job = tmp_path / "job.yaml"
    dump_mapping(job_mapping("ppo"), job)
    res = plan_runtime_job(job, tmp_path / "out", emit_launch=True, emit_sbatch=True, quiet=True)
    out = res["out_dir"]
    sb = (out / "submit.sbatch").read_text()
    assert "#SBATCH --nodes=1" in sb and "#SBATCH --gpus-per-node=8" in sb and "srun" in sb and "rpeg_b200.runtime.run" in sb
    assert sb.index("slurm_preflight --expected-gpus 8") < sb.index("--contract-from") < sb.index("rpeg_b200.runtime.run")
    assert (out / "metrics/analytical_comparison.json").exists()
    for f in ("baseline_plan.yaml", "optimized_plan.yaml", "run.yaml", "plots/optimizer_input.gantt.svg",
              "plots/optimizer_output.gantt.svg", "metrics/analytical_comparison.json", "submit.sh"):
        assert (out / f).exists(), f
    cmp_ = json.loads((out / "metrics/analytical_comparison.json").read_text())
    assert cmp_["schema_version"] == "rpeg.analytical_comparison.v1"
    assert cmp_["output"]["makespan_s"] <= cmp_["input"]["makespan_s"] * (1 + 1e-9)
    assert "127.0.0.1" in (out / "submit.sh").read_text()
    compiled = compile_runtime_plan(out / "run.yaml")
    assert compiled.optimized_plan.plan_hash == res["plan_hash"] and compiled.execution_order is not None
    graph, ctx, events = execute(compiled, tmp_path)
    assert verify_runtime_trace(compiled, graph, events)["ok"]


@pytest.mark.parametrize("algorithm,ac_share,tau", [("ppo", False, None), ("ppo", False, 1), ("grpo", False, None),
                                                     ("dpo", False, None), ("ppo", True, None)])
def test_metadata_execution_of_spread_plans(tmp_path, algorithm, ac_share, tau):
    width = 1 if algorithm == "ppo" else 2        # six PPO vertices on eight GPUs must not wrap onto one another
    run = spread_job(tmp_path, algorithm, ac_share=ac_share, tau=tau, width=width)
    compiled = compile_runtime_plan(run)
    graph, ctx, events = execute(compiled, tmp_path)
    kinds = {n.kind for n in graph.nodes.values()}
    assert ExecNodeType.OP in kinds and (ExecNodeType.COMM in kinds or ExecNodeType.RESHARD in kinds)
    report = verify_runtime_trace(compiled, graph, events)
    assert report["ok"] and report["verified_nodes"] == len(graph.nodes)
    # operators hold their worker and their GPUs; no two overlapping nodes shared a key
    op = next(n for n in graph.nodes.values() if n.kind is ExecNodeType.OP)
    assert any(k.startswith("worker:") for k in op.resource_keys) and sum(k.startswith("gpu:") for k in op.resource_keys) == width
    if algorithm != "dpo":
        split = [n for n in graph.nodes.values() if n.exec_node.n_seqs is not None]
        assert split, "generation was not split by the length quantiles"
    if tau:
        gen = [e for e in events if e["event"] == "finish" and e["node_id"].startswith("g_pi@") and "weight_version" in e["counters"]]
        assert {(e["step"], e["counters"]["weight_version"]) for e in gen} == {(1, 0), (2, 0), (3, 1)}
        assert all(e["counters"]["shadow"] for e in gen)


def test_schema_rejections(tmp_path):
    run = spread_job(tmp_path, "grpo")
    raw = load_mapping(run)
    with pytest.raises(RuntimeConfigError, match="schema_version"):
        RuntimeRunConfig.from_mapping({**raw, "schema_version": "rpeg.run.v0"})
    with pytest.raises(RuntimeConfigError, match="unknown top-level"):
        RuntimeRunConfig.from_mapping({**raw, "surprise": 1})
    with pytest.raises(RuntimeConfigError):
        RuntimeRunConfig.from_mapping({**raw, "runtime": {**raw["runtime"], "no_such_knob": True}})
    bad = {**raw, "workload": {**raw["workload"], "batch_size": 32}}
    dump_mapping(bad, tmp_path / "bad_run.yaml")
    with pytest.raises(RuntimeConfigError, match="batch_size"):
        compile_runtime_plan(tmp_path / "bad_run.yaml")
    bad = {**raw, "training": {**raw["training"], "max_steps": 2}}
    dump_mapping(bad, tmp_path / "bad_run2.yaml")
    with pytest.raises(RuntimeConfigError, match="horizon"):
        compile_runtime_plan(tmp_path / "bad_run2.yaml")
    # an edited plan no longer matches its hash
    plan = load_mapping(tmp_path / "optimized_plan.yaml")
    first = next(iter(plan["plan"]))
    plan["plan"][first]["microbatch"] = 2
    with pytest.raises(RuntimeConfigError, match="hash"):
        OptimizedPlan.from_mapping(plan)


def test_host_side_failure_injection_and_verifier(tmp_path):
    compiled = compile_runtime_plan(spread_job(tmp_path, "grpo", steps=2))
    with pytest.raises(RuntimeExecutionError, match="injected failure"):
        execute(compiled, tmp_path, MetadataOnlyOperationHandler(compiled, fail_on={"t_pi@1": 1}), name="fail.jsonl")
    events = read_trace(tmp_path / "fail.jsonl")
    errs = [e for e in events if e["event"] == "finish" and e["status"] == "error"]
    assert len(errs) == 1 and "t_pi@1" in errs[0]["node_id"] and "injected" in errs[0]["message"]
    graph, _, good = execute(compiled, tmp_path, name="good.jsonl")
    report = verify_runtime_trace(compiled, graph, events, raise_on_error=False)
    assert not report["ok"] and any("no successful start/finish" in m for m in report["errors"])
    # tampering: a consumer that started before its producer finished, and a wrong weight version
    t_min = min(e["timestamp"] for e in good)
    moved = [dict(e) for e in good]
    victim = next(n for n in graph.topological_order if graph.nodes[n].dependencies)
    for e in moved:
        if e["node_id"] == victim and e["event"] == "start":
            e["timestamp"] = t_min - 1.0
    with pytest.raises(RuntimeExecutionError, match="dependency"):
        verify_runtime_trace(compiled, graph, moved)
    wrong = [json.loads(json.dumps(e)) for e in good]
    for e in wrong:
        if e["event"] == "finish" and "weight_version" in (e.get("counters") or {}):
            e["counters"]["weight_version"] += 5
            break
    with pytest.raises(RuntimeExecutionError, match="weight version"):
        verify_runtime_trace(compiled, graph, wrong)


def test_executor_respects_resources_and_timeouts(tmp_path):
    compiled = compile_runtime_plan(spread_job(tmp_path, "ppo", steps=2))
    graph, ctx, events = execute(compiled, tmp_path, max_concurrency=2)
    assert len(ctx.completed) == len(graph.nodes)
    running, peak = set(), 0
    for e in events:
        if e["event"] == "start":
            running.add(e["node_id"])
            peak = max(peak, len(running))
        elif e["event"] == "finish":
            running.discard(e["node_id"])
    assert peak <= 2

    class Stuck(MetadataOnlyOperationHandler):
        async def execute(self, node, context):
            import asyncio
            await asyncio.sleep(5)

    with pytest.raises(RuntimeExecutionError, match="timeout"):
        execute(compiled, tmp_path, Stuck(compiled), name="stuck.jsonl", node_timeout_s=0.05)


# ---------------------------------------------------------------------------------- run CLI, replay, metrics
def test_run_cli_modes_and_exit_codes(tmp_path, capsys):
    from rpeg_b200.runtime.run import main as run_main
    run = spread_job(tmp_path, "grpo", steps=2)
    assert run_main(["--config", str(run), "--dry-run"]) == 0
    summary = json.loads(capsys.readouterr().out)
    assert summary["algorithm"] == "grpo" and summary["runtime_graph"]["node_count"] > 0 and summary["workers"]
    assert run_main(["--config", str(run), "--execute-graph-metadata"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["verification"]["ok"] and out["alerts"] == "ok" and out["summary"]["logical_steps"] == 2
    for f in ("metrics/summary.json", "metrics/metrics.prom", "metrics/alerts.json", "metrics/dashboard.html", "traces/run.jsonl"):
        assert (tmp_path / f).exists(), f
    prom = (tmp_path / "metrics/metrics.prom").read_text()
    assert 'rpeg_runtime_nodes_finished{run_id="grpo-test"}' in prom
    bad = load_mapping(run)
    bad["device_space"]["gpus_per_node"] = 4
    dump_mapping(bad, tmp_path / "bad.yaml")
    assert run_main(["--config", str(tmp_path / "bad.yaml"), "--dry-run"]) == 2
    assert "runtime error:" in capsys.readouterr().err
    from rpeg_b200.runtime.plot_trace import main as plot_main
    assert plot_main(["--trace", str(tmp_path / "traces/run.jsonl"), "--config", str(run), "--output", str(tmp_path / "g.svg")]) == 0
    assert (tmp_path / "g.svg").read_text().startswith("<svg")


def test_replay_restores_the_interval_checkpoint_and_runs_the_suffix(tmp_path):
    from rpeg_b200.runtime import checkpoint as ckpt
    from rpeg_b200.runtime.run import execute_compiled
    run = spread_job(tmp_path, "grpo", steps=4, checkpoints={"interval_steps": 2},
                     monitoring={"graph_replay_retries": 1, "test_inject_failure_after_checkpoint_step": 2,
                                 "test_inject_failure_attempt": 0})
    compiled = compile_runtime_plan(run)
    res = execute_compiled(compiled, "metadata")
    assert res["error"] is None and res["attempts"] == 2
    rep = res["verification"]
    assert rep["ok"] and rep["replay_attempts"] == 1 and rep["recoveries"] == 1 and rep["restored_steps"] == [2]
    events = read_trace(tmp_path / "traces/run.jsonl")
    rec = next(e for e in events if e["event"] == "recover")
    assert rec["counters"]["restored_step"] == 2 and rec["counters"]["weight_versions"] == {"actor": 2}
    # steps 1-2 ran once, steps 3-4 only in the second attempt; versions continue at 3
    t_pi = [(e["step"], e["counters"]["produced_weight"]["version"]) for e in events
            if e["event"] == "finish" and e["node_id"].startswith("t_pi@") and e["status"] == "ok"]
    assert t_pi == [(1, 1), (2, 2), (3, 3), (4, 4)]
    idx = ckpt.load_index(tmp_path / "checkpoints")
    assert idx["latest_interval"] == str(tmp_path / "checkpoints/step_2") and idx["latest_final"] == str(tmp_path / "checkpoints/final")
    assert ckpt.read_weight_versions(tmp_path / "checkpoints/final")["latest"] == {"actor": 4}
    alerts = json.loads((tmp_path / "metrics/alerts.json").read_text())
    assert alerts["schema_version"] == "rpeg.runtime_alerts.v1" and alerts["status"] == "critical"
    assert any(a["rule"] == "max_replay_attempts" for a in alerts["alerts"])
    # without retries the same injection is fatal
    run2 = spread_job(tmp_path / "b", "grpo", steps=4, checkpoints={"interval_steps": 2},
                      monitoring={"test_inject_failure_after_checkpoint_step": 2}) if (tmp_path / "b").mkdir() is None else None
    res2 = execute_compiled(compile_runtime_plan(run2), "metadata")
    assert res2["error"] and "injected failure" in res2["error"] and not res2["verification"]["ok"]


def test_resume_from_checkpoint_runs_only_the_suffix(tmp_path):
    from rpeg_b200.runtime.run import execute_compiled
    (tmp_path / "a").mkdir()
    first = spread_job(tmp_path / "a", "dpo", steps=2, checkpoints={"interval_steps": 1})
    assert execute_compiled(compile_runtime_plan(first), "metadata")["error"] is None
    (tmp_path / "b").mkdir()
    second = spread_job(tmp_path / "b", "dpo", steps=2, checkpoints={"interval_steps": 1, "resume_from": str(tmp_path / "a/checkpoints")})
    # the newest usable checkpoint of the first run is its final one (step 2): nothing is left to run but lifecycle nodes
    res = execute_compiled(compile_runtime_plan(second), "metadata")
    assert res["error"] is None and res["verification"]["ok"] and res["summary"]["nodes_finished"] == 0


def test_checkpoint_flat_shards_reslice_across_dp_degrees(tmp_path):
    import torch
    from rpeg_b200.runtime import checkpoint as ckpt
    full = torch.arange(1000, dtype=torch.float32)
    w = torch.randn(7, 9).bfloat16()
    for r in range(4):                                       # written by 4 ranks, 250 elements each
        ckpt.save_flat_shards(tmp_path / "step_1/actor", r, 4, {"adam.m": full[r * 250:(r + 1) * 250], **({"weights": w} if r == 0 else {})},
                              ranges={"adam.m": (r * 250, (r + 1) * 250, 1000)})
    ckpt.finalize_worker_meta(tmp_path / "step_1/actor", 4)
    ckpt.write_weight_versions(tmp_path / "step_1", step=1, latest={"actor": 1}, retained={"actor": [0, 1]}, tau={"actor": 1})
    ckpt.register_checkpoint(tmp_path, name="step_1", kind="interval", step=1, workers=["actor"])
    assert ckpt.verify_checkpoint(tmp_path / "step_1", ["actor"])["errors"] == []
    for lo, hi in ((0, 334), (334, 667), (667, 1000)):       # read back by 3 ranks
        assert torch.equal(ckpt.load_flat_range(tmp_path / "step_1/actor", "adam.m", lo, hi), full[lo:hi])
    assert torch.equal(ckpt.load_tensor(tmp_path / "step_1/actor", "weights"), w)
    assert ckpt.versions_needed_after(5, 2) == [3, 4, 5]
    # a truncated shard makes the checkpoint unusable
    f = tmp_path / "step_1/actor/rank2.bin"
    f.write_bytes(f.read_bytes()[:-8])
    assert ckpt.latest_usable_checkpoint(tmp_path) is None


def _tiny_checkpoint(root, name, step, kind="interval", payload=None):
    import torch
    from rpeg_b200.runtime import checkpoint as ckpt
    t = payload if payload is not None else torch.arange(64, dtype=torch.float32) + step
    ckpt.save_flat_shards(root / name / "actor", 0, 1, {"adam.m": t}, ranges={"adam.m": (0, 64, 64)})
    ckpt.finalize_worker_meta(root / name / "actor", 1)
    ckpt.write_weight_versions(root / name, step=step, latest={"actor": step}, retained={"actor": [step]}, tau={"actor": 0})
    return ckpt.register_checkpoint(root, name=name, kind=kind, step=step, workers=["actor"])


def test_interval_checkpoints_are_pruned_by_count_like_the_reference(tmp_path):
    """``keep_last_interval_steps`` is the NUMBER of interval checkpoints kept (0 removes all of them), final checkpoints
    stay, and the index holds paths under the output directory with ``latest_interval`` recomputed after pruning."""
    from rpeg_b200.runtime import checkpoint as ckpt
    for step in (100, 200, 300, 400):
        _tiny_checkpoint(tmp_path, f"step_{step}", step)
    _tiny_checkpoint(tmp_path, "final", 400, kind="final")
    assert ckpt.prune_checkpoints(tmp_path, None) == []
    assert ckpt.prune_checkpoints(tmp_path, 2) == ["step_100", "step_200"]
    idx = ckpt.load_index(tmp_path)
    assert [c["name"] for c in idx["checkpoints"]] == ["step_300", "step_400", "final"]
    assert idx["latest_interval"] == str(tmp_path / "step_400") and idx["latest_final"] == str(tmp_path / "final")
    assert not (tmp_path / "step_100").exists() and (tmp_path / "step_300").is_dir()
    assert all(c["path"] == str(tmp_path / c["name"]) for c in idx["checkpoints"])
    assert ckpt.prune_checkpoints(tmp_path, 0) == ["step_300", "step_400"]
    idx = ckpt.load_index(tmp_path)
    assert idx["latest_interval"] is None and [c["name"] for c in idx["checkpoints"]] == ["final"]
    assert ckpt.latest_usable_checkpoint(tmp_path)["name"] == "final"


def test_checkpoint_selection_rejects_empty_and_silently_damaged_entries(tmp_path):
    """An entry without worker directories is not something to restore from unless it declares itself metadata only; a
    rank file of the right size with changed bytes is caught by its sha256; overlapping shards are refused on load."""
    import torch
    from rpeg_b200.runtime import checkpoint as ckpt
    _tiny_checkpoint(tmp_path, "step_1", 1)
    (tmp_path / "step_2").mkdir()
    ckpt.write_weight_versions(tmp_path / "step_2", step=2, latest={"actor": 2}, retained={"actor": [2]}, tau={"actor": 0})
    ckpt.register_checkpoint(tmp_path, name="step_2", kind="interval", step=2, workers=[])
    assert ckpt.latest_usable_checkpoint(tmp_path)["name"] == "step_1"          # the empty newer entry is skipped
    ckpt.register_checkpoint(tmp_path, name="step_2", kind="interval", step=2, workers=[], extra={"metadata_only": True})
    assert ckpt.latest_usable_checkpoint(tmp_path)["name"] == "step_2"
    ckpt.register_checkpoint(tmp_path, name="step_2", kind="interval", step=2, workers=[])
    f = tmp_path / "step_1/actor/rank0.bin"
    raw = bytearray(f.read_bytes())
    raw[10] ^= 0xFF
    f.write_bytes(bytes(raw))                                                   # same size, different content
    assert ckpt.latest_usable_checkpoint(tmp_path)["name"] == "step_1"          # sizes alone do not see it
    assert ckpt.latest_usable_checkpoint(tmp_path, verify_hashes=True) is None
    assert any("sha256" in e for e in ckpt.verify_checkpoint(tmp_path / "step_1", ["actor"], hashes=True)["errors"])
    # two ranks that both claim elements 40..49
    full = torch.arange(100, dtype=torch.float32)
    ckpt.save_flat_shards(tmp_path / "ov/actor", 0, 2, {"adam.m": full[:50]}, ranges={"adam.m": (0, 50, 100)})
    ckpt.save_flat_shards(tmp_path / "ov/actor", 1, 2, {"adam.m": full[40:100]}, ranges={"adam.m": (40, 100, 100)})
    ckpt.finalize_worker_meta(tmp_path / "ov/actor", 2)
    with pytest.raises(RuntimeExecutionError, match="overlap"):
        ckpt.load_flat_range(tmp_path / "ov/actor", "adam.m", 0, 100)


def test_disaggregated_family_refuses_graph_replay(tmp_path):
    """Generation and training on disjoint GPUs write no tensor checkpoint, so a replay could only re-apply updates on
    top of the advanced state: the engine backend refuses ``graph_replay_retries > 0`` for this family."""
    from rpeg_b200.runtime.engine_backend import validate_engine_plan
    cfg = job_mapping("grpo", steps=3, runtime={"default_backend": "engine", "gen_slots": 8, "micro_tokens": 1024})
    cfg["device_space"] = {"racks": 1, "nodes_per_rack": 1, "gpus_per_node": 4}
    cfg["optimizer"].update(plan_family="disaggregated")
    dump_mapping(cfg, tmp_path / "job.yaml")
    compiled = plan_runtime_job(tmp_path / "job.yaml", tmp_path / "out", quiet=True)["compiled"]
    assert validate_engine_plan(compiled) == "disaggregated"
    compiled.run_config.monitoring.graph_replay_retries = 1
    with pytest.raises(RuntimeConfigError, match="graph_replay_retries"):
        validate_engine_plan(compiled)


def test_metrics_alert_rules_and_fingerprints():
    from rpeg_b200.runtime.metrics import compare_artifact_numeric_fingerprints, evaluate_alerts, prometheus_text, summarize_trace, tensor_fingerprint
    import torch
    ev = [
        {"run_id": "r", "node_id": "g_pi@0", "event": "start", "status": "ok", "timestamp": 10.0, "step": 1,
         "counters": {"kind": "OP", "role": "GEN", "model": "actor", "resources": ["gpu:0:0:0"]}},
        {"run_id": "r", "node_id": "g_pi@0", "event": "finish", "status": "ok", "timestamp": 12.0, "step": 1,
         "counters": {"duration_s": 2.0, "generated_tokens": 4000, "decode_steps": 100, "kv_pages_taken": 10, "kv_pages_returned": 9}},
        {"run_id": "r", "node_id": "t_pi@0", "event": "start", "status": "ok", "timestamp": 12.0, "step": 1,
         "counters": {"kind": "OP", "role": "TRAIN", "model": "actor"}},
        {"run_id": "r", "node_id": "t_pi@0", "event": "finish", "status": "ok", "timestamp": 13.0, "step": 1,
         "counters": {"duration_s": 1.0, "loss": float("nan"), "grad_norm": 2.5, "train_tokens": 8000,
                      "produced_weight": {"model": "actor", "version": 1}}},
    ]
    s = summarize_trace(ev)
    assert s["generation_tokens"] == 4000 and s["generation_tokens_per_s_node"] == 2000.0 and s["wall_time_s"] == 3.0
    assert s["nonfinite_losses"] == 1 and s["latest_grad_norm"] == 2.5 and s["kv_pool_pages_outstanding"] == 1
    a = evaluate_alerts(s, {"min_generation_tokens_per_s_wall": {"value": 5000, "severity": "warning"}})
    rules = {x["rule"]: x["severity"] for x in a["alerts"]}
    assert rules == {"max_nonfinite_losses": "critical", "max_kv_pool_pages_outstanding": "critical",
                     "min_generation_tokens_per_s_wall": "warning"} and a["status"] == "critical"
    assert 'rpeg_runtime_weight_versions_produced{run_id="r",key="actor"} 1' in prometheus_text(s)
    x = torch.randn(100)
    fa, fb = {"logp": tensor_fingerprint(x)}, {"logp": tensor_fingerprint(x + 1e-9)}
    assert compare_artifact_numeric_fingerprints(fa, fb)["ok"]
    assert not compare_artifact_numeric_fingerprints(fa, {"logp": tensor_fingerprint(x + 1e-2)})["ok"]
    ia = {"tok": tensor_fingerprint(torch.arange(10))}
    ib = {"tok": tensor_fingerprint(torch.arange(10) + (torch.arange(10) == 3))}
    assert not compare_artifact_numeric_fingerprints(ia, ib)["ok"]


def test_full_validator_phases(tmp_path, capsys):
    from rpeg_b200.runtime.validate_full import main as validate_main, validate_full
    run = spread_job(tmp_path, "ppo", steps=2, width=1)
    rep = validate_full(run, work_dir=tmp_path / "work")
    assert rep["ok"] and [p["phase"] for p in rep["phases"]] == ["input", "unroll", "lower", "runtime_graph", "metadata_execution"]
    lower_facts = rep["phases"][2]
    assert lower_facts["by_kind"]["op"] > 0 and lower_facts["quantile_split_nodes"] > 0
    bad = load_mapping(run)
    bad["workload"]["context_length"] = 64
    dump_mapping(bad, tmp_path / "bad.yaml")
    assert validate_main(["--config", str(tmp_path / "bad.yaml")]) == 2
    out = json.loads(capsys.readouterr().out)
    assert not out["ok"] and out["phases"][-1]["phase"] == "unroll" and "context_length" in out["phases"][-1]["error"]


def _checkpoint_rank(rank: int, world: int, root: str, port: int) -> None:
    """One gloo rank: saves three interval checkpoints through the hook with a handler that writes a shard per rank."""
    import os
    from pathlib import Path
    from types import SimpleNamespace

    import torch
    import torch.distributed as dist
    from rpeg_b200.runtime import checkpoint as ckpt
    from rpeg_b200.runtime.recovery import CheckpointingHook
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)

    class Handler:
        def save_checkpoint(self, step, path, kind):
            ckpt.save_flat_shards(Path(path) / "actor", rank, world, {"adam.m": torch.full((8,), float(step))},
                                  ranges={"adam.m": (rank * 8, rank * 8 + 8, world * 8)})
            dist.barrier()
            if rank == 0:
                ckpt.finalize_worker_meta(Path(path) / "actor", world)
            dist.barrier()
            return {"workers": ["actor"], "bytes": 32, "files": 1}

    run = SimpleNamespace(checkpoints=SimpleNamespace(output_dir=root, keep_last_interval_steps=2, interval_steps=1, save_final=False),
                          monitoring=SimpleNamespace(), training=SimpleNamespace(max_steps=9), resolve=lambda p: Path(p))
    graph = SimpleNamespace(nodes={})
    hook = CheckpointingHook.__new__(CheckpointingHook)
    hook.inner, hook.graph, hook.run, hook.trace, hook.attempt, hook.latest, hook.saved_steps = Handler(), graph, run, None, 0, {"actor": 0}, []
    for step in (1, 2, 3):
        hook.latest["actor"] = step
        hook.save(step, "interval")
    dist.destroy_process_group()


def test_only_one_rank_registers_and_prunes_checkpoints(tmp_path):
    """Three gloo ranks save through the same hook: every rank writes its shard, the index is written by rank 0 alone
    (one entry per checkpoint, pruning by count) and no rank trips over a directory another one is removing."""
    import torch.multiprocessing as mp
    from rpeg_b200.runtime import checkpoint as ckpt
    mp.spawn(_checkpoint_rank, args=(3, str(tmp_path), 29631), nprocs=3, join=True)
    idx = ckpt.load_index(tmp_path)
    assert [c["name"] for c in idx["checkpoints"]] == ["step_2", "step_3"] and not (tmp_path / "step_1").exists()
    entry = ckpt.latest_usable_checkpoint(tmp_path, verify_hashes=True)
    assert entry["name"] == "step_3" and entry["workers"] == ["actor"]
    assert ckpt.load_flat_range(tmp_path / "step_3/actor", "adam.m", 0, 24).tolist() == [3.0] * 24
