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


def spread_job(tmp_path, algorithm="ppo", steps=3, ac_share=False, tau=None, width=2, **extra):
    """A plan/run pair with every vertex on its own GPUs (so the graph has COMM and RESHARD nodes),
    built by hand instead of searched."""
    cfg = job_mapping(algorithm, steps, **extra)
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
        g0 = (i * width) % SPACE.G
        plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = Allocation((0, 0, g0), (1, 1, width)), (1, 1, width), 1
    conf = Configuration(rpeg, plan, SPACE, False, TransferResourcePolicy("both_endpoints", "both_endpoints"))
    lowered = lower(rpeg, unroll(rpeg, steps), plan, suite, steps, workload=wl)
    trace = schedule(lowered, NodeCostModel(hw, suite, wl, optimizer_stage=1), SPACE,
                     transfer_resource_policy=conf.transfer_resource_policy)
    d = optimized_plan_to_dict(conf, algorithm, wl, None, execution_schedule_to_dict(trace, horizon=steps))
    dump_mapping(d, tmp_path / "optimized_plan.yaml")
    run = run_config_mapping(cfg, run_id=cfg["run_id"], algorithm=algorithm, workload=wl, space=SPACE, hw=hw,
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


def test_job_planner_emits_a_compilable_pair(tmp_path):
    job = tmp_path / "job.yaml"
    dump_mapping(job_mapping("ppo"), job)
    res = plan_runtime_job(job, tmp_path / "out", emit_launch=True, quiet=True)
    out = res["out_dir"]
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
