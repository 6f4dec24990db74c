"""CPU tests: candidate directory, move kernels, SA determinism, exhaustive-vs-SA on a micro
instance, plan files and hashes, fused pipeline schedules, the pipeline driver."""
import itertools
import json
import random

import pytest

from rpeg_b200.analytic.cost import NodeCostModel
from rpeg_b200.analytic.memory import MemoryPolicy, NodeMemoryModel
from rpeg_b200.analytic.models import ModelSpec, ModelSuite
from rpeg_b200.analytic.workload import Workload
from rpeg_b200.core.types import Allocation, DeviceSpace, Model, packing_geometry
from rpeg_b200.ir.plan import ExecutionPlan
from rpeg_b200.ir.serialize import (compute_plan_hash, execution_schedule_to_dict, load_optimized_plan, load_plan,
                                    optimized_plan_to_dict, plan_from_dict, plan_to_dict, save_optimized_plan, save_plan)
from rpeg_b200.ir.templates import build_GRPO_RPEG, build_PPO_RPEG
from rpeg_b200.planner.pipeline import Baselines, load_yaml, run_pipeline, validate_config
from rpeg_b200.runtime.fused_pipeline import (FusedPipelineError, FusedPipelineModel, FusedPipelineSchedule, PRIORITY_MODES,
                                              build_fused_pipeline_schedule, validate_fused_pipeline_schedule)
from rpeg_b200.search.cache import EvalCache
from rpeg_b200.search.evaluate import Configuration, evaluate_cached, is_valid
from rpeg_b200.search.moves import (build_candidate_directory, move_gen, multi_move_pair, valid_dp_degrees, valid_mb_counts,
                                    valid_pp_degrees, valid_tp_degrees)
from rpeg_b200.search.optimizer import OptimizerConfig, optimize, polish
from test_planner_core import SPACE, SUITE, WL, example_hw, spread_plan

MICRO = ModelSpec(4, 256, 512, 1000)
MICRO_SUITE = ModelSuite({m: MICRO for m in Model})
MICRO_WL = Workload(16, 1, 32, 64)
MICRO_SPACE = DeviceSpace(1, 1, 2)


def test_degree_rules():
    assert valid_tp_degrees(4) == [1, 2, 4]
    assert valid_pp_degrees(1, 8, 4, 32) == [1, 2, 4, 8, 16, 32]
    assert valid_dp_degrees(1, 2, 12, 2) == [1, 2, 3, 4]
    assert valid_mb_counts(1, 4, 64) == [1]
    assert valid_mb_counts(2, 1, 64) == [2, 4, 8]          # mb | 64, pp <= mb, 64/mb >= 8
    assert valid_mb_counts(4, 16, 64) == []                # 4 prompts per replica is below the minimum of 8


def test_candidate_directory_sorted_and_feasible():
    r = build_PPO_RPEG(SUITE, WL)
    cm = NodeCostModel(example_hw(), SUITE, WL)
    mm = NodeMemoryModel.from_policy(example_hw(), SUITE, WL, MemoryPolicy(), trainable=frozenset(r.trainable))
    d = build_candidate_directory(r, SUITE, SPACE, WL, cm, mm)
    for v in r.vertices:
        rows = d.table[v.id]
        assert rows and [x[6] for x in rows] == sorted(x[6] for x in rows)
        assert all(packing_geometry(x[0], x[1], x[2], SPACE.G) is not None for x in rows)
        assert d.index[v.id][rows[3][:6]] == 3


def _search(seed, **kw):
    r = build_PPO_RPEG(SUITE, WL)
    cfg = Configuration(r, spread_plan(r), SPACE)
    oc = OptimizerConfig(E_max=250, E_struct=120, T_init=0.05, T_min=0.05, T_warm=0.1, stag_window=10, seed=seed, workers=1,
                         T_cand={Model.ACTOR: {0, 1}, Model.CRITIC: {0}, Model.AC_SHARE: set()}, **kw)
    cache, rep = EvalCache(), []
    best = optimize(cfg, SUITE, WL, example_hw(), 3, oc, cache, rep)
    return best, rep[0], cache


def test_search_is_deterministic_under_seed_and_improves():
    a, ra, cache = _search(42)
    b, rb, _ = _search(42)
    assert a.plan.fingerprint() == b.plan.fingerprint() and ra.best_score == rb.best_score
    r = build_PPO_RPEG(SUITE, WL)
    base, _, _, _ = evaluate_cached(Configuration(r, spread_plan(r), SPACE), EvalCache(), SUITE, WL, example_hw(), 3)
    assert ra.best_score > base and ra.best_feasible
    mm = NodeMemoryModel.from_policy(example_hw(), SUITE, WL, MemoryPolicy(), trainable=frozenset(a.rpeg.trainable))
    assert is_valid(a, SUITE, WL, mm)
    c, rc, _ = _search(7)
    assert rc.evaluations <= 250 + 6


def test_ablation_flags_run():
    for kw in (dict(fixed_mb=True), dict(uniform_vertex=True), dict(hard_oom=True), dict(geometric_cooling=True)):
        _, rep, _ = _search(1, **kw)
        assert rep.best_score > 0


def test_sa_reaches_exhaustive_optimum_on_micro_instance():
    hw = example_hw()
    r = build_GRPO_RPEG(MICRO_SUITE, MICRO_WL)
    cm = NodeCostModel(hw, MICRO_SUITE, MICRO_WL)
    mm = NodeMemoryModel.from_policy(hw, MICRO_SUITE, MICRO_WL, MemoryPolicy(), trainable=frozenset(r.trainable))
    d = build_candidate_directory(r, MICRO_SUITE, MICRO_SPACE, MICRO_WL, cm, mm)
    per_vertex = []
    for v in r.vertices:
        opts = []
        for row in d.table[v.id]:
            dp, pp, tp, r_ext, n_ext, mb = row[:6]
            g_ext = packing_geometry(dp, pp, tp, 2)[0]
            for g0 in range(0, 2, g_ext):
                opts.append((v.id, Allocation((0, 0, g0), (r_ext, n_ext, g_ext)), (dp, pp, tp), mb))
        per_vertex.append(opts)
    cache = EvalCache()
    best = 0.0
    for combo in itertools.product(*per_vertex):
        plan = ExecutionPlan()
        for vid, a, pi, mb in combo:
            plan.sigma[vid], plan.pi[vid], plan.mb[vid] = a, pi, mb
        s, _, feas, _ = evaluate_cached(Configuration(r, plan, MICRO_SPACE), cache, MICRO_SUITE, MICRO_WL, hw, 2)
        if feas:
            best = max(best, s)
    start = ExecutionPlan()
    for v in r.vertices:
        start.sigma[v.id], start.pi[v.id], start.mb[v.id] = Allocation((0, 0, 0), (1, 1, 1)), (1, 1, 1), 1
    oc = OptimizerConfig(E_max=400, E_struct=400, seed=3, workers=1, algorithm="grpo", T_cand={Model.ACTOR: {0}})
    rep = []
    found = optimize(Configuration(r, start, MICRO_SPACE), MICRO_SUITE, MICRO_WL, hw, 2, oc, EvalCache(), rep)
    found = polish(found, MICRO_SUITE, MICRO_WL, hw, 2, oc, EvalCache())
    s, _, feas, _ = evaluate_cached(found, EvalCache(), MICRO_SUITE, MICRO_WL, hw, 2)
    assert feas and s >= 0.97 * best


def test_plan_files_round_trip(tmp_path):
    r = build_PPO_RPEG(SUITE, WL)
    cfg = Configuration(r, spread_plan(r), SPACE, intra_stage_fusion=False)
    for name in ("p.yaml", "p.json"):
        path = str(tmp_path / name)
        save_plan(cfg, path, quiet=True)
        back = load_plan(path, r)
        assert back.fingerprint() == cfg.plan.fingerprint()
    _, trace, _, _ = evaluate_cached(cfg, EvalCache(), SUITE, WL, example_hw(), 2)
    sched = execution_schedule_to_dict(trace, horizon=2)
    assert sched["policy"] == "rpeg_critical_path_list_v1" and [n["dispatch_index"] for n in sched["nodes"]] == list(range(len(trace.start)))
    path = str(tmp_path / "opt.yaml")
    d = save_optimized_plan(cfg, path, "ppo", WL, source_config_hash="abc", execution_schedule=sched)
    assert d["schema_version"] == "rpeg.optimized_plan.v1" and d["plan_hash"].startswith("sha256:")
    loaded = load_optimized_plan(path)
    assert loaded["plan_hash"] == d["plan_hash"] == compute_plan_hash(loaded)
    assert plan_from_dict(loaded, r).fingerprint() == cfg.plan.fingerprint()
    loaded["plan"]["g_pi"]["microbatch"] = 2
    with open(path, "w") as f:
        json.dump(loaded, f)
    with pytest.raises(ValueError):
        load_optimized_plan(str(path).replace(".yaml", ".yaml"))


def test_fused_pipeline_schedules():
    a = FusedPipelineModel.uniform("actor", pipeline_stages=4, microbatches=6, forward_s=1.0, backward_s=2.0, activation_bytes=10)
    c = FusedPipelineModel.uniform("critic", pipeline_stages=4, microbatches=6, forward_s=0.5, backward_s=1.0, activation_bytes=7, reverse=True)
    best = build_fused_pipeline_schedule((a, c))
    stage_work = sum(m.microbatches * (m.forward_s[0] + m.backward_s[0]) for m in (a, c))
    assert best.optimizer == "deterministic_blocking_safe_portfolio_v2" and best.optimizer_candidates >= 2
    if best.baseline_makespan_s is not None:          # the greedy rule may fail the rendezvous simulation
        assert best.makespan_s <= best.baseline_makespan_s + 1e-9
    assert best.makespan_s >= stage_work - 1e-9       # a stage cannot finish before its own work is done
    n_valid = 0
    for mode in PRIORITY_MODES:
        try:
            s = build_fused_pipeline_schedule((a, c), optimization=mode)
        except FusedPipelineError:
            continue
        validate_fused_pipeline_schedule(s)
        assert len(s.tasks) == 2 * 2 * 4 * 6
        n_valid += 1
    assert n_valid == best.optimizer_candidates and n_valid >= 2   # the model-serial orders always pass
    assert FusedPipelineSchedule.from_dict(best.to_dict()).schedule_hash == best.schedule_hash
    assert [i["task_id"] for i in best.local_instructions("critic", 3)][0] == "critic:F0:s0"
    with pytest.raises(FusedPipelineError):
        build_fused_pipeline_schedule((a, c), activation_capacity_bytes=5)
    with pytest.raises(FusedPipelineError):
        FusedPipelineModel.uniform("x", pipeline_stages=4, microbatches=2, forward_s=1, backward_s=1, activation_bytes=0)


def test_pipeline_driver_on_example_config(tmp_path):
    cfg = load_yaml("configs/example_ppo_32gpu.yaml")
    assert isinstance(cfg["hardware"]["flops_per_gpu"], float)     # '4.4e14' parsed as a number
    cfg["optimizer"].update(e_max=150, e_struct=80, workers=1)
    cfg["output"] = {"seed": 42, "opt_plan": str(tmp_path / "opt.yaml"), "base_plan": str(tmp_path / "base.yaml")}
    res = run_pipeline(cfg)
    rows = res["rows"]
    assert rows[2]["tokens_per_s"] >= rows[1]["tokens_per_s"] >= 0.9 * rows[0]["tokens_per_s"]
    assert (tmp_path / "opt.yaml").exists() and (tmp_path / "base.yaml").exists()
    bad = dict(cfg, policy={"algorithm": "rlhf"})
    with pytest.raises(ValueError):
        validate_config(bad)
