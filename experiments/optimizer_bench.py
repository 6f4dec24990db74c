"""How close does the annealing search get to the true optimum?

    python experiments/optimizer_bench.py [--instances micro2,micro4] [--seeds 10] [--evals 400] [--output bench.json]

On instances small enough to enumerate (a few GPUs, small models) every combination of per-vertex
candidates and placements is evaluated, which gives the global optimum of the same objective the
search maximises. The search then runs from the trivial start plan with N seeds; the report lists,
per instance, the size of the space, the optimum, the mean and worst optimality gap, how often the
optimum was hit (within 0.1 %), evaluations and wall time per run, and the share of the space a run
visits. Counterpart of the reference's experiments/optimizer_bench.py:338-632.
"""
from __future__ import annotations

import argparse
import itertools
import json
import statistics
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from rpeg_b200.analytic.cost import NodeCostModel  # noqa: E402
from rpeg_b200.analytic.hardware import b200_nvswitch  # noqa: E402
from rpeg_b200.analytic.memory import MemoryPolicy, NodeMemoryModel  # noqa: E402
from rpeg_b200.analytic.models import ModelSpec, ModelSuite  # noqa: E402
from rpeg_b200.analytic.workload import Workload  # noqa: E402
from rpeg_b200.core.types import Allocation, DeviceSpace, Model, packing_geometry  # noqa: E402
from rpeg_b200.ir.plan import ExecutionPlan  # noqa: E402
from rpeg_b200.ir.templates import build_rpeg  # noqa: E402
from rpeg_b200.search.cache import EvalCache  # noqa: E402
from rpeg_b200.search.evaluate import Configuration, evaluate_cached  # noqa: E402
from rpeg_b200.search.moves import build_candidate_directory  # noqa: E402
from rpeg_b200.search.optimizer import OptimizerConfig, optimize, polish  # noqa: E402

INSTANCES = {
    # name: (algorithm, GPUs in one node, model (L, d, d_ff, V), workload (B, K, S, T), K_eval)
    "micro2": ("grpo", 2, (4, 256, 512, 1000), (16, 1, 32, 64), 2),
    "micro4": ("grpo", 4, (8, 512, 1024, 4000), (32, 1, 32, 128), 2),
    "dpo4": ("dpo", 4, (8, 512, 1024, 4000), (32, 1, 64, 64), 2),
    "ppo2": ("ppo", 2, (4, 256, 512, 1000), (16, 1, 32, 64), 2),
}


def enumerate_space(rpeg, suite, space, wl, hw, k_eval, policy):
    cm = NodeCostModel(hw, suite, wl, optimizer_stage=policy.optimizer_stage, activation_checkpointing=policy.activation_checkpointing)
    mm = NodeMemoryModel.from_policy(hw, suite, wl, policy, trainable=frozenset(rpeg.trainable))
    d = build_candidate_directory(rpeg, suite, space, wl, cm, mm)
    per_vertex = []
    for v in rpeg.vertices:
        opts = []
        for row in d.table[v.id]:
            dp, pp, tp, r_ext, n_ext, mb = row[:6]
            g_ext = packing_geometry(dp, pp, tp, space.G)[0]
            for g0 in range(0, space.G - g_ext + 1, g_ext):
                opts.append((v.id, Allocation((0, 0, g0), (r_ext, n_ext, g_ext)), (dp, pp, tp), mb))
        per_vertex.append(opts)
    size = 1
    for o in per_vertex:
        size *= len(o)
    cache = EvalCache()
    best, feasible = 0.0, 0
    for combo in itertools.product(*per_vertex):
        plan = ExecutionPlan()
        for vid, a, pi, mb in combo:
            plan.sigma[vid], plan.pi[vid], plan.mb[vid] = a, pi, mb
        s, _, ok, _ = evaluate_cached(Configuration(rpeg, plan, space), cache, suite, wl, hw, k_eval, policy)
        if ok:
            feasible += 1
            best = max(best, s)
    return size, feasible, best


def bench_instance(name: str, seeds: int, evals: int) -> dict:
    algo, gpus, (L, d, f, V), (B, K, S, T), k_eval = INSTANCES[name]
    suite = ModelSuite({m: ModelSpec(L, d, f, V) for m in Model})
    wl, space, hw, policy = Workload(B, K, S, T), DeviceSpace(1, 1, gpus), b200_nvswitch(), MemoryPolicy()
    tau = {Model.ACTOR: 0, Model.CRITIC: 0} if algo == "ppo" else {Model.ACTOR: 0}
    rpeg = build_rpeg(algo, suite, wl, tau=tau)
    t0 = time.perf_counter()
    size, feasible, optimum = enumerate_space(rpeg, suite, space, wl, hw, k_eval, policy)
    t_enum = time.perf_counter() - t0
    start = ExecutionPlan()
    for v in rpeg.vertices:
        start.sigma[v.id], start.pi[v.id], start.mb[v.id] = Allocation((0, 0, 0), (1, 1, 1)), (1, 1, 1), 1
    gaps, hits, used, walls = [], 0, [], []
    for seed in range(1, seeds + 1):
        t_cand = {m: {0} for m in tau}
        if algo == "ppo":
            t_cand[Model.AC_SHARE] = set()
        oc = OptimizerConfig(E_max=evals, E_struct=evals, seed=seed, workers=1, algorithm=algo, T_cand=t_cand,
                             structural_candidates=frozenset({"separate"}) if algo == "ppo" else None)
        cache, rep = EvalCache(), []
        t1 = time.perf_counter()
        found = optimize(Configuration(rpeg, start, space), suite, wl, hw, k_eval, oc, cache, rep)
        found = polish(found, suite, wl, hw, k_eval, oc, cache)
        walls.append(time.perf_counter() - t1)
        s, _, ok, _ = evaluate_cached(found, EvalCache(), suite, wl, hw, k_eval, policy)
        gap = 1.0 - (s / optimum if (ok and optimum > 0) else 0.0)
        gaps.append(gap)
        hits += gap <= 1e-3
        used.append(cache.stats()["misses"])
    return {"instance": name, "algorithm": algo, "gpus": gpus, "space_size": size, "feasible_plans": feasible, "optimum_tokens_per_s": optimum,
            "enumeration_s": t_enum, "seeds": seeds, "budget_evals": evals, "mean_gap": statistics.mean(gaps), "worst_gap": max(gaps),
            "hit_rate": hits / seeds, "mean_evaluations": statistics.mean(used), "mean_wall_s": statistics.mean(walls),
            "coverage": statistics.mean(used) / max(1, size)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--instances", default="micro2,micro4")
    ap.add_argument("--seeds", type=int, default=10)
    ap.add_argument("--evals", type=int, default=400)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    rows = [bench_instance(n, args.seeds, args.evals) for n in args.instances.split(",")]
    for r in rows:
        print(f"{r['instance']:8s} space {r['space_size']:8d} ({r['feasible_plans']} feasible)  optimum {r['optimum_tokens_per_s']:.4e} tok/s  "
              f"gap mean {100 * r['mean_gap']:.2f}% worst {100 * r['worst_gap']:.2f}%  hits {100 * r['hit_rate']:.0f}%  "
              f"evals {r['mean_evaluations']:.0f}  coverage {100 * r['coverage']:.1f}%  {r['mean_wall_s']:.2f} s/run")
    if args.output:
        Path(args.output).write_text(json.dumps(rows, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
