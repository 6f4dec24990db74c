"""End-to-end analytical driver: workload YAML (+ calibrated hardware YAML) -> baselines ->
simulated-annealing search -> polish -> results table and plan files.

Keeps the reference CLI and file formats (pipeline.py:65-388 config handling, :389-1245 baselines,
:1247-1765 main): sections ``hardware`` (grid + alpha-beta constants, mergeable from ``--hw``),
``models`` {actor, critic, reward}, ``workload``, ``policy`` {algorithm, allow_ac_share},
``optimizer`` (k_eval, e_max, e_struct, k_x, t_*, stag_window, staleness_candidates, ablation
flags), ``output`` {plots, plots_dir, log_file, base_plan, opt_plan, seed}. The reporting
baselines always use the synchronous graph (tau = 0); the search is seeded with the concurrent
heuristic plan (or ``--seed-plan``).
"""
from __future__ import annotations

import argparse
import copy
import itertools
import re
import sys
import time
from typing import Dict, List, Optional, Tuple

import yaml

from ..analytic.cost import NodeCostModel
from ..analytic.hardware import Hardware
from ..analytic.memory import MemoryPolicy, NodeMemoryModel
from ..analytic.models import ModelSpec, ModelSuite
from ..analytic.workload import Workload
from ..core.log import init_logging, print_run_header
from ..core.types import Allocation, DeviceSpace, Model, packing_geometry
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from ..ir.serialize import load_plan, save_plan
from ..ir.templates import build_rpeg
from ..search.cache import EvalCache
from ..search.evaluate import Configuration, evaluate_cached, is_valid
from ..search.inter_model import DEFAULT_T_CAND
from ..search.moves import CandidateDirectory, build_candidate_directory
from ..search.optimizer import OptimizerConfig, SearchReport, optimize, polish

_HW_REQUIRED = ("flops_per_gpu", "memory_per_gpu", "memory_bandwidth",
                "alpha_coll_g", "beta_coll_g", "alpha_coll_n", "beta_coll_n", "alpha_coll_r", "beta_coll_r",
                "alpha_p2p_g", "beta_p2p_g", "alpha_p2p_n", "beta_p2p_n", "alpha_p2p_r", "beta_p2p_r")
_HW_OPTIONAL = ("gemm_m_half", "gemm_k_half", "decode_bw_eff", "non_gemm_constant", "non_gemm_scaling",
                "non_gemm_batch_cal", "op_generation_scale", "op_inference_scale", "op_training_scale",
                "activation_comm_overhead_s", "weight_comm_scale", "reshard_scale", "fabric", "fused_overlap",
                "ffn_matrices", "sustained_flops_fraction", "attention_flops_eff", "elementwise_s_per_token_layer",
                "gen_max_concurrency", "gen_kv_budget_bytes", "decode_step_overhead_s", "expected_lengths",
                "gen_shared_prompt_cost")


def make_yaml_loader():
    """YAML loader that also reads ``1e-6`` / ``4.4e14`` (no dot) as floats, which PyYAML's
    default resolver treats as strings."""
    class Loader(yaml.SafeLoader):
        pass

    Loader.add_implicit_resolver(
        "tag:yaml.org,2002:float",
        re.compile(r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                        |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
                        |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                        |[-+]?\.(?:inf|Inf|INF)|\.(?:nan|NaN|NAN))$""", re.X),
        list("-+0123456789."))
    return Loader


def load_yaml(path: str) -> dict:
    with open(path) as f:
        return yaml.load(f, Loader=make_yaml_loader()) or {}


def _require(d: dict, *keys: str, section: str = "") -> None:
    for k in keys:
        if k not in d:
            raise ValueError(f"[{section or 'config'}] missing required key '{k}'")


def validate_config(cfg: dict) -> None:
    _require(cfg, "hardware", "models", "workload", "optimizer")
    hw = cfg["hardware"]
    _require(hw, "racks", "nodes_per_rack", "gpus_per_node", *_HW_REQUIRED, section="hardware")
    if min(hw["racks"], hw["nodes_per_rack"], hw["gpus_per_node"]) < 1:
        raise ValueError("[hardware] racks, nodes_per_rack, gpus_per_node must all be >= 1")
    algo = cfg.get("policy", {}).get("algorithm", "ppo")
    if algo not in ("ppo", "grpo", "dpo"):
        raise ValueError(f"[policy] unsupported algorithm '{algo}' (supported: ppo, grpo, dpo)")
    roles = {"dpo": ("actor",), "grpo": ("actor", "reward")}.get(algo, ("actor", "critic", "reward"))
    for role in roles:
        _require(cfg["models"], role, section="models")
        _require(cfg["models"][role], "layers", "hidden_dim", "ffn_dim", "vocab_size", section=f"models.{role}")
    _require(cfg["workload"], "batch_size", "samples_per_prompt", "context_length", "generation_length", section="workload")
    _require(cfg["optimizer"], "k_eval", section="optimizer")
    if cfg["optimizer"]["k_eval"] < 1:
        raise ValueError("[optimizer] k_eval must be >= 1")
    for name in (cfg["optimizer"].get("staleness_candidates") or {}):
        if name not in ("actor", "critic", "ac_share"):
            raise ValueError(f"[optimizer.staleness_candidates] unknown model '{name}'")


def build_device_space(cfg: dict) -> DeviceSpace:
    hw = cfg["hardware"]
    return DeviceSpace(int(hw["racks"]), int(hw["nodes_per_rack"]), int(hw["gpus_per_node"]))


def build_hardware(cfg: dict) -> Hardware:
    hw = cfg["hardware"]
    kw = {k: float(hw[k]) for k in _HW_REQUIRED}
    for k in _HW_OPTIONAL:
        if k in hw:
            kw[k] = hw[k] if k == "fabric" else float(hw[k])
    return Hardware(**kw)


def _spec(d: dict) -> ModelSpec:
    return ModelSpec(int(d["layers"]), int(d["hidden_dim"]), int(d["ffn_dim"]), int(d["vocab_size"]),
                     int(d.get("dtype_bytes", 2)), int(d.get("head_dim", 128)), d.get("parameter_count"))


def build_suite(cfg: dict) -> ModelSuite:
    m = cfg["models"]
    actor = _spec(m["actor"])
    specs = {Model.ACTOR: actor, Model.REFERENCE: _spec(m["reference"]) if "reference" in m else actor, Model.AC_SHARE: actor}
    if "critic" in m:
        specs[Model.CRITIC] = _spec(m["critic"])
    if "reward" in m:
        specs[Model.REWARD] = _spec(m["reward"])
    return ModelSuite(specs)


def build_workload(cfg: dict) -> Workload:
    w = cfg["workload"]
    q = w.get("gen_quantiles")
    quant = tuple((float(a), int(b)) for a, b in q) if q else None
    if quant:
        fr = [a for a, _ in quant]
        if fr != sorted(fr) or abs(fr[-1] - 1.0) > 1e-9 or quant[-1][1] > int(w["generation_length"]):
            raise ValueError("[workload.gen_quantiles] fractions must increase to 1.0 and lengths stay within generation_length")
    return Workload(int(w["batch_size"]), int(w["samples_per_prompt"]), int(w["context_length"]), int(w["generation_length"]), quant)


def build_optimizer_config(cfg: dict, allow_ac_share: bool, algorithm: str = "ppo") -> OptimizerConfig:
    o = cfg["optimizer"]
    sc = o.get("staleness_candidates")
    names = {"actor": Model.ACTOR, "critic": Model.CRITIC, "ac_share": Model.AC_SHARE}
    if algorithm in ("grpo", "dpo"):
        t_cand = {Model.ACTOR: set(sc["actor"]) if sc and "actor" in sc else {0, 1}}
    elif sc is None and allow_ac_share:
        t_cand = None
    else:
        t_cand = copy.deepcopy(DEFAULT_T_CAND)
        for name, vals in (sc or {}).items():
            t_cand[names[name]] = set(vals)
        if not allow_ac_share:
            t_cand[Model.AC_SHARE] = set()
    structures = o.get("structural_candidates")
    return OptimizerConfig(
        K_x=o.get("k_x", 6), T_max=o.get("t_max", 50), E_max=o.get("e_max", 5000), E_struct=o.get("e_struct", 400),
        T_cand=t_cand, structural_candidates=frozenset(structures) if structures else None,
        lambda_ac=o.get("lambda_ac", 0.15), score_eps=o.get("score_eps", 1e-4), T_init=o.get("t_init", 0.30),
        T_warm=o.get("t_warm", 0.10), T_min=o.get("t_min", 0.03), stag_window=o.get("stag_window", 20),
        alpha_pair=o.get("alpha_pair", 0.28), max_throughput_loss=o.get("max_throughput_loss", 0.0), algorithm=algorithm,
        fixed_mb=o.get("fixed_mb", False), uniform_vertex=o.get("uniform_vertex", False), no_polish=o.get("no_polish", False),
        hard_oom=o.get("hard_oom", False), geometric_cooling=o.get("geometric_cooling", False),
        memory_optimizer_stage=o.get("memory_optimizer_stage", 2),
        memory_activation_checkpointing=o.get("memory_activation_checkpointing", True),
        seed=cfg.get("output", {}).get("seed"), workers=o.get("workers"), verbose=bool(o.get("verbose", False)))


# ---------------------------------------------------------------------------------- baselines
class Baselines:
    def __init__(self, rpeg: RPEG, suite: ModelSuite, workload: Workload, hw: Hardware, space: DeviceSpace,
                 policy: MemoryPolicy, directory: Optional[CandidateDirectory] = None):
        self.rpeg, self.suite, self.workload, self.hw, self.space, self.policy = rpeg, suite, workload, hw, space, policy
        self.cost = NodeCostModel(hw, suite, workload, optimizer_stage=policy.optimizer_stage,
                                  activation_checkpointing=policy.activation_checkpointing)
        self.mem = NodeMemoryModel.from_policy(hw, suite, workload, policy, trainable=frozenset(rpeg.trainable))
        self.dir = directory or build_candidate_directory(rpeg, suite, space, workload, self.cost, self.mem)

    def _cfg(self, plan: ExecutionPlan) -> Configuration:
        return Configuration(self.rpeg, plan, self.space)

    def _assign(self, plan: ExecutionPlan, vid: str, row, origin=(0, 0, 0)) -> None:
        dp, pp, tp, r_ext, n_ext, mb = row[:6]
        g_ext = packing_geometry(dp, pp, tp, self.space.G)[0]
        plan.sigma[vid], plan.pi[vid], plan.mb[vid] = Allocation(tuple(origin), (r_ext, n_ext, g_ext)), (dp, pp, tp), mb

    def greedy(self) -> Optional[Configuration]:
        """Fastest memory-feasible strategy per vertex, everything at origin (0, 0, 0)."""
        plan = ExecutionPlan()
        for v in self.rpeg.vertices:
            if not self.dir.table[v.id]:
                return None
            self._assign(plan, v.id, self.dir.table[v.id][0])
        cfg = self._cfg(plan)
        if is_valid(cfg, self.suite, self.workload, self.mem):
            return cfg
        # back off per vertex to slower candidates until the whole plan fits
        for depth in range(1, 50):
            for v in self.rpeg.vertices:
                rows = self.dir.table[v.id]
                if depth < len(rows):
                    trial = plan.copy()
                    self._assign(trial, v.id, rows[depth])
                    if is_valid(self._cfg(trial), self.suite, self.workload, self.mem):
                        return self._cfg(trial)
        return cfg

    def fully_colocated(self) -> Optional[Configuration]:
        """Fastest strategy per vertex among those that span the whole machine."""
        total = self.space.num_devices()
        plan = ExecutionPlan()
        for v in self.rpeg.vertices:
            rows = [r for r in self.dir.table[v.id] if r[0] * r[1] * r[2] == total]
            if not rows:
                return None
            self._assign(plan, v.id, rows[0])
        return self._cfg(plan)

    def depth_groups(self) -> List[List[str]]:
        """Vertices grouped by longest-path depth over data edges: members of a group are independent."""
        depth = {v.id: 0 for v in self.rpeg.vertices}
        for v in self.rpeg.topological_vertices():
            for e in self.rpeg.data_edges:
                if e.src.id == v.id:
                    depth[e.dst.id] = max(depth[e.dst.id], depth[v.id] + 1)
        groups: Dict[int, List[str]] = {}
        for vid, d in depth.items():
            groups.setdefault(d, []).append(vid)
        return [groups[d] for d in sorted(groups)]

    def _slices(self, k: int) -> Optional[List[Tuple[Tuple[int, int, int], Tuple[int, int, int]]]]:
        """Cut the machine into ``k`` equal boxes along racks, then nodes, then GPUs."""
        R, N, G = self.space.R, self.space.N, self.space.G
        for axis, size in ((0, R), (1, N), (2, G)):
            if size % k == 0 and size >= k:
                ext = [R, N, G]
                ext[axis] = size // k
                out = []
                for i in range(k):
                    org = [0, 0, 0]
                    org[axis] = i * ext[axis]
                    out.append((tuple(org), tuple(ext)))
                return out
        return None

    def _best_in_box(self, vid: str, box_extent) -> Optional[tuple]:
        for row in self.dir.table[vid]:
            dp, pp, tp, r_ext, n_ext, _mb = row[:6]
            g_ext = packing_geometry(dp, pp, tp, self.space.G)[0]
            if r_ext <= box_extent[0] and n_ext <= box_extent[1] and g_ext <= box_extent[2]:
                return row
        return None

    def concurrent(self) -> Optional[Configuration]:
        """Run independent vertices side by side on equal device slices; per group pick the slice
        count that minimises max-over-slices of the summed member times; drop to fewer slices (more
        sharing) while the plan does not fit in memory; fall back to ``greedy``."""
        groups = self.depth_groups()
        choice: List[int] = []
        per_group_options: List[List[Tuple[float, int, dict]]] = []
        for group in groups:
            options = []
            for k in range(len(group), 0, -1):
                slices = self._slices(k)
                if slices is None:
                    continue
                assign, load, ok = {}, [0.0] * k, True
                for i, vid in enumerate(sorted(group, key=lambda x: -self._fastest_time(x))):
                    j = min(range(k), key=lambda s: load[s])
                    row = self._best_in_box(vid, slices[j][1])
                    if row is None:
                        ok = False
                        break
                    assign[vid] = (row, slices[j][0])
                    load[j] += row[6]
                if ok:
                    options.append((max(load), -k, assign))
            if not options:
                return self.greedy()
            options.sort(key=lambda o: (o[0], o[1]))
            per_group_options.append(options)
            choice.append(0)
        for _ in range(sum(len(o) for o in per_group_options) + 1):
            plan = ExecutionPlan()
            for gi, opts in enumerate(per_group_options):
                for vid, (row, origin) in opts[choice[gi]][2].items():
                    self._assign(plan, vid, row, origin)
            cfg = self._cfg(plan)
            if is_valid(cfg, self.suite, self.workload, self.mem):
                return cfg
            # relax the most concurrent group first
            movable = [gi for gi, opts in enumerate(per_group_options) if choice[gi] + 1 < len(opts)]
            if not movable:
                break
            gi = max(movable, key=lambda g: -per_group_options[g][choice[g]][1])
            choice[gi] += 1
        return self.greedy()

    def _fastest_time(self, vid: str) -> float:
        rows = self.dir.table[vid]
        return rows[0][6] if rows else 0.0

    def naive_concurrent(self) -> Optional[Configuration]:
        """Hand layout: generation and reference on all GPUs, the other inference and training
        vertices on complementary halves."""
        halves = self._slices(2)
        full = self._slices(1)
        if halves is None or full is None:
            return None
        plan = ExecutionPlan()
        side = 0
        for v in self.rpeg.vertices:
            whole = v.kind.role.value == "GEN" or v.id == "i_ref"
            origin, extent = full[0] if whole else halves[side % 2]
            if not whole:
                side += 1
            row = self._best_in_box(v.id, extent)
            if row is None:
                return None
            self._assign(plan, v.id, row, origin)
        return self._cfg(plan)


# ---------------------------------------------------------------------------------- reporting
def summarize(name: str, cfg: Optional[Configuration], cache, suite, workload, hw, K_eval, policy) -> Optional[dict]:
    if cfg is None:
        return None
    score, trace, feasible, _ = evaluate_cached(cfg, cache, suite, workload, hw, K_eval, policy)
    cm = NodeCostModel(hw, suite, workload, optimizer_stage=policy.optimizer_stage,
                       activation_checkpointing=policy.activation_checkpointing)
    flops = sum(cm._work(n) for n in trace.start if n.kind.value == "op")
    # the trace spans K_eval iterations while tokens/s and the makespan are per iteration: so is the FLOP rate
    return {"name": name, "tokens_per_s": score, "makespan_s": trace.makespan(), "pflops": flops / max(K_eval, 1) / trace.makespan() / 1e15,
            "utilization": trace.utilization(), "active_gpus": trace.n_active(), "feasible": feasible, "trace": trace}


def _span(lo: int, n: int) -> str:
    return f"{lo}" if n == 1 else f"{lo}-{lo + n - 1}"


def _where(a) -> str:
    (r0, n0, g0), (re, ne, ge) = a.origin, a.extent
    return f"r{_span(r0, re)} n[{_span(n0, ne)}] g[{_span(g0, ge)}]"


def print_plan_changes(base: Optional[Configuration], best: Configuration) -> None:
    """One line per vertex: parallelism, microbatches and placement of the starting plan and, after ``->``, what the
    search changed. The layout and the labels are those of the reference's result listing (pipeline.py:1741-1747),
    so scripts that read its logs read these too."""
    print("\n  Per-vertex plan (base \u2192 optimal):")
    print(f"    {'':2} {'vertex':<7} {'parallelism (dp,pp,tp)':<24} {'mb':>5}  placement (rack, nodes, gpus)")
    print(f"    {'':2} {'\u2500' * 6:<7} {'\u2500' * 22:<24} {'\u2500' * 5:>5}  {'\u2500' * 42}")
    for vid in sorted(best.plan.pi):
        new_pi, new_mb, new_at = best.plan.pi[vid], best.plan.mb.get(vid, 1), _where(best.plan.sigma[vid])
        if base is not None and vid in base.plan.pi:
            old_pi, old_mb, old_at = base.plan.pi[vid], base.plan.mb.get(vid, 1), _where(base.plan.sigma[vid])
        else:
            old_pi, old_mb, old_at = new_pi, new_mb, new_at
        fmt = lambda t: "(" + ",".join(str(x) for x in t) + ")"
        par = fmt(old_pi) if old_pi == new_pi else f"{fmt(old_pi)} -> {fmt(new_pi)}"
        mb = f"{old_mb}" if old_mb == new_mb else f"{old_mb}->{new_mb}"
        at = old_at if old_at == new_at else f"{old_at}  ->  {new_at}"
        changed = "*" if (old_pi, old_mb, old_at) != (new_pi, new_mb, new_at) else " "
        print(f"    {changed:2} {vid:<7} {par:<24} {mb:>5}  {at}")


def print_table(rows: List[dict], total_gpus: int) -> None:
    """Result table with the reference's row labels and column order (Greedy, Conc. Heuristic, Optimized, delta against
    greedy)."""
    rows = [r for r in rows if r]
    first, last = rows[0], rows[-1]
    delta = f"{100 * (last['tokens_per_s'] / first['tokens_per_s'] - 1):+.1f}%" if len(rows) > 1 and first["tokens_per_s"] > 0 else ""
    head = f"  {'Metric':<28}" + "".join(f"  {r['name']:>16}" for r in rows) + f"  {'\u0394 (vs greedy)':>14}"
    print("\n" + head)
    print(f"  {'\u2500' * 28}" + "".join(f"  {'\u2500' * 16}" for _ in rows) + f"  {'\u2500' * 14}")
    print(f"  {'Throughput (tokens/s)':<28}" + "".join(f"  {r['tokens_per_s']:>16.4e}" for r in rows) + f"  {delta:>14}")
    print(f"  {'Makespan (s)':<28}" + "".join(f"  {r['makespan_s']:>16.4e}" for r in rows))
    print(f"  {'Throughput (PFLOP/s)':<28}" + "".join(f"  {r['pflops']:>16.4f}" for r in rows) + f"  {delta:>14}")
    print(f"  {'GPU utilization':<28}" + "".join(f"  {100 * r['utilization']:>15.1f}%" for r in rows))
    print(f"  {'Active GPUs':<28}" + "".join(f"  {r['active_gpus']:>16}" for r in rows))
    print(f"  baseline_feasible: {bool(first['feasible'])}")


def run_pipeline(cfg: dict, *, time_budget_s: Optional[float] = None, seed_plan: Optional[str] = None,
                 debug: bool = False, make_plots: Optional[bool] = None) -> dict:
    """Programmatic form of the CLI. Returns the result rows, the best configuration and the
    search report."""
    validate_config(cfg)
    policy_cfg = cfg.get("policy", {})
    algo = policy_cfg.get("algorithm", "ppo")
    allow_ac = bool(policy_cfg.get("allow_ac_share", False)) and algo == "ppo"
    out = cfg.get("output", {})
    space, hw, suite, workload = build_device_space(cfg), build_hardware(cfg), build_suite(cfg), build_workload(cfg)
    opt_cfg = build_optimizer_config(cfg, allow_ac, algo)
    K_eval = int(cfg["optimizer"]["k_eval"])
    mem_policy = opt_cfg.memory_policy()
    print_run_header("RPEG plan search", algorithm=algo, devices=f"{space.R} x {space.N} x {space.G} = {space.num_devices()}",
                     batch=f"B={workload.B} K={workload.K} S={workload.S} T={workload.T}", k_eval=K_eval, seed=opt_cfg.seed)
    sync_rpeg = build_rpeg(algo, suite, workload)                       # tau = 0 everywhere
    tau0 = {m: sorted(opt_cfg.T_cand[m])[0] if (opt_cfg.T_cand and opt_cfg.T_cand.get(m)) else 0 for m in sync_rpeg.trainable}
    user_rpeg = build_rpeg(algo, suite, workload, tau=tau0)
    cache = EvalCache()
    base = Baselines(sync_rpeg, suite, workload, hw, space, mem_policy)
    t0 = time.perf_counter()
    greedy, conc = base.greedy(), base.concurrent()
    rows = [summarize("Greedy", greedy, cache, suite, workload, hw, K_eval, mem_policy),
            summarize("Conc. Heuristic", conc, cache, suite, workload, hw, K_eval, mem_policy)]
    for r in rows:
        if r:
            print(f"{r['name']}: {r['tokens_per_s']:.4e} tokens/s | makespan: {r['makespan_s']:.3f} s | feasible={r['feasible']}")
    seed_cfg = conc or greedy
    if seed_plan:
        seed_cfg = Configuration(user_rpeg, load_plan(seed_plan, user_rpeg), space)
    if seed_cfg is None:
        raise RuntimeError("no feasible starting plan: the models do not fit on this machine under the memory policy")
    if out.get("base_plan"):
        save_plan(Configuration(sync_rpeg, seed_cfg.plan, space), out["base_plan"])
    if time_budget_s:
        opt_cfg.deadline = time.perf_counter() + float(time_budget_s)
        opt_cfg.E_max = opt_cfg.E_struct = 10 ** 9
        opt_cfg.__post_init__()
    report: List[SearchReport] = []
    start = Configuration(user_rpeg, seed_cfg.plan, space)
    best = optimize(start, suite, workload, hw, K_eval, opt_cfg, cache, report)
    _, _, best_feasible, _ = evaluate_cached(best, cache, suite, workload, hw, K_eval, mem_policy)
    if best_feasible and not opt_cfg.no_polish:
        opt_cfg.deadline = None
        best = polish(best, suite, workload, hw, K_eval, opt_cfg, cache, ac_share=Model.AC_SHARE in best.rpeg.trainable)
    wall = time.perf_counter() - t0
    rows.append(summarize("Optimized", best, cache, suite, workload, hw, K_eval, mem_policy))
    st = cache.stats()
    print("\n  Search statistics")
    print(f"    wall time   {wall:.1f}s")
    print(f"    cache       hits={st['hits']}  misses={st['misses']}  total={st['hits'] + st['misses']}  hit_rate={100 * st['hit_rate']:.1f}%")
    print(f"    evaluations {report[0].evaluations}")
    print("\n  Structure")
    print(f"    ac_share    {Model.AC_SHARE in best.rpeg.trainable}")
    print("    tau         {" + ", ".join(f"{getattr(m, 'value', m)}:{t}" for m, t in sorted(best.rpeg.tau.items(), key=lambda kv: str(kv[0]))) + "}")
    print_plan_changes(seed_cfg, best)
    print_table(rows, space.num_devices())
    ref = rows[1] or rows[0]
    if ref and rows[2]:
        print(f"  Improvement over {ref['name']}: {100 * (rows[2]['tokens_per_s'] / ref['tokens_per_s'] - 1):+.1f}%")
    print(report[0].moves)
    if out.get("opt_plan"):
        save_plan(best, out["opt_plan"])
    do_plots = out.get("plots", False) if make_plots is None else make_plots
    if do_plots:
        try:
            from ..utils.visualize import exec_to_dot, rpeg_to_dot, trace_to_gantt_svg, unrolled_to_dot
            import os
            d = out.get("plots_dir", "figures")
            os.makedirs(d, exist_ok=True)
            trace_to_gantt_svg(rows[-1]["trace"], os.path.join(d, "optimized.gantt.svg"), space)
            if rows[1]:
                trace_to_gantt_svg(rows[1]["trace"], os.path.join(d, "baseline.gantt.svg"), space)
            # the three graphs of the compilation: algorithm template, unrolled iterations, lowered executable
            rpeg_to_dot(best.rpeg, os.path.join(d, "rpeg.dot"))
            from ..passes.lower import lower
            from ..passes.unroll import unroll
            un = unroll(best.rpeg, K_eval)
            unrolled_to_dot(un, os.path.join(d, "unrolled.dot"))
            exec_to_dot(lower(best.rpeg, un, best.plan, suite, K_eval, workload=workload,
                              intra_stage_fusion=best.intra_stage_fusion), os.path.join(d, "executable.dot"))
        except Exception as exc:  # plotting never fails a search
            print(f"  (plots skipped: {exc})")
    return {"rows": rows, "best": best, "report": report[0], "wall_s": wall, "cache": st}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="RPEG analytical plan optimizer")
    ap.add_argument("--config", required=True, help="workload/optimizer YAML")
    ap.add_argument("--hw", default=None, help="calibrated hardware YAML (flat keys) merged into the hardware section")
    ap.add_argument("--plots", action="store_true")
    ap.add_argument("--debug", action="store_true")
    ap.add_argument("--seed-plan", default=None, help="plan file to start the search from")
    ap.add_argument("--time", type=float, default=None, help="wall-clock search budget in seconds")
    args = ap.parse_args(argv)
    cfg = load_yaml(args.config)
    if args.hw:
        cfg.setdefault("hardware", {}).update(load_yaml(args.hw))
    init_logging(cfg.get("output", {}).get("log_file"), debug=args.debug)
    try:
        run_pipeline(cfg, time_budget_s=args.time, seed_plan=args.seed_plan, debug=args.debug,
                     make_plots=True if args.plots else None)
    except ValueError as exc:
        print(f"configuration error: {exc}", file=sys.stderr)
        return 2
    return 0
