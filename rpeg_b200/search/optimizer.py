"""Simulated-annealing plan search over parallelism, placement, microbatching, actor-critic
sharing, stage fusion and staleness, plus the greedy polishing pass.

Algorithm (same design and defaults as the reference, RPEG/search/optimizer.py:33-1188):
  outer loop  over structural settings (template, fusion flag, staleness vector), each with an
              evaluation budget ``E_struct`` and, under a wall-clock deadline, an equal time share;
  restarts    the first chain of a structure starts from the seed plan at ``T_init``; later chains
              restart warm from the best elite of that structure family at ``T_warm`` (random
              restart if none is valid); two restarts without a new evaluation end the structure;
  chain step  with probability ``alpha_pair * min(1, T/T_init)`` a donor/receiver pair move, else
              up to ``K_x`` single-vertex neighbours; cache misses are evaluated in parallel by a
              process pool (best-of-K); Metropolis acceptance of the best neighbour on the relative
              score difference with constant temperature (optional geometric cooling); a chain ends
              after ``stag_window`` consecutive rejections;
  bookkeeping global best (strict improvement by ``score_eps``), best feasible, top-``K_elite``
              distinct feasible plans per family; shared-trunk plans are scored with a
              ``(1 - lambda_ac)`` factor; optional efficiency objective ``raw * utilization`` within a
              throughput-loss bound.
The search owns a ``random.Random(seed)``; pool workers are pure functions, so a run is
reproducible from its seed whenever no wall-clock deadline is set.
"""
from __future__ import annotations

import math
import multiprocessing as mp
import os
import random
import time
from dataclasses import dataclass, field
from typing import Dict, FrozenSet, List, Optional, Set, Tuple

from ..analytic.cost import NodeCostModel
from ..analytic.hardware import Hardware
from ..analytic.memory import MemoryPolicy, NodeMemoryModel
from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import Model
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from ..passes.lower import lower
from ..passes.unroll import unroll
from . import evaluate as ev
from .cache import EvalCache
from .evaluate import Configuration, eval_worker, evaluate_cached, evaluation_cache_key, is_valid
from .inter_model import DEFAULT_T_CAND, InterModelConfig, Iter_inter_model_candidates
from .moves import (CandidateDirectory, MoveStats, SearchFlags, build_candidate_directory, move_gen, multi_move_pair,
                    sample_strategy)

_STRUCTURES = frozenset({"separate", "fused", "ac_share"})


@dataclass
class OptimizerConfig:
    K_x: int = 6
    T_max: int = 50
    E_max: int = 5000
    E_struct: int = 400
    T_cand: Optional[Dict[Model, Set[int]]] = None
    structural_candidates: Optional[FrozenSet[str]] = None
    lambda_ac: float = 0.15
    score_eps: float = 1e-4
    T_init: float = 0.30
    T_warm: float = 0.05
    T_min: float = 0.01
    K_elite: int = 3
    alpha_pair: float = 0.28
    stag_window: int = 20
    max_throughput_loss: float = 0.0
    I_max: int = 0
    R_max: int = 10000
    T_cool: float = 0.0
    algorithm: str = "ppo"
    deadline: Optional[float] = None
    deadline_per_struct: Optional[float] = None
    fixed_mb: bool = False
    uniform_vertex: bool = False
    no_polish: bool = False
    hard_oom: bool = False
    geometric_cooling: bool = False
    memory_optimizer_stage: int = 2
    memory_activation_checkpointing: bool = True
    memory_runtime_overhead_fraction: float = 0.0
    memory_worker_overhead_bytes: float = 0.0
    memory_semantic_activation_cache_bytes: float = 0.0
    memory_max_worker_groups_per_gpu: int = 0
    memory_kv_cache_budget_bytes: float = 0.0
    memory_activation_token_cap: int = 0
    seed: Optional[int] = None
    workers: Optional[int] = None   # process-pool size; default min(K_x, cpu count); 1 disables the pool
    verbose: bool = False

    def __post_init__(self) -> None:
        if self.structural_candidates is not None:
            self.structural_candidates = frozenset(self.structural_candidates)
            unknown = self.structural_candidates - _STRUCTURES
            if unknown or not self.structural_candidates:
                raise ValueError("structural_candidates must be a non-empty subset of " + ", ".join(sorted(_STRUCTURES)))
        self.memory_policy()  # validates the memory knobs
        if self.I_max <= 0:
            self.I_max = max(1, int(0.5 * self.E_struct / ((self.K_x + 1) / 2)))
        self.T_cool = (self.T_min / self.T_init) ** (1.0 / (0.7 * self.I_max))

    def memory_policy(self) -> MemoryPolicy:
        return MemoryPolicy(self.memory_optimizer_stage, self.memory_activation_checkpointing,
                            self.memory_runtime_overhead_fraction, self.memory_worker_overhead_bytes,
                            self.memory_semantic_activation_cache_bytes, self.memory_max_worker_groups_per_gpu,
                            self.memory_kv_cache_budget_bytes, self.memory_activation_token_cap)

    def flags(self) -> SearchFlags:
        return SearchFlags(self.fixed_mb, self.uniform_vertex)


def penalized_score(raw: float, rpeg: RPEG, cfg: OptimizerConfig, ac_share: bool) -> float:
    return raw * (1.0 - cfg.lambda_ac) if (ac_share and cfg.lambda_ac != 0.0) else raw


def structure_name(ic: InterModelConfig) -> str:
    return "ac_share" if ic.ac_share else ("fused" if ic.intra_stage_fusion else "separate")


def plan_fingerprint(plan: ExecutionPlan) -> tuple:
    return tuple((v, plan.pi[v], plan.sigma[v].origin if v in plan.sigma else None, plan.mb.get(v)) for v in sorted(plan.pi))


@dataclass
class SearchReport:
    evaluations: int = 0
    cache: dict = field(default_factory=dict)
    wall_s: float = 0.0
    structures: List[dict] = field(default_factory=list)
    best_score: float = 0.0
    best_feasible: bool = False
    moves: str = ""


class _Search:
    def __init__(self, base: Configuration, suite, workload, hw, K_eval, cfg: OptimizerConfig, cache: EvalCache):
        self.base, self.suite, self.workload, self.hw, self.K_eval, self.cfg, self.cache = base, suite, workload, hw, K_eval, cfg, cache
        self.rng = random.Random(cfg.seed) if cfg.seed is not None else random.Random(random.getrandbits(64))
        self.policy = cfg.memory_policy()
        self.flags = cfg.flags()
        self.cost_model = NodeCostModel(hw, suite, workload, optimizer_stage=self.policy.optimizer_stage,
                                        activation_checkpointing=self.policy.activation_checkpointing)
        self.E = 0
        self.best: Tuple[Optional[Configuration], float] = (None, -math.inf)
        self.best_feasible: Tuple[Optional[Configuration], float] = (None, -math.inf)
        self.best_raw = 0.0
        self.elite: Dict[tuple, List[Tuple[float, ExecutionPlan]]] = {}
        self.elite_seen: Dict[tuple, set] = {}
        self.stats = MoveStats()
        self.accepted = {"strategy": 0, "placement": 0}
        self.rejected = 0
        self.report = SearchReport()
        n = cfg.workers if cfg.workers is not None else min(cfg.K_x, os.cpu_count() or 1)
        self.pool = mp.get_context("fork").Pool(n) if n > 1 else None

    # ---- helpers
    def close(self) -> None:
        if self.pool is not None:
            self.pool.close()
            self.pool.join()
            self.pool = None

    def mem_model(self, rpeg: RPEG) -> NodeMemoryModel:
        return NodeMemoryModel.from_policy(self.hw, self.suite, self.workload, self.policy, trainable=frozenset(rpeg.trainable),
                                           shadow_models=frozenset(m for m in rpeg.trainable if rpeg.tau.get(m, 0) > 0))

    def objective(self, raw: float, trace, ic: InterModelConfig) -> float:
        s = raw
        d = self.cfg.max_throughput_loss
        if d > 0.0 and trace is not None:
            self.best_raw = max(self.best_raw, raw)
            s = raw * 1e-12 if raw < (1.0 - d) * self.best_raw else raw * max(trace.utilization(), 1e-6)
        return penalized_score(s, None, self.cfg, ic.ac_share)

    def record(self, config: Configuration, raw: float, trace, feasible: bool, ic: InterModelConfig) -> float:
        score = self.objective(raw, trace, ic)
        if feasible:
            self._elite_insert(ic.family(), raw, config.plan)
        if score > self.best[1] * (1.0 + self.cfg.score_eps) or self.best[0] is None:
            self.best = (config, score)
        if feasible and score > self.best_feasible[1]:
            self.best_feasible = (config, score)
        return score

    def _elite_insert(self, family, raw: float, plan: ExecutionPlan) -> None:
        fp = plan_fingerprint(plan)
        seen = self.elite_seen.setdefault(family, set())
        if fp in seen:
            return
        lst = self.elite.get(family, [])
        if len(lst) >= self.cfg.K_elite and raw <= lst[-1][0]:
            return
        self.elite[family] = sorted(lst + [(raw, plan)], key=lambda x: -x[0])[: self.cfg.K_elite]
        seen.add(fp)

    def result(self) -> Configuration:
        return self.best_feasible[0] if self.best_feasible[0] is not None else self.best[0]

    def out_of_budget(self) -> bool:
        return self.E >= self.cfg.E_max or (self.cfg.deadline is not None and time.perf_counter() >= self.cfg.deadline)

    # ---- restarts
    def random_plan(self, config: Configuration) -> ExecutionPlan:
        plan = ExecutionPlan()
        verts = list(config.rpeg.vertices)
        fused = set()
        if config.intra_stage_fusion:
            by_id = {v.id: v for v in verts}
            if not {"t_pi", "t_V"} <= set(by_id):
                raise RuntimeError("intra-stage fusion requires t_pi and t_V")
            for _ in range(100):
                s = sample_strategy(self.rng, by_id["t_pi"], self.suite, config.device_space, self.workload, flags=self.flags)
                if s is not None and self.suite.specs[by_id["t_V"].kind.model].L % s[1][1] == 0:
                    break
            else:
                raise RuntimeError("no actor/critic-compatible fused layout found")
            for vid in ("t_pi", "t_V"):
                plan.sigma[vid], plan.pi[vid], plan.mb[vid] = s
                fused.add(vid)
        for v in verts:
            if v.id in fused:
                continue
            for _ in range(100):
                s = sample_strategy(self.rng, v, self.suite, config.device_space, self.workload, flags=self.flags)
                if s is not None:
                    break
            else:
                raise RuntimeError(f"could not sample a strategy for {v.id}")
            plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = s
        return plan

    def random_restart(self, config: Configuration, mem, attempts: int = 50) -> Optional[Configuration]:
        for _ in range(attempts):
            try:
                cand = Configuration(config.rpeg, self.random_plan(config), config.device_space, config.intra_stage_fusion,
                                     config.transfer_resource_policy)
            except RuntimeError:
                return None
            if is_valid(cand, self.suite, self.workload, mem):
                return cand
        return None

    # ---- neighbour evaluation (best of K, misses in parallel)
    def evaluate_many(self, cands: List[Configuration]):
        out, todo = [], []
        for c in cands:
            key = evaluation_cache_key(c, self.policy)
            if key in self.cache:
                out.append((c, *self.cache.get(key), False))
            else:
                todo.append((c, key))
        if todo:
            args = [(c, self.suite, self.workload, self.hw, self.K_eval, self.policy) for c, _ in todo]
            res = self.pool.map(eval_worker, args) if (self.pool is not None and len(todo) > 1) else [eval_worker(a) for a in args]
            for (c, key), (s, t, f) in zip(todo, res):
                self.cache.put(key, s, t, f)
                out.append((c, s, t, f, True))
        return out

    # ---- one structural setting
    def run_structure(self, rpeg: RPEG, ic: InterModelConfig, directory: CandidateDirectory, struct_deadline: Optional[float]) -> dict:
        cfg = self.cfg
        mem = self.mem_model(rpeg)
        mk = lambda plan: Configuration(rpeg, plan, self.base.device_space, ic.intra_stage_fusion,  # noqa: E731
                                        self.base.transfer_resource_policy)
        seed_cfg = mk(self.base.plan)
        info = {"structure": structure_name(ic), "tau": {m.value: t for m, t in ic.tau.items()}, "evaluations": 0,
                "restarts": 0, "best": -math.inf}
        if is_valid(seed_cfg, self.suite, self.workload, mem):
            config = seed_cfg
        else:
            config = self.random_restart(mk(ExecutionPlan()), mem)
            if config is None:
                if not {v.id for v in rpeg.vertices} <= (set(seed_cfg.plan.sigma) & set(seed_cfg.plan.pi) & set(seed_cfg.plan.mb)):
                    info["skipped"] = "no valid start"
                    return info
                config = seed_cfg  # infeasible seed, searched under the soft memory penalty
        E_s, r, idle_restarts, exhausted = 0, 0, 0, False

        def budget_hit() -> bool:
            return E_s >= cfg.E_struct or (struct_deadline is not None and time.perf_counter() >= struct_deadline)

        while r < cfg.R_max and not exhausted:
            E_at_restart = E_s
            if r > 0:
                elites = self.elite.get(ic.family(), [])
                nxt = None
                if elites:
                    warm = mk(elites[0][1])
                    if is_valid(warm, self.suite, self.workload, mem):
                        nxt = warm
                if nxt is None:
                    nxt = self.random_restart(config, mem)
                if nxt is None:
                    r += 1
                    idle_restarts += 1
                    exhausted = idle_restarts >= 2
                    continue
                config, idle_restarts = nxt, 0
                info["restarts"] += 1
            raw, trace, feasible, miss = evaluate_cached(config, self.cache, self.suite, self.workload, self.hw, self.K_eval, self.policy)
            if miss:
                self.E += 1
                E_s += 1
            score = self.record(config, raw, trace, feasible, ic)
            info["best"] = max(info["best"], score)
            T = cfg.T_warm if r > 0 else cfg.T_init
            executable, rejections = None, 0
            while True:
                if self.out_of_budget():
                    info["evaluations"] = E_s
                    info["stop"] = "global budget"
                    return info
                if budget_hit():
                    exhausted = True
                    break
                pair = self.rng.random() < cfg.alpha_pair * min(1.0, T / cfg.T_init)
                if pair:
                    nb = multi_move_pair(config, self.suite, self.workload, self.rng, flags=self.flags)
                    if nb is None:
                        self.stats.n_pair_failed += 1
                        T = max(cfg.T_min, T * cfg.T_cool)
                        continue
                    self.stats.n_pair_proposed += 1
                    cands = [nb]
                else:
                    if executable is None:
                        executable = lower(rpeg, unroll(rpeg, self.K_eval), config.plan, self.suite, self.K_eval,
                                           workload=self.workload, intra_stage_fusion=config.intra_stage_fusion)
                    cands = move_gen(config, executable, trace, directory, cfg.K_x, cfg.T_max, T, cfg.T_init, self.rng,
                                     self.stats, self.flags)
                if not cands:
                    break
                top = (-math.inf, None, None)
                for c, s_raw, t, f, was_miss in self.evaluate_many(cands):
                    if was_miss:
                        self.E += 1
                        E_s += 1
                    s = self.record(c, s_raw, t, f, ic)
                    info["best"] = max(info["best"], s)
                    if s > top[0]:
                        top = (s, c, t)
                if self.out_of_budget():
                    info["evaluations"] = E_s
                    info["stop"] = "global budget"
                    return info
                if budget_hit():
                    exhausted = True
                if top[1] is not None and not exhausted:
                    delta = (top[0] - score) / (abs(score) + 1e-12)
                    if abs(delta) >= 1e-6:
                        accept = delta >= 0.0 or self.rng.random() < math.exp(delta / T)
                        if accept:
                            if pair:
                                self.stats.n_pair_accepted += 1
                            else:
                                moved_strategy = top[1].plan.pi != config.plan.pi or top[1].plan.mb != config.plan.mb
                                self.accepted["strategy" if moved_strategy else "placement"] += 1
                            config, score, trace = top[1], top[0], top[2]
                            executable, rejections = None, 0
                        else:
                            if pair:
                                self.stats.n_pair_rejected += 1
                            else:
                                self.rejected += 1
                            rejections += 1
                if cfg.geometric_cooling:
                    T = max(cfg.T_min, T * cfg.T_cool)
                if exhausted or (cfg.stag_window > 0 and rejections >= cfg.stag_window):
                    break
            r += 1
            if E_s == E_at_restart:
                idle_restarts += 1
                exhausted = exhausted or idle_restarts >= 2
            else:
                idle_restarts = 0
        info["evaluations"] = E_s
        return info

    def run(self) -> Configuration:
        cfg = self.cfg
        t0 = time.perf_counter()
        raw, trace, feasible, _ = evaluate_cached(self.base, self.cache, self.suite, self.workload, self.hw, self.K_eval, self.policy)
        self.E = 1
        base_ic = InterModelConfig(False, dict(self.base.rpeg.tau), cfg.algorithm, self.base.intra_stage_fusion)
        self.record(self.base, raw, trace, feasible, base_ic)
        structs = list(Iter_inter_model_candidates(self.suite, self.workload, cfg.T_cand or DEFAULT_T_CAND, cfg.algorithm))
        if cfg.structural_candidates is not None:
            structs = [s for s in structs if structure_name(s[1]) in cfg.structural_candidates]
        if not structs:
            raise ValueError(f"structural_candidates exclude every candidate for algorithm={cfg.algorithm}")
        directory, dir_for = None, None
        for i, (rpeg, ic) in enumerate(structs):
            if self.out_of_budget():
                break
            deadline = None
            if cfg.deadline is not None:
                left = max(0.0, cfg.deadline - time.perf_counter())
                deadline = time.perf_counter() + left / (len(structs) - i)
            if dir_for != rpeg.vertex_ids():
                directory = build_candidate_directory(rpeg, self.suite, self.base.device_space, self.workload, self.cost_model,
                                                      self.mem_model(rpeg), flags=self.flags)
                dir_for = rpeg.vertex_ids()
            info = self.run_structure(rpeg, ic, directory, deadline)
            self.report.structures.append(info)
            if cfg.verbose:
                print(f"[search] {info}")
        self.report.evaluations = self.E
        self.report.cache = self.cache.stats()
        self.report.wall_s = time.perf_counter() - t0
        self.report.best_score = self.best_feasible[1] if self.best_feasible[0] is not None else self.best[1]
        self.report.best_feasible = self.best_feasible[0] is not None
        self.report.moves = self.stats.summary(self.accepted["strategy"], self.accepted["placement"], self.rejected)
        return self.result()


def optimize(base_config: Configuration, suite: ModelSuite, workload: Workload, hw: Hardware, K_eval: int,
             opt_config: OptimizerConfig, cache: EvalCache, report: Optional[list] = None) -> Configuration:
    """Search for the plan with the best (penalised) throughput. Returns the best memory-feasible
    configuration found, or the best overall if none is feasible. Appends a ``SearchReport`` to
    ``report`` when a list is passed."""
    ev.ABLATION_HARD_OOM = opt_config.hard_oom  # before the pool forks
    search = _Search(base_config, suite, workload, hw, K_eval, opt_config, cache)
    try:
        best = search.run()
    finally:
        search.close()
    if report is not None:
        report.append(search.report)
    return best


def polish(best_config: Configuration, suite: ModelSuite, workload: Workload, hw: Hardware, K_eval: int,
           opt_config: OptimizerConfig, cache: EvalCache, directory: Optional[CandidateDirectory] = None,
           ac_share: bool = False, max_rounds: int = 50) -> Configuration:
    """Deterministic greedy coordinate descent around the search result: per vertex (id order),
    evaluate every strategy within a window of its directory position at origin (0, 0, 0) and apply
    the best strict improvement among feasible ones; repeat until a pass changes nothing
    (reference: RPEG/search/optimizer.py:949-1188)."""
    ev.ABLATION_HARD_OOM = opt_config.hard_oom
    search = _Search(best_config, suite, workload, hw, K_eval, opt_config, cache)
    try:
        rpeg, space = best_config.rpeg, best_config.device_space
        if directory is None:
            directory = build_candidate_directory(rpeg, suite, space, workload, search.cost_model, search.mem_model(rpeg),
                                                  flags=search.flags)
        ic = InterModelConfig(ac_share, dict(rpeg.tau), opt_config.algorithm, best_config.intra_stage_fusion)
        config = best_config
        raw, trace, _, _ = evaluate_cached(config, cache, suite, workload, hw, K_eval, search.policy)
        score = search.objective(raw, trace, ic)
        from ..core.types import Allocation, packing_geometry
        for _ in range(max_rounds):
            improved = False
            for v in sorted(rpeg.vertices, key=lambda x: x.id):
                rows = directory.table[v.id]
                n = len(rows)
                if n == 0:
                    continue
                w = max(5, int(n * opt_config.T_min / opt_config.T_init))
                j_star = directory.position(v.id, config.plan)
                targets = [v.id]
                peer_L = None
                if config.intra_stage_fusion and v.id in ("t_pi", "t_V"):
                    peer = "t_V" if v.id == "t_pi" else "t_pi"
                    targets.append(peer)
                    peer_L = suite.specs[rpeg.vertex(peer).kind.model].L
                cands = []
                for j in range(max(0, j_star - w), min(n - 1, j_star + w) + 1):
                    if j == j_star:
                        continue
                    dp, pp, tp, r_ext, n_ext, mb = rows[j][:6]
                    geom = packing_geometry(dp, pp, tp, space.G)
                    if geom is None or (peer_L is not None and peer_L % pp):
                        continue
                    plan = config.plan.copy()
                    for t in targets:
                        plan.sigma[t], plan.pi[t], plan.mb[t] = Allocation((0, 0, 0), (r_ext, n_ext, geom[0])), (dp, pp, tp), mb
                    cands.append(Configuration(rpeg, plan, space, config.intra_stage_fusion, config.transfer_resource_policy))
                top = (score, None)
                for c, s_raw, t, f, _miss in search.evaluate_many(cands):
                    if f:
                        s = search.objective(s_raw, t, ic)
                        if s > top[0]:
                            top = (s, c)
                if top[1] is not None:
                    config, score = top[1], top[0]
                    improved = True
            if not improved:
                break
        return config
    finally:
        search.close()
