"""Per-device memory model: weights, optimizer state, gradients, activations, KV cache, and the
peak over everything a plan puts on one GPU.

Byte formulas follow the reference (RPEG/model/memory.py:23-66, 273-537): a pipeline stage holds
``ceil(L/pp)`` layers split over ``tp`` plus an unsplit embedding on the first stage and head on the
last; Adam state is 12 bytes per parameter divided by ``dp`` under ZeRO>=1; gradients are divided
by ``dp`` under ZeRO-2; training activations use sqrt(L) checkpointing; inference activations take
the widest of attention / FFN / LM-head per token; the KV cache is ``2*sb*(B/dp)*K*(S+T)*(L/pp)*
(d/tp)``.

``device_peaks`` is the worker-liveness model of RPEG/model/memory.py:608-841: state that stays on
a GPU for the whole run (optimizer shards of trained models, serving copies on other workers,
frozen weights) is summed, and on top of it sits the largest single operator (its weights if not
already resident, plus its transient data); fused actor/critic training contributes the members'
static parts plus the peak of the fused pipeline schedule.
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, FrozenSet, List, Optional, Tuple

from ..core.types import Model, Role
from ..passes.lower import ExecNode, ExecNodeType, ExecutableRPEG
from .hardware import Hardware
from .models import ModelSuite
from .workload import Workload


def training_activation_bytes_per_microbatch(node: ExecNode, suite: ModelSuite, workload: Workload, *,
                                             activation_checkpointing: bool, token_cap: int = 0) -> float:
    if node.model is None or node.pi is None or node.mb is None:
        raise ValueError(f"{node.id}: training activation accounting needs model, pi and mb")
    spec = suite.specs[node.model]
    dp, pp, tp = node.pi
    b_local = workload.B * workload.K / (dp * node.mb)
    L_pp = math.ceil(spec.L / pp)
    layer_peak = max(2 * spec.d + 6 * spec.d / tp, 2 * spec.d + 2 * spec.d_ff / tp)
    if activation_checkpointing:
        c = max(1, math.isqrt(L_pp))
        per_token = math.ceil(L_pp / c) * spec.d + c * layer_peak
    else:
        per_token = L_pp * layer_peak
    tokens = b_local * (workload.S + workload.T)
    if token_cap > 0:           # the engine packs sequences into microbatches of at most this many tokens
        tokens = min(tokens, token_cap)
    return spec.dtype_bytes * tokens * per_token


@dataclass(frozen=True)
class MemoryPolicy:
    optimizer_stage: int = 2
    activation_checkpointing: bool = True
    runtime_overhead_fraction: float = 0.0
    worker_overhead_bytes: float = 0.0
    semantic_activation_cache_bytes: float = 0.0
    max_worker_groups_per_gpu: int = 0
    kv_cache_budget_bytes: float = 0.0      # > 0: paged KV with a fixed pool per GPU instead of a static full-length cache
    activation_token_cap: int = 0           # > 0: tokens per packed microbatch, bounds every activation estimate

    def __post_init__(self):
        if self.optimizer_stage not in (0, 1, 2):
            raise ValueError("optimizer_stage must be 0, 1, or 2")
        if not 0.0 <= self.runtime_overhead_fraction < 1.0:
            raise ValueError("runtime_overhead_fraction must be in [0, 1)")
        if min(self.worker_overhead_bytes, self.semantic_activation_cache_bytes, self.max_worker_groups_per_gpu) < 0:
            raise ValueError("memory policy sizes must be >= 0")


def optimizer_stage(name: str) -> int:
    key = str(name or "none").strip().lower().replace("-", "_")
    table = {"none": 0, "adamw": 0, "zero1": 1, "zero_1": 1, "zero_stage_1": 1, "stage1": 1,
             "zero2": 2, "zero_2": 2, "zero_stage_2": 2, "stage2": 2}
    if key not in table:
        raise ValueError(f"unsupported distributed optimizer mode {name!r}")
    return table[key]


@dataclass(frozen=True)
class NodeMemoryModel:
    hw: Hardware
    suite: ModelSuite
    workload: Workload
    eps_rt: float = 0.0
    trainable: FrozenSet[Model] = frozenset()
    shadow_models: FrozenSet[Model] = frozenset()
    optimizer_stage: int = 2
    worker_overhead_bytes: float = 0.0
    semantic_activation_cache_bytes: float = 0.0
    max_worker_groups_per_gpu: int = 0
    activation_checkpointing: bool = True
    kv_cache_budget_bytes: float = 0.0
    activation_token_cap: int = 0
    _shard_cache: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_policy(cls, hw, suite, workload, policy: MemoryPolicy, *, trainable=frozenset(), shadow_models=frozenset()):
        return cls(hw, suite, workload, eps_rt=policy.runtime_overhead_fraction, trainable=frozenset(trainable),
                   shadow_models=frozenset(shadow_models), optimizer_stage=policy.optimizer_stage,
                   worker_overhead_bytes=policy.worker_overhead_bytes,
                   semantic_activation_cache_bytes=policy.semantic_activation_cache_bytes,
                   max_worker_groups_per_gpu=policy.max_worker_groups_per_gpu,
                   activation_checkpointing=policy.activation_checkpointing,
                   kv_cache_budget_bytes=policy.kv_cache_budget_bytes, activation_token_cap=policy.activation_token_cap)

    def __post_init__(self):
        if self.optimizer_stage not in (0, 1, 2):
            raise ValueError("optimizer_stage must be 0, 1, or 2")

    # ---- capacity / single-node peak
    def capacity(self) -> float:
        return (1 - self.eps_rt) * self.hw.memory_per_gpu

    _eff_capacity = capacity

    def is_locally_feasible(self, node: ExecNode) -> bool:
        return self.peak_bytes(node) <= self.capacity()

    def peak_bytes(self, node: ExecNode) -> float:
        return self.weight_bytes(node) + self.role_extra_bytes(node, with_optimizer=True)

    def role_extra_bytes(self, node: ExecNode, with_optimizer: bool = False) -> float:
        role = node.role
        if role is Role.TRAINING:
            extra = self.gradient_bytes(node) + self.train_activation_bytes(node)
            return extra + (self.optimizer_bytes(node) if with_optimizer else 0.0)
        if role is Role.GENERATION:
            return self.kv_cache_bytes(node) + self.inference_activation_bytes(node)
        return self.inference_activation_bytes(node)

    # ---- weights
    def layer_params(self, model: Model) -> int:
        s = self.suite.specs[model]
        return 4 * s.d * s.d + 2 * s.d * s.d_ff

    def stage_params(self, model: Model, p: int, pp: int) -> Tuple[int, int]:
        """(tp-split, unsplit) parameter counts of pipeline stage ``p`` (1-based)."""
        s = self.suite.specs[model]
        emb, head = s.V * s.d, s.d
        split = math.ceil(s.L / pp) * self.layer_params(model)
        first = emb if p == 1 else 0
        if model in (Model.ACTOR, Model.REFERENCE):
            last = emb
        elif model in (Model.CRITIC, Model.REWARD):
            last = head
        elif model is Model.AC_SHARE:
            last = emb + head
        else:
            raise ValueError(model)
        return split, first + (last if p == pp else 0)

    def shard_params(self, node: ExecNode) -> int:
        key = (node.model, node.pi[1], node.pi[2])
        if key not in self._shard_cache:
            pp, tp = node.pi[1], node.pi[2]
            split, unsplit = max((self.stage_params(node.model, p, pp) for p in range(1, pp + 1)), key=lambda t: t[0] + t[1])
            self._shard_cache[key] = math.ceil(split / tp) + unsplit
        return self._shard_cache[key]

    _w_shard = shard_params

    def weight_bytes(self, node: ExecNode) -> float:
        return self.shard_params(node) * self.suite.specs[node.model].dtype_bytes

    def optimizer_bytes(self, node: ExecNode) -> float:
        dp = node.pi[0] if self.optimizer_stage >= 1 else 1
        return 12 * self.shard_params(node) / dp

    def gradient_bytes(self, node: ExecNode) -> float:
        dp = node.pi[0] if self.optimizer_stage >= 2 else 1
        return self.suite.specs[node.model].dtype_bytes * self.shard_params(node) / dp

    def train_activation_bytes(self, node: ExecNode) -> float:
        per_mb = training_activation_bytes_per_microbatch(node, self.suite, self.workload,
                                                          activation_checkpointing=self.activation_checkpointing,
                                                          token_cap=self.activation_token_cap)
        return min(node.mb, node.pi[1]) * per_mb

    def inference_activation_bytes(self, node: ExecNode) -> float:
        s, w = self.suite.specs[node.model], self.workload
        dp, _, tp = node.pi
        b_local = w.B * w.K / (dp * (node.mb if node.mb is not None else 1))
        seq = w.S if node.role is Role.GENERATION else w.S + w.T
        per_token = max(2 * s.d + 6 * s.d / tp, 2 * s.d + 2 * s.d_ff / tp, s.d + s.V)
        tokens = b_local * seq
        if self.activation_token_cap > 0:
            tokens = min(tokens, self.activation_token_cap)
        return s.dtype_bytes * tokens * per_token

    def kv_cache_bytes(self, node: ExecNode) -> float:
        s, w = self.suite.specs[node.model], self.workload
        dp, pp, tp = node.pi
        full = 2 * s.dtype_bytes * (w.B / dp) * w.K * (w.S + w.T) * (s.L / pp) * (s.d / tp)
        # A paged cache with continuous batching holds only the rows in flight: the pool is a fixed budget.
        return min(full, self.kv_cache_budget_bytes) if self.kv_cache_budget_bytes > 0 else full

    def static_bytes(self, model: Model, shard: int, trained: bool, dp: int = 1) -> float:
        sb = self.suite.specs[model].dtype_bytes
        if not trained:
            return sb * shard
        return sb * shard + 12 * shard / (dp if self.optimizer_stage >= 1 else 1) + sb * shard / (dp if self.optimizer_stage >= 2 else 1)


def _fused_activation_peak(members: List[ExecNode], mm: NodeMemoryModel) -> float:
    from ..runtime.fused_pipeline import FusedPipelineModel, build_fused_pipeline_schedule

    by_v = {m.template_id: m for m in members if m.op is not None}
    plain = sum(mm.train_activation_bytes(m) for m in members)
    if set(by_v) != {"t_pi", "t_V"}:
        return plain
    actor, critic = by_v["t_pi"], by_v["t_V"]
    if actor.pi is None or actor.mb is None or critic.pi != actor.pi or critic.mb != actor.mb:
        return plain
    pp = int(actor.pi[1])
    scale = max(float(mm.suite.n_params(actor.model)), float(mm.suite.n_params(critic.model)), 1.0)

    def mk(name, node, reverse):
        work = float(mm.suite.n_params(node.model)) / scale
        act = int(training_activation_bytes_per_microbatch(node, mm.suite, mm.workload,
                                                           activation_checkpointing=mm.activation_checkpointing))
        return FusedPipelineModel.uniform(name, pipeline_stages=pp, microbatches=int(node.mb), forward_s=work,
                                          backward_s=2.0 * work, activation_bytes=act, reverse=reverse)

    sched = build_fused_pipeline_schedule((mk("actor", actor, False), mk("critic", critic, True)))
    return float(max(sched.peak_activation_bytes, default=0))


def device_peaks(executable: ExecutableRPEG, mm: NodeMemoryModel) -> Dict[Tuple[int, int, int], float]:
    per_device: Dict[Tuple[int, int, int], List[ExecNode]] = defaultdict(list)
    ops = [n for n in executable.nodes if n.kind is ExecNodeType.OP]
    for n in ops:
        for a in n.allocs:
            for c in a.coords():
                per_device[c].append(n)
    shard = {n.id: mm.shard_params(n) for n in ops}
    wbytes = {n.id: mm.weight_bytes(n) for n in ops}
    extra = {n.id: mm.role_extra_bytes(n) for n in ops}
    groups: Dict[str, List[ExecNode]] = defaultdict(list)
    for n in ops:
        if n.fusion_group:
            groups[n.fusion_group].append(n)
    fused_peak = {g: _fused_activation_peak(ms, mm) for g, ms in groups.items()}
    liveness = len(mm.trainable) > 0
    overhead_per_worker = mm.worker_overhead_bytes + mm.semantic_activation_cache_bytes

    def wkey(n: ExecNode):
        return (n.model, n.allocs[0].origin, n.allocs[0].extent)

    def max_with_fusion(costs: Dict[str, float], nodes: List[ExecNode]) -> float:
        best, fused = 0.0, defaultdict(float)
        for n in nodes:
            if n.fusion_group:
                fused[n.fusion_group] += costs[n.id] - mm.train_activation_bytes(n)
            else:
                best = max(best, costs[n.id])
        for g in fused:
            best = max(best, fused[g] + fused_peak[g])
        return best

    peaks: Dict[Tuple[int, int, int], float] = {}
    for dev, nodes in per_device.items():
        workers = {wkey(n) for n in nodes}
        if mm.max_worker_groups_per_gpu > 0 and len(workers) > mm.max_worker_groups_per_gpu:
            peaks[dev] = math.inf
            continue
        base = len(workers) * overhead_per_worker
        if not liveness:
            info: Dict[Model, list] = {}
            for n in nodes:
                trained = n.role is Role.TRAINING
                cur = info.setdefault(n.model, [shard[n.id], trained, n.pi[0]])
                cur[0] = max(cur[0], shard[n.id])
                if trained:
                    cur[1], cur[2] = True, n.pi[0]
            static = sum(mm.static_bytes(m, s, t, dp) for m, (s, t, dp) in info.items())
            peaks[dev] = base + static + max_with_fusion(extra, nodes)
            continue
        opt: Dict[Model, Tuple[int, int]] = {}
        train_workers = defaultdict(set)
        for n in nodes:
            if n.model in mm.trainable and n.role is Role.TRAINING:
                train_workers[n.model].add(wkey(n))
        serving: Dict[tuple, int] = {}
        frozen: Dict[Model, float] = {}
        for n in nodes:
            if n.model in mm.trainable:
                if n.role is Role.TRAINING:
                    if n.model not in opt or shard[n.id] > opt[n.model][0]:
                        opt[n.model] = (shard[n.id], n.pi[0])
                elif wkey(n) not in train_workers[n.model]:
                    serving[wkey(n)] = max(serving.get(wkey(n), 0), shard[n.id])
            else:
                frozen[n.model] = max(frozen.get(n.model, 0.0), wbytes[n.id])
        persistent = sum(12 * ws / (dp if mm.optimizer_stage >= 1 else 1) for ws, dp in opt.values())
        persistent += sum(mm.suite.specs[k[0]].dtype_bytes * ws for k, ws in serving.items())
        persistent += sum(frozen.values())
        op_cost = {n.id: (extra[n.id] if (wkey(n) in serving or n.model in frozen) else wbytes[n.id] + extra[n.id])
                   for n in nodes}
        peaks[dev] = base + persistent + max_with_fusion(op_cost, nodes)
    return peaks


_device_peaks = device_peaks


def mem_feasible(executable: ExecutableRPEG, mm: NodeMemoryModel) -> bool:
    cap = mm.capacity()
    return all(p <= cap for p in device_peaks(executable, mm).values())


def mem_worst_violation(executable: ExecutableRPEG, mm: NodeMemoryModel) -> Optional[Tuple[Tuple[int, int, int], float, float]]:
    cap = mm.capacity()
    worst = None
    for dev, p in device_peaks(executable, mm).items():
        if p > cap and (worst is None or p > worst[1]):
            worst = (dev, p, cap)
    return worst
