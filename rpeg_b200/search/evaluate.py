"""Scoring of one candidate configuration: validity, the unroll -> lower -> cost -> schedule
pipeline, the soft out-of-memory penalty and the cache around it.

Semantics of the reference (RPEG/search/evaluate.py:38-442): throughput is
``K_eval * B*K*(S+T) / makespan``; a plan whose worst device exceeds capacity keeps its raw score
times ``exp(-40 * (peak/cap - 1))`` (floor 1e-12) unless hard rejection is on; a model consumed
with positive staleness must live on devices disjoint from its trainer (the old version has to
survive while the new one is produced), which is a hard constraint.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from ..analytic.cost import NodeCostModel
from ..analytic.hardware import Hardware
from ..analytic.memory import MemoryPolicy, NodeMemoryModel, mem_feasible, mem_worst_violation
from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import (Allocation, DeviceSpace, RPEG_TRANSFER_RESOURCE_POLICY, TransferResourcePolicy,
                          packing_geometry, rectangular_node_layouts)
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from ..passes.lower import lower
from ..passes.unroll import unroll
from ..schedule.scheduler import schedule
from ..schedule.trace import Trace
from .cache import EvalCache, config_hash

OOM_BETA = 40.0
ABLATION_HARD_OOM = False


@dataclass
class Configuration:
    rpeg: RPEG
    plan: ExecutionPlan
    device_space: DeviceSpace
    intra_stage_fusion: bool = False
    transfer_resource_policy: Optional[TransferResourcePolicy] = None


def is_compatible(alloc: Allocation, pi: Tuple[int, int, int], space: DeviceSpace) -> bool:
    dp, pp, tp = pi
    geom = packing_geometry(dp, pp, tp, space.G)
    if geom is None:
        return False
    g_ext, nodes = geom
    r_ext, n_ext, a_g = alloc.extent
    return a_g == g_ext and (r_ext, n_ext) in rectangular_node_layouts(nodes, space.R, space.N) and alloc.fits(space)


def allocations_overlap(a: Allocation, b: Allocation) -> bool:
    return a.overlaps(b)


def stale_publication_layout_valid(config: Configuration) -> bool:
    for e in config.rpeg.pub_edges:
        if int(config.rpeg.tau.get(e.src.kind.model, 0)) > 0 and config.plan.sigma[e.src.id].overlaps(config.plan.sigma[e.dst.id]):
            return False
    return True


def fusion_pair_valid(config: Configuration) -> bool:
    plan = config.plan
    if "t_pi" not in plan.sigma or "t_V" not in plan.sigma:
        return False
    return (plan.sigma["t_pi"] == plan.sigma["t_V"] and plan.pi["t_pi"] == plan.pi["t_V"]
            and plan.mb["t_pi"] == plan.mb["t_V"] and plan.pi["t_pi"][1] > 1 and plan.mb["t_pi"] >= plan.pi["t_pi"][1])


def is_valid(config: Configuration, suite: ModelSuite, workload: Workload, mem_model: NodeMemoryModel) -> bool:
    plan, space = config.plan, config.device_space
    for v in config.rpeg.vertices:
        if v.id not in plan.sigma or v.id not in plan.pi or v.id not in plan.mb:
            return False
        dp, pp, tp = plan.pi[v.id]
        mb = plan.mb[v.id]
        if workload.B % dp or space.G % tp or suite.specs[v.kind.model].L % pp:
            return False
        if pp == 1:
            if mb != 1:
                return False
        elif (workload.B // dp) % mb:
            return False
        if not is_compatible(plan.sigma[v.id], (dp, pp, tp), space):
            return False
    if not stale_publication_layout_valid(config):
        return False
    if config.intra_stage_fusion and not fusion_pair_valid(config):
        return False
    try:
        lowered = lower(config.rpeg, unroll(config.rpeg, 1), plan, suite, 1, workload=workload,
                        intra_stage_fusion=config.intra_stage_fusion)
    except (KeyError, ValueError):
        return False
    return mem_feasible(lowered, mem_model)


def evaluate(config: Configuration, suite: ModelSuite, workload: Workload, hw: Hardware, K_eval: int,
             memory_policy: MemoryPolicy = MemoryPolicy()):
    """Returns ``(throughput, trace, lowered graph)``."""
    lowered = lower(config.rpeg, unroll(config.rpeg, K_eval), config.plan, suite, K_eval, workload=workload,
                    intra_stage_fusion=config.intra_stage_fusion)
    cm = NodeCostModel(hw, suite, workload, optimizer_stage=memory_policy.optimizer_stage,
                       activation_checkpointing=memory_policy.activation_checkpointing)
    trace = schedule(lowered, cm, config.device_space,
                     transfer_resource_policy=config.transfer_resource_policy or RPEG_TRANSFER_RESOURCE_POLICY)
    score = trace.throughput(W_step=workload.B * workload.K * (workload.S + workload.T), K=K_eval)
    return score, trace, lowered


def memory_model_for(config: Configuration, suite, workload, hw, policy: MemoryPolicy) -> NodeMemoryModel:
    return NodeMemoryModel.from_policy(hw, suite, workload, policy, trainable=frozenset(config.rpeg.trainable),
                                       shadow_models=frozenset(m for m in config.rpeg.trainable if config.rpeg.tau.get(m, 0) > 0))


def evaluation_cache_key(config: Configuration, policy: MemoryPolicy = MemoryPolicy()) -> str:
    tp = (config.transfer_resource_policy or RPEG_TRANSFER_RESOURCE_POLICY).to_dict()
    return (f"{config_hash(config.rpeg, config.plan)}:mem:fusion={int(config.intra_stage_fusion)}:"
            f"transfer={','.join(tp.values())}:{policy.optimizer_stage}:{int(policy.activation_checkpointing)}:"
            f"{policy.runtime_overhead_fraction:.12g}:{policy.worker_overhead_bytes:.12g}:"
            f"activation_cache={policy.semantic_activation_cache_bytes:.12g}:groups={policy.max_worker_groups_per_gpu}"
            + (f":kv={policy.kv_cache_budget_bytes:.12g}:tok={policy.activation_token_cap}"
               if (policy.kv_cache_budget_bytes or policy.activation_token_cap) else ""))


def _penalised(raw: float, lowered, mem_model: NodeMemoryModel) -> Tuple[float, bool]:
    violation = mem_worst_violation(lowered, mem_model)
    if violation is None:
        return raw, True
    if ABLATION_HARD_OOM:
        return 0.0, False
    _, need, cap = violation
    return raw * max(math.exp(-OOM_BETA * max(0.0, need / cap - 1.0)), 1e-12), False


def evaluate_uncached(config, suite, workload, hw, K_eval, policy: MemoryPolicy = MemoryPolicy()) -> Tuple[float, Trace, bool]:
    raw, trace, lowered = evaluate(config, suite, workload, hw, K_eval, policy)
    if not stale_publication_layout_valid(config):
        return 0.0, trace, False
    score, feasible = _penalised(raw, lowered, memory_model_for(config, suite, workload, hw, policy))
    return score, trace, feasible


def evaluate_cached(config, cache: EvalCache, suite, workload, hw, K_eval, memory_policy: MemoryPolicy = MemoryPolicy()):
    """Returns ``(score, trace, feasible, was_miss)``."""
    key = evaluation_cache_key(config, memory_policy)
    if key in cache:
        score, trace, feasible = cache.get(key)
        return score, trace, feasible, False
    score, trace, feasible = evaluate_uncached(config, suite, workload, hw, K_eval, memory_policy)
    cache.put(key, score, trace, feasible)
    return score, trace, feasible, True


def eval_worker(args):
    """Pool worker: pure function of its arguments (no cache, no RNG)."""
    config, suite, workload, hw, K_eval = args[:5]
    policy = args[5] if len(args) > 5 and args[5] is not None else MemoryPolicy()
    return evaluate_uncached(config, suite, workload, hw, K_eval, policy)
