"""Compile (run file + optimized plan) into everything execution needs: the rebuilt RPEG, the
lowered graph for ``training.max_steps`` iterations, worker specs, transfer specs and the validated
dispatch order, after checking that plan and run agree and that the plan is exactly executable.

Checks kept from the reference (RPEG/runtime/compiler.py:217-809):
  * run-vs-plan agreement on algorithm, workload, device space, fusion flag;
  * exactness: ``B*K % minibatch == 0``, ``B*K % dp == 0``, ``minibatch % dp == 0`` for training,
    ``G % tp == 0``, ``L % pp == 0``, allocation size ``= dp*pp*tp`` with a valid packing geometry,
    ``pp == 1 => mb == 1``, local batch divisible by the microbatch count, stale consumers disjoint
    from their trainer;
  * the saved execution schedule (if required) covers the node set, respects dependencies and never
    overlaps two nodes on a device they both reserve;
  * per-device memory under the run's memory policy.
Workers: operators of the same model on the same allocation share one worker ``wg_<first vertex>``
(one resident model instance that switches layout), everything else gets its own.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

from ..analytic.hardware import Hardware, b200_nvswitch
from ..analytic.memory import MemoryPolicy, NodeMemoryModel, mem_worst_violation, optimizer_stage
from ..analytic.models import RULE_REWARD_SPEC, ModelSpec, ModelSuite
from ..analytic.workload import Workload
from ..core.types import Allocation, DeviceSpace, Model, Role, TransferResourcePolicy, packing_geometry
from ..ir.plan import ExecutionPlan
from ..ir.serialize import MODEL_BY_NAME
from ..ir.templates import build_rpeg
from ..passes.lower import ExecNodeType, ExecutableRPEG, lower
from ..passes.transfer_resources import reserved_allocations
from ..passes.unroll import UnrolledRPEG, unroll
from ..search.evaluate import Configuration, is_compatible, stale_publication_layout_valid
from .cluster import ClusterInventory, GPURef, inventory_from_file, local_inventory, slurm_inventory
from .errors import RuntimeConfigError
from .graph import RuntimeGraph, build_runtime_graph
from .schema import OptimizedPlan, RuntimeRunConfig


@dataclass(frozen=True)
class WorkerSpec:
    worker_id: str
    vertex_id: str
    model: str
    role: str
    backend: str
    allocation: Allocation
    devices: Tuple[GPURef, ...]
    parallelism: Tuple[int, int, int]
    microbatch: int
    vertex_ids: Tuple[str, ...] = ()
    roles: Tuple[str, ...] = ()
    vertex_parallelisms: Tuple[Tuple[str, Tuple[int, int, int]], ...] = ()
    vertex_microbatches: Tuple[Tuple[str, int], ...] = ()

    @property
    def owned_vertex_ids(self) -> Tuple[str, ...]:
        return self.vertex_ids or (self.vertex_id,)

    @property
    def owns_training(self) -> bool:
        return "TRAIN" in (self.roles or (self.role,))

    def parallelism_for(self, vertex_id: str) -> Tuple[int, int, int]:
        return dict(self.vertex_parallelisms).get(vertex_id, self.parallelism)

    @property
    def has_layout_transitions(self) -> bool:
        return len({p for _, p in self.vertex_parallelisms}) > 1


@dataclass(frozen=True)
class TransferSpec:
    node_id: str
    kind: str
    label: Optional[str]
    payload_in_bytes: int
    src_allocation: Allocation
    dst_allocation: Allocation


@dataclass(frozen=True)
class CompiledRuntimePlan:
    run_config: RuntimeRunConfig
    optimized_plan: OptimizedPlan
    device_space: DeviceSpace
    model_suite: ModelSuite
    workload: Workload
    config: Configuration
    unrolled: UnrolledRPEG
    lowered: ExecutableRPEG
    inventory: ClusterInventory
    workers: Tuple[WorkerSpec, ...]
    transfers: Tuple[TransferSpec, ...]
    execution_order: Optional[Tuple[str, ...]] = None

    def checkpoint_barrier_steps(self) -> Tuple[int, ...]:
        iv = self.run_config.checkpoints.interval_steps
        return tuple(s - 1 for s in range(1, self.run_config.training.max_steps + 1) if iv > 0 and s % iv == 0)

    def runtime_graph(self) -> RuntimeGraph:
        return build_runtime_graph(self.lowered, self.workers, preferred_order=self.execution_order,
                                   transfer_resource_policy=self.config.transfer_resource_policy,
                                   checkpoint_barrier_steps=self.checkpoint_barrier_steps())

    def summary(self) -> Dict[str, Any]:
        g = self.runtime_graph()
        return {"run_id": self.run_config.run_id, "algorithm": self.run_config.algorithm.name,
                "workers": [{"worker_id": w.worker_id, "vertex_ids": list(w.owned_vertex_ids), "model": w.model,
                             "backend": w.backend, "parallelism": dict(zip(("dp", "pp", "tp"), w.parallelism)),
                             "microbatch": w.microbatch, "devices": [f"{d.hostname}:cuda:{d.local_cuda_index}" for d in w.devices],
                             "layout_transitions": w.has_layout_transitions} for w in self.workers],
                "transfers": [{"node_id": t.node_id, "kind": t.kind, "label": t.label, "payload_in_bytes": t.payload_in_bytes}
                              for t in self.transfers],
                "lowered_nodes": len(self.lowered.nodes), "lowered_edges": len(self.lowered.edges),
                "runtime_graph": {"node_count": len(g.nodes), "edge_count": len(g.edges), "counts": g.summary()["counts"],
                                  "topological_order": list(g.topological_order)}}


def _suite(run: RuntimeRunConfig) -> ModelSuite:
    def spec(m) -> ModelSpec:
        return ModelSpec(m.layers, m.hidden_dim, m.ffn_dim, m.vocab_size, 2, m.head_dim)

    actor = spec(run.models["actor"])
    specs = {Model.ACTOR: actor, Model.AC_SHARE: actor,
             Model.REFERENCE: spec(run.models["reference"]) if "reference" in run.models else actor}
    if "critic" in run.models:
        specs[Model.CRITIC] = spec(run.models["critic"])
    # a rule-based reward has no model entry; the template's reward vertex then costs (almost) nothing
    specs[Model.REWARD] = spec(run.models["reward"]) if "reward" in run.models else RULE_REWARD_SPEC
    return ModelSuite(specs)


def transfer_policy_from_runtime(run: RuntimeRunConfig) -> TransferResourcePolicy:
    """Peer-memory pushes are written by the source GPU's copy kernel into the destination's
    buffers: with ``direct_source_overlap`` the source may keep computing (destination-only
    reservation), otherwise both ends are held (reference: RPEG/runtime/transfer_policy.py:16-52)."""
    mode = "destination_only" if run.runtime.direct_source_overlap else "both_endpoints"
    return TransferResourcePolicy(weight=mode, activation=mode)


def _validate_run_vs_plan(run: RuntimeRunConfig, plan: OptimizedPlan) -> None:
    raw = plan.raw
    if plan.algorithm != run.algorithm.name:
        raise RuntimeConfigError(f"plan algorithm {plan.algorithm!r} differs from run algorithm {run.algorithm.name!r}")
    w, pw = run.workload, raw.get("workload") or {}
    mine = {"batch_size": w.batch_size, "samples_per_prompt": w.samples_per_prompt, "context_length": w.context_length,
            "generation_length": w.generation_length}
    for k, v in mine.items():
        if int(pw.get(k, -1)) != v:
            raise RuntimeConfigError(f"workload.{k}={v} differs from the plan's {pw.get(k)}")
    pq = pw.get("gen_quantiles")
    if (pq or None) != ([list(q) for q in w.gen_quantiles] if w.gen_quantiles else None):
        raise RuntimeConfigError("workload.gen_quantiles differ between run file and plan (they shape the graph)")
    ds, pds = run.device_space, raw.get("device_space") or {}
    if (ds.racks, ds.nodes_per_rack, ds.gpus_per_node) != (pds.get("racks"), pds.get("nodes_per_rack"), pds.get("gpus_per_node")):
        raise RuntimeConfigError("device_space differs between run file and plan")
    if bool((raw.get("structure") or {}).get("intra_stage_fusion", False)) != bool(run.runtime.intra_stage_fusion):
        raise RuntimeConfigError("runtime.intra_stage_fusion differs from the plan's structure.intra_stage_fusion")


def _validate_exactness(cfg: Configuration, space: DeviceSpace, suite: ModelSuite, wl: Workload, run: RuntimeRunConfig) -> None:
    rollout = wl.B * wl.K
    mini = rollout if run.algorithm.minibatch_size is None else int(run.algorithm.minibatch_size)
    if mini < 1 or rollout % mini:
        raise RuntimeConfigError(f"rollout batch B*K={rollout} must be divisible by algorithm.minibatch_size={mini}")
    for v in cfg.rpeg.vertices:
        a, (dp, pp, tp), mb = cfg.plan.sigma[v.id], cfg.plan.pi[v.id], cfg.plan.mb[v.id]
        if min(dp, pp, tp, mb) <= 0:
            raise RuntimeConfigError(f"{v.id}: dp, pp, tp and microbatch must all be > 0")
        if rollout % dp:
            raise RuntimeConfigError(f"{v.id}: rollout batch {rollout} is not divisible by dp={dp}")
        train = v.kind.role is Role.TRAINING
        if train and mini % dp:
            raise RuntimeConfigError(f"{v.id}: minibatch {mini} is not divisible by dp={dp}")
        if space.G % tp:
            raise RuntimeConfigError(f"{v.id}: GPUs per node {space.G} not divisible by tp={tp}")
        if suite.specs[v.kind.model].L % pp:
            raise RuntimeConfigError(f"{v.id}: {suite.specs[v.kind.model].L} layers not divisible by pp={pp}")
        if a.size() != dp * pp * tp or packing_geometry(dp, pp, tp, space.G) is None or not is_compatible(a, (dp, pp, tp), space):
            raise RuntimeConfigError(f"{v.id}: allocation {a} does not fit dp*pp*tp={dp * pp * tp} on this device space")
        if pp == 1 and mb != 1:
            raise RuntimeConfigError(f"{v.id}: pp=1 requires microbatch=1")
        local = (mini if train else rollout) // dp
        if pp > 1 and local % mb:
            raise RuntimeConfigError(f"{v.id}: local batch {local} not divisible by microbatch count {mb}")
    if not stale_publication_layout_valid(cfg):
        raise RuntimeConfigError("a model consumed with positive staleness must be served from devices disjoint from its trainer")


def _validated_order(run: RuntimeRunConfig, plan: OptimizedPlan, lowered: ExecutableRPEG, policy) -> Optional[Tuple[str, ...]]:
    sched = plan.schedule
    if sched is None:
        if run.runtime.require_optimized_schedule:
            raise RuntimeConfigError("runtime.require_optimized_schedule is true but the plan has no execution_schedule")
        return None
    if sched.horizon != run.training.max_steps:
        raise RuntimeConfigError(f"execution_schedule.horizon={sched.horizon} differs from training.max_steps={run.training.max_steps}")
    order = tuple(sched.order())
    want = {n.id for n in lowered.nodes}
    if set(order) != want or len(order) != len(want):
        raise RuntimeConfigError(f"execution_schedule node set mismatch: missing={sorted(want - set(order))[:10]} "
                                 f"extra={sorted(set(order) - want)[:10]}")
    t = {n["node_id"]: (float(n["predicted_start_s"]), float(n["predicted_finish_s"])) for n in sched.nodes}
    eps = 1e-9
    for e in lowered.edges:
        if t[e.src.id][1] > t[e.dst.id][0] + eps:
            raise RuntimeConfigError(f"execution_schedule violates dependency {e.src.id}->{e.dst.id}")
    by_id = {n.id: n for n in lowered.nodes}
    preds = {n.id: set() for n in lowered.nodes}
    succs = {n.id: set() for n in lowered.nodes}
    for e in lowered.edges:
        preds[e.dst.id].add(e.src.id)
        succs[e.src.id].add(e.dst.id)
    per_dev: Dict[tuple, List[tuple]] = {}
    for n in lowered.nodes:
        devs = set()
        for a in reserved_allocations(n, policy=policy, predecessors=preds, successors=succs, by_id=by_id):
            devs.update(a.coords())
        for d in devs:
            per_dev.setdefault(d, []).append((*t[n.id], n.id))
    for d, spans in per_dev.items():
        spans.sort()
        ps, pf, pid = spans[0]
        for s, f, nid in spans[1:]:
            same_group = by_id[pid].fusion_group is not None and by_id[pid].fusion_group == by_id[nid].fusion_group
            if s < pf - eps and not (same_group and abs(s - ps) <= eps and abs(f - pf) <= eps):
                raise RuntimeConfigError(f"execution_schedule overlaps {pid} and {nid} on logical GPU {d}")
            if f > pf:
                ps, pf, pid = s, f, nid
    return order


def _worker_specs(cfg: Configuration, inventory: ClusterInventory, backend: str) -> Tuple[WorkerSpec, ...]:
    groups: Dict[tuple, List] = {}
    for v in cfg.rpeg.vertices:
        a = cfg.plan.sigma[v.id]
        groups.setdefault((v.kind.model.value, a.origin, a.extent), []).append(v)
    out = []
    for (model, origin, extent), verts in groups.items():
        lead = next((v for v in verts if v.kind.role is Role.TRAINING), verts[0])
        a = cfg.plan.sigma[lead.id]
        out.append(WorkerSpec(
            worker_id=f"wg_{verts[0].id}", vertex_id=lead.id, model=model, role=lead.kind.role.value, backend=backend,
            allocation=a, devices=inventory.resolve_allocation(a), parallelism=cfg.plan.pi[lead.id], microbatch=cfg.plan.mb[lead.id],
            vertex_ids=tuple(v.id for v in verts), roles=tuple(v.kind.role.value for v in verts),
            vertex_parallelisms=tuple((v.id, cfg.plan.pi[v.id]) for v in verts),
            vertex_microbatches=tuple((v.id, cfg.plan.mb[v.id]) for v in verts)))
    return tuple(out)


def memory_policy_from_run(run: RuntimeRunConfig) -> MemoryPolicy:
    return MemoryPolicy(optimizer_stage=optimizer_stage(run.optimizer_runtime.distributed_optimizer),
                        activation_checkpointing=run.optimizer_runtime.activation_checkpointing,
                        runtime_overhead_fraction=run.hardware.memory_reserve_fraction,
                        worker_overhead_bytes=run.hardware.worker_overhead_bytes,
                        semantic_activation_cache_bytes=run.hardware.semantic_activation_cache_bytes,
                        max_worker_groups_per_gpu=run.hardware.max_worker_groups_per_gpu,
                        kv_cache_budget_bytes=float(run.hardware.kv_cache_budget_bytes),
                        activation_token_cap=int(run.hardware.activation_token_cap))


def compile_runtime_plan(run_config, *, dry_run: bool = False, inventory: Optional[ClusterInventory] = None) -> CompiledRuntimePlan:
    run = run_config if isinstance(run_config, RuntimeRunConfig) else RuntimeRunConfig.load(run_config)
    plan = OptimizedPlan.load(run.resolve(run.optimized_plan.path), run.optimized_plan.expected_hash)
    _validate_run_vs_plan(run, plan)
    suite = _suite(run)
    wl = Workload(run.workload.batch_size, run.workload.samples_per_prompt, run.workload.context_length,
                  run.workload.generation_length, run.workload.quantile_tuples())
    space = DeviceSpace(run.device_space.racks, run.device_space.nodes_per_rack, run.device_space.gpus_per_node)
    structure = plan.raw.get("structure") or {}
    tau = {MODEL_BY_NAME[k]: int(v) for k, v in (structure.get("tau") or {}).items() if k in MODEL_BY_NAME}
    algo = "ac_share" if structure.get("ac_share") else plan.algorithm
    rpeg = build_rpeg(algo, suite, wl, tau=tau or None)
    eplan = ExecutionPlan()
    for vid, pv in plan.vertices.items():
        eplan.sigma[vid], eplan.pi[vid], eplan.mb[vid] = Allocation(pv.origin, pv.extent), (pv.dp, pv.pp, pv.tp), pv.microbatch
    missing = [v.id for v in rpeg.vertices if v.id not in eplan.sigma]
    if missing:
        raise RuntimeConfigError(f"plan has no entry for vertices {missing}")
    policy = TransferResourcePolicy.from_dict(structure.get("transfer_resource_policy")) if structure.get("transfer_resource_policy") \
        else transfer_policy_from_runtime(run)
    cfg = Configuration(rpeg, eplan, space, bool(run.runtime.intra_stage_fusion), policy)
    _validate_exactness(cfg, space, suite, wl, run)
    K = run.training.max_steps
    unrolled = unroll(rpeg, K)
    lowered = lower(rpeg, unrolled, eplan, suite, K, workload=wl, intra_stage_fusion=cfg.intra_stage_fusion)
    order = _validated_order(run, plan, lowered, policy)
    if inventory is not None:
        inv = inventory
    elif run.cluster.inventory:
        inv = inventory_from_file(run.resolve(run.cluster.inventory), space)
    elif run.cluster.launcher.type == "slurm" and (os.environ.get("SLURM_JOB_NODELIST") or os.environ.get("SLURM_NODELIST")):
        inv = slurm_inventory(space)                      # inside an allocation: the hosts Slurm gave this job
    else:
        inv = local_inventory(space)
    workers = _worker_specs(cfg, inv, run.runtime.default_backend)
    hw = b200_nvswitch(mem=float(run.hardware.memory_per_gpu_bytes))
    mm = NodeMemoryModel.from_policy(hw, suite, wl, memory_policy_from_run(run), trainable=frozenset(rpeg.trainable),
                                     shadow_models=frozenset(m for m in rpeg.trainable if rpeg.tau.get(m, 0) > 0))
    bad = mem_worst_violation(lowered, mm)
    if bad is not None:
        raise RuntimeConfigError(f"plan needs {bad[1] / 1e9:.1f} GB on logical GPU {bad[0]} but only {bad[2] / 1e9:.1f} GB are usable")
    transfers = tuple(TransferSpec(n.id, n.kind.value, n.label, n.payload_in_bytes, n.allocs[0], n.allocs[-1])
                      for n in lowered.nodes if n.kind is not ExecNodeType.OP)
    return CompiledRuntimePlan(run, plan, space, suite, wl, cfg, unrolled, lowered, inv, workers, transfers, order)
