"""Job planner: one high-level YAML in, a complete plan/run pair out.

``plan_runtime_job`` builds the algorithm graph, the hardware and memory policy from the job file,
searches a plan (with a few seeds if the first attempts end infeasible), schedules the baseline and
the optimized plan at the training horizon and writes into the output directory:

  baseline_plan.yaml                       fastest per-vertex candidates, everything at origin 0
  optimized_plan.yaml                      ``rpeg.optimized_plan.v1`` with the recorded dispatch order
  plots/optimizer_{input,output}.gantt.svg predicted schedules
  metrics/analytical_comparison.json       ``rpeg.analytical_comparison.v1``
  run.yaml                                 ``rpeg.run.v1`` run file referring to the plan by hash
  submit.sh (optional)                     a torchrun launch line for the node (``--emit-launch``)

and finally compiles the pair once as a dry run, so a job that would be rejected at start-up is
rejected here. Reference: RPEG/runtime/job_plan.py:71-327 (flow), :470-530 (hardware), :607-682
(optimizer and memory policy), :685-782 (run file), :881 (CLI).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

from ..analytic.cost import NodeCostModel
from ..analytic.hardware import Hardware, b200_nvswitch
from ..analytic.memory import MemoryPolicy, NodeMemoryModel, optimizer_stage
from ..analytic.models import RULE_REWARD_SPEC, ModelSpec, ModelSuite
from ..analytic.workload import Workload
from ..core.types import DeviceSpace, Model, TransferResourcePolicy
from ..ir.serialize import execution_schedule_to_dict, load_plan, optimized_plan_to_dict, plan_to_dict
from ..ir.templates import build_rpeg
from ..passes.lower import lower
from ..passes.unroll import unroll
from ..schedule.scheduler import schedule
from ..search.cache import EvalCache
from ..search.evaluate import Configuration, evaluate_cached
from ..search.optimizer import OptimizerConfig, SearchReport, optimize, polish
from .errors import RuntimeConfigError
from .io import dump_mapping, load_mapping

COMPARISON_SCHEMA = "rpeg.analytical_comparison.v1"
PROFILE_SCHEMA = "rpeg.generation_profile.v1"
_MODEL_NAMES = {"actor": Model.ACTOR, "critic": Model.CRITIC, "reference": Model.REFERENCE, "reward": Model.REWARD,
                "ac_share": Model.AC_SHARE}


# ------------------------------------------------------------------------------ job file -> objects
def job_workload(cfg: dict, base_dir: Path) -> Workload:
    w = cfg.get("workload") or {}
    for k in ("batch_size", "context_length", "generation_length"):
        if k not in w:
            raise RuntimeConfigError(f"[workload] {k} is required")
    q = w.get("gen_quantiles")
    prof = cfg.get("generation_profile") or {}
    if q is None and prof.get("path"):
        p = Path(prof["path"])
        profile = load_mapping(p if p.is_absolute() else base_dir / p)
        if profile.get("schema_version") != PROFILE_SCHEMA:
            raise RuntimeConfigError(f"generation profile must declare schema_version: {PROFILE_SCHEMA}")
        if int(profile.get("max_new_tokens", -1)) != int(w["generation_length"]):
            raise RuntimeConfigError("generation profile max_new_tokens differs from workload.generation_length")
        q = profile.get("quantiles")
    quant = tuple((float(a), int(b)) for a, b in q) if q else None
    return Workload(int(w["batch_size"]), int(w.get("samples_per_prompt", 1)), int(w["context_length"]),
                    int(w["generation_length"]), quant)


def job_device_space(cfg: dict) -> DeviceSpace:
    ds = cfg.get("device_space") or cfg.get("hardware") or {}
    return DeviceSpace(int(ds.get("racks", 1)), int(ds.get("nodes_per_rack", 1)), int(ds.get("gpus_per_node", 1)))


def job_hardware(cfg: dict, base_dir: Optional[Path] = None) -> Hardware:
    """Three forms: ``preset: b200_nvswitch`` (measured B200 numbers, fields may be overridden), flat
    alpha/beta keys, or ``network: {intra_node, intra_rack, inter_rack}: {latency, bandwidth}``. ``file: hw.yaml``
    (a ``calibrate.py`` output or a ``cost_calibration`` fragment, relative to the job file) is laid under the keys
    written in the job file itself, so a job can be planned with this machine's measured constants.
    ``preflight: preflight.jsonl`` (the per-node lines of ``runtime.slurm_preflight``) sets ``memory_per_gpu`` to the
    smallest GPU found unless the job file gives it."""
    hw = dict(cfg.get("hardware") or {})
    names = set(Hardware.field_names())
    if hw.get("file"):
        path = Path(str(hw["file"]))
        if not path.is_absolute() and base_dir is not None:
            path = Path(base_dir) / path
        if not path.exists():
            raise RuntimeConfigError(f"[hardware] file {path} does not exist")
        measured = load_mapping(path) or {}
        hw = {**{k: v for k, v in measured.items() if k in names}, **hw}
    if hw.get("preflight") and "memory_per_gpu" not in hw and "memory_per_gpu_bytes" not in hw:
        # lines written by runtime.slurm_preflight on every node: plan with the smallest GPU that was actually found
        from .slurm_preflight import hardware_from_preflight, read_rows
        path = Path(str(hw["preflight"]))
        if not path.is_absolute() and base_dir is not None:
            path = Path(base_dir) / path
        if not path.exists():
            raise RuntimeConfigError(f"[hardware] preflight file {path} does not exist")
        ds = cfg.get("device_space") or {}
        nodes = int(ds.get("racks", 1)) * int(ds.get("nodes_per_rack", 1))
        hw["memory_per_gpu"] = float(hardware_from_preflight(read_rows(path), expected_nodes=nodes)[1])
    extra = {k: (hw[k] if k == "fabric" else float(hw[k])) for k in hw if k in names}
    if "memory_per_gpu_bytes" in hw and "memory_per_gpu" not in hw:
        extra["memory_per_gpu"] = float(hw["memory_per_gpu_bytes"])
    if str(hw.get("preset", "b200_nvswitch" if "alpha_coll_g" not in hw and "network" not in hw else "")) == "b200_nvswitch":
        return _engine_limits(b200_nvswitch().with_updates(**extra), cfg)
    if "alpha_coll_g" in hw:
        return _engine_limits(Hardware(**extra), cfg)
    net = hw.get("network") or {}
    tiers = {"g": net.get("intra_node") or {"latency": 1e-6, "bandwidth": 270e9},
             "n": net.get("intra_rack") or {"latency": 50e-6, "bandwidth": 22e9},
             "r": net.get("inter_rack") or {"latency": 100e-6, "bandwidth": 11e9}}
    kw: Dict[str, Any] = {"flops_per_gpu": 280e12, "memory_per_gpu": 80e9, "memory_bandwidth": 1.8e12}
    for t, link in tiers.items():
        for kind in ("coll", "p2p"):
            kw[f"alpha_{kind}_{t}"], kw[f"beta_{kind}_{t}"] = float(link["latency"]), 1.0 / float(link["bandwidth"])
    kw.update(extra)
    return _engine_limits(Hardware(**kw), cfg)


def _engine_limits(hw: Hardware, cfg: dict) -> Hardware:
    """Jobs for the engine backend: the generator's slot count and paged KV pool bound how many rows decode
    together; the cost model prices generation with them unless the job file set the fields itself."""
    rt, rh = cfg.get("runtime") or {}, cfg.get("runtime_hardware") or {}
    if str(rt.get("default_backend", "")) != "engine":
        return hw
    upd = {}
    if not hw.gen_max_concurrency > 0 and rt.get("gen_slots"):
        upd["gen_max_concurrency"] = float(rt["gen_slots"])
    if not hw.gen_kv_budget_bytes > 0 and float(rh.get("kv_cache_budget_bytes", 0) or 0) > 0:
        upd["gen_kv_budget_bytes"] = float(rh["kv_cache_budget_bytes"])
    return hw.with_updates(**upd) if upd else hw


def _spec(m: dict) -> ModelSpec:
    for k in ("layers", "hidden_dim", "ffn_dim", "vocab_size"):
        if k not in m:
            raise RuntimeConfigError(f"[models] {k} is required for every model with its own architecture")
    return ModelSpec(int(m["layers"]), int(m["hidden_dim"]), int(m["ffn_dim"]), int(m["vocab_size"]),
                     int(m.get("dtype_bytes", 2)), int(m.get("head_dim", 128)),
                     None if m.get("parameter_count") is None else int(m["parameter_count"]))


def job_suite(cfg: dict) -> ModelSuite:
    models = cfg.get("models") or {}
    if "actor" not in models:
        raise RuntimeConfigError("[models] an 'actor' entry is required")
    actor = _spec(models["actor"])

    def of(name: str) -> ModelSpec:
        m = models.get(name)
        return actor if m is None or str(m.get("source", "")).lower() == "actor" else _spec(m)

    specs = {Model.ACTOR: actor, Model.AC_SHARE: actor, Model.REFERENCE: of("reference")}
    if "critic" in models:
        specs[Model.CRITIC] = of("critic")
    # without an entry the reward is a rule computed on the host: the vertex stays in the graph at (almost) no cost
    specs[Model.REWARD] = of("reward") if "reward" in models else RULE_REWARD_SPEC
    return ModelSuite(specs)


def _checkpointing(value):
    """True / False, or a number in (0, 1): the fraction of the layers that are recomputed in the backward pass."""
    if isinstance(value, (int, float)) and not isinstance(value, bool):
        v = min(1.0, max(0.0, float(value)))
        return bool(v) if v in (0.0, 1.0) else v
    return bool(value)


def job_memory_policy(cfg: dict) -> MemoryPolicy:
    opt_rt, opt, rh = cfg.get("optimizer_runtime") or {}, cfg.get("optimizer") or {}, cfg.get("runtime_hardware") or {}
    return MemoryPolicy(
        optimizer_stage=optimizer_stage(str(opt_rt.get("distributed_optimizer", "zero1"))),
        activation_checkpointing=_checkpointing(opt_rt.get("activation_checkpointing", True)),
        runtime_overhead_fraction=float(opt.get("memory_reserve_fraction", rh.get("memory_reserve_fraction", 0.10))),
        worker_overhead_bytes=float(rh.get("worker_overhead_bytes", 10 * 1024 ** 3)),
        semantic_activation_cache_bytes=float(rh.get("semantic_activation_cache_bytes", 0)),
        max_worker_groups_per_gpu=int(rh.get("max_worker_groups_per_gpu", 0)),
        kv_cache_budget_bytes=float(rh.get("kv_cache_budget_bytes", 0)),
        activation_token_cap=int(rh.get("activation_token_cap", 0)))


def job_transfer_policy(cfg: dict) -> TransferResourcePolicy:
    mode = "destination_only" if bool((cfg.get("runtime") or {}).get("direct_source_overlap", False)) else "both_endpoints"
    return TransferResourcePolicy(weight=mode, activation=mode)


def job_optimizer_config(cfg: dict, algorithm: str, policy: MemoryPolicy, ac_share: bool, seed: int) -> OptimizerConfig:
    o = cfg.get("optimizer") or {}
    stale = o.get("staleness_candidates")
    tau_fixed = {k: int(v) for k, v in ((cfg.get("policy") or {}).get("tau") or {}).items()}
    t_cand: Dict[Model, set] = {}
    for name in ("actor", "critic", "ac_share"):
        if stale and name in stale:
            t_cand[_MODEL_NAMES[name]] = {int(x) for x in stale[name]}
        elif name in tau_fixed:
            t_cand[_MODEL_NAMES[name]] = {tau_fixed[name]}
        else:
            t_cand[_MODEL_NAMES[name]] = {0}
    if not ac_share:
        t_cand[Model.AC_SHARE] = set()
    if algorithm in ("grpo", "dpo"):
        t_cand = {Model.ACTOR: t_cand[Model.ACTOR]}
    structures = o.get("structural_candidates")
    return OptimizerConfig(
        K_x=int(o.get("k_x", 1)), T_max=int(o.get("t_max", 10)), E_max=int(o.get("e_max", 8)), E_struct=int(o.get("e_struct", 4)),
        T_cand=t_cand, structural_candidates=frozenset(structures) if structures else None,
        lambda_ac=float(o.get("lambda_ac", 0.15)), score_eps=float(o.get("score_eps", 1e-4)), T_init=float(o.get("t_init", 0.30)),
        T_warm=float(o.get("t_warm", 0.05)), T_min=float(o.get("t_min", 0.01)), K_elite=int(o.get("k_elite", 3)),
        stag_window=int(o.get("stag_window", 4)), alpha_pair=float(o.get("alpha_pair", 0.28)),
        max_throughput_loss=float(o.get("max_throughput_loss", 0.0)), algorithm=algorithm,
        fixed_mb=bool(o.get("fixed_mb", False)), uniform_vertex=bool(o.get("uniform_vertex", False)),
        no_polish=bool(o.get("no_polish", False)), hard_oom=bool(o.get("hard_oom", False)),
        geometric_cooling=bool(o.get("geometric_cooling", False)),
        memory_optimizer_stage=policy.optimizer_stage, memory_activation_checkpointing=policy.activation_checkpointing,
        memory_runtime_overhead_fraction=policy.runtime_overhead_fraction,
        memory_worker_overhead_bytes=policy.worker_overhead_bytes,
        memory_semantic_activation_cache_bytes=policy.semantic_activation_cache_bytes,
        memory_max_worker_groups_per_gpu=policy.max_worker_groups_per_gpu,
        memory_kv_cache_budget_bytes=policy.kv_cache_budget_bytes,
        memory_activation_token_cap=policy.activation_token_cap,
        seed=seed, workers=int(o.get("workers", 1)), verbose=bool(o.get("verbose", False)))


# ------------------------------------------------------------------------------ plans and schedules
def fastest_at_origin_baseline(rpeg, suite, workload, hw, space, policy: MemoryPolicy) -> Optional[Configuration]:
    """The optimizer's input: fastest memory-feasible candidate per vertex, all at origin (0,0,0)."""
    from ..planner.pipeline import Baselines
    return Baselines(rpeg, suite, workload, hw, space, policy).greedy()


def predicted_schedule(config: Configuration, suite, workload, hw, horizon: int, policy: MemoryPolicy):
    unrolled = unroll(config.rpeg, horizon)
    lowered = lower(config.rpeg, unrolled, config.plan, suite, horizon, workload=workload,
                    intra_stage_fusion=config.intra_stage_fusion)
    cost = NodeCostModel(hw, suite, workload, optimizer_stage=policy.optimizer_stage,
                         activation_checkpointing=policy.activation_checkpointing)
    kw = {} if config.transfer_resource_policy is None else {"transfer_resource_policy": config.transfer_resource_policy}
    return schedule(lowered, cost, config.device_space, **kw), lowered


def data_parallel_configuration(rpeg, space: DeviceSpace, suite, workload, hw, k_eval: int, policy: MemoryPolicy, fusion: bool,
                                transfer_policy, *, pipeline_train: bool = False, tp_generation: int = 0) -> Optional[Configuration]:
    """The plan families the engine backend executes, all on the whole device space: every vertex data parallel over
    all GPUs (``pi = (G, 1, 1)``), or, with ``pipeline_train``, generation and inference data parallel and every
    training vertex pipeline parallel over all GPUs (``pi = (1, G, 1)``: gradients and optimizer state of a stage
    only, weights switched back to the replicated layout after each update). The smallest microbatch count that the
    memory model accepts is taken (a pipeline needs at least as many microbatches as stages to fill)."""
    from ..core.types import Allocation, Role
    from ..ir.plan import ExecutionPlan
    from ..search.evaluate import evaluate_uncached
    g = space.num_devices()
    full = Allocation((0, 0, 0), (space.R, space.N, space.G))
    last = None
    for mb in (1, 2, 4, 8, 16, 32, 64):
        plan = ExecutionPlan()
        for v in rpeg.vertices:
            if pipeline_train and v.kind.role is Role.TRAINING:
                plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = full, (1, g, 1), max(mb, g)
            elif tp_generation and v.kind.role is Role.GENERATION:
                # groups of t GPUs decode the rows of their prompts on 1/t of the weights and KV heads each (t = G: every
                # GPU decodes the whole batch); the publication edge from the data-parallel training vertex to this one
                # is a layout switch (RESHARD node)
                t = g if tp_generation is True else int(tp_generation)
                plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = full, (g // t, 1, t), 1
            else:
                plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = full, (g, 1, 1), mb
        last = Configuration(rpeg, plan, space, fusion, transfer_policy)
        try:
            feasible = evaluate_uncached(last, suite, workload, hw, k_eval, policy)[2]
        except Exception:
            feasible = False
        if feasible:
            return last
    return None


def disaggregated_configuration(rpeg, space: DeviceSpace, suite, workload, hw, k_eval: int, policy: MemoryPolicy, fusion: bool,
                                transfer_policy, gen_gpus: Optional[int] = None) -> Optional[Configuration]:
    """Generation data parallel on the first ``gen_gpus`` GPUs of the node (default: half), every other vertex data
    parallel on the rest: the placement under which a staleness ``tau > 0`` lets generation of the next iterations overlap
    training of the current one. The engine backend executes it for GRPO (``engine.async_rl``)."""
    from ..core.types import Allocation, Role
    from ..ir.plan import ExecutionPlan
    from ..search.evaluate import evaluate_uncached
    if space.R * space.N != 1 or space.G < 2:
        raise RuntimeConfigError("[optimizer] plan_family disaggregated needs one node with at least two GPUs")
    ng = int(gen_gpus) if gen_gpus else space.G // 2
    if not 0 < ng < space.G:
        raise RuntimeConfigError(f"[optimizer] gen_gpus must be between 1 and {space.G - 1}")
    gen_alloc, rest_alloc = Allocation((0, 0, 0), (1, 1, ng)), Allocation((0, 0, ng), (1, 1, space.G - ng))
    for mb in (1, 2, 4, 8, 16, 32, 64):
        plan = ExecutionPlan()
        for v in rpeg.vertices:
            if v.kind.role is Role.GENERATION:
                plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = gen_alloc, (ng, 1, 1), mb
            else:
                plan.sigma[v.id], plan.pi[v.id], plan.mb[v.id] = rest_alloc, (space.G - ng, 1, 1), mb
        conf = Configuration(rpeg, plan, space, fusion, transfer_policy)
        try:
            if evaluate_uncached(conf, suite, workload, hw, k_eval, policy)[2]:
                return conf
        except Exception:
            continue
    return None


def validated_seed_plan(cfg: dict, base_dir: Path, rpeg, space: DeviceSpace, algorithm: str, ac_share: bool):
    """Optional ``optimizer.seed_plan_path``: must describe the same algorithm, device space,
    vertex set, staleness and structure as the job (reference: RPEG/runtime/job_plan.py:335-433)."""
    raw_path = (cfg.get("optimizer") or {}).get("seed_plan_path")
    if not raw_path:
        return None
    p = Path(raw_path)
    art = load_mapping(p if p.is_absolute() else base_dir / p)
    if art.get("algorithm") and str(art["algorithm"]).lower() != algorithm:
        raise RuntimeConfigError(f"seed plan algorithm {art.get('algorithm')!r} differs from the job's {algorithm!r}")
    if art.get("device_space") != {"racks": space.R, "nodes_per_rack": space.N, "gpus_per_node": space.G}:
        raise RuntimeConfigError("seed plan device_space differs from the job's")
    if set((art.get("plan") or {}).keys()) != {v.id for v in rpeg.vertices}:
        raise RuntimeConfigError("seed plan vertex set differs from the job's algorithm graph")
    st = art.get("structure") or {}
    if bool(st.get("ac_share", False)) != ac_share:
        raise RuntimeConfigError("seed plan ac_share differs from the job's policy")
    return load_plan(str(p if p.is_absolute() else base_dir / p), rpeg)


def _runtime_model(models: dict, name: str) -> dict:
    m = dict(models[name])
    out = {"source": "random_init" if str(m.get("source", "random_init")).lower() in ("local", "random_init", "synthetic") else m["source"],
           "dtype": m.get("dtype", "bfloat16")}
    for k in ("checkpoint_path", "layers", "hidden_dim", "ffn_dim", "vocab_size", "head_dim", "num_heads", "num_kv_heads",
              "rope_theta", "rms_eps"):
        if m.get(k) is not None:
            out[k] = m[k]
    return out


def run_config_mapping(cfg: dict, *, run_id: str, algorithm: str, workload: Workload, space: DeviceSpace, hw: Hardware,
                       policy: MemoryPolicy, plan_file: str, plan_hash: str, fusion: bool) -> dict:
    models = cfg.get("models") or {}
    out_models = {"actor": _runtime_model(models, "actor")}
    for name in ("critic", "reward", "reference"):
        m = models.get(name)
        if m is None:
            continue
        if str(m.get("source", "")).lower() == "actor":
            out_models[name] = {**out_models["actor"], **{k: v for k, v in m.items() if k not in ("source",)}}
        else:
            out_models[name] = _runtime_model(models, name)
    runtime = {"default_backend": "metadata", "trace_path": "traces/run.jsonl", "log_dir": "logs", "store_dir": "store",
               "require_optimized_schedule": True, **dict(cfg.get("runtime") or {}), "intra_stage_fusion": fusion}
    opt_rt = {"distributed_optimizer": {0: "none", 1: "zero1", 2: "zero2"}[policy.optimizer_stage],
              "activation_checkpointing": policy.activation_checkpointing, **dict(cfg.get("optimizer_runtime") or {})}
    monitoring = {"summary_path": "metrics/summary.json", "metrics_path": "metrics/metrics.prom",
                  "alert_path": "metrics/alerts.json", "dashboard_path": "metrics/dashboard.html",
                  **dict(cfg.get("monitoring") or {})}
    return {
        "schema_version": "rpeg.run.v1", "run_id": run_id,
        "optimized_plan": {"path": plan_file, "expected_hash": plan_hash, "require_exact_match": True},
        "algorithm": {"name": algorithm, **dict(cfg.get("algorithm") or {})},
        "training": {"max_steps": 1, "save_every_steps": 1, "eval_every_steps": 1, "log_every_steps": 1,
                     **dict(cfg.get("training") or {})},
        "workload": {"batch_size": workload.B, "samples_per_prompt": workload.K, "context_length": workload.S,
                     "generation_length": workload.T,
                     "gen_quantiles": [list(q) for q in workload.gen_quantiles] if workload.gen_quantiles else None},
        "models": out_models, "tokenizer": {"source": "synthetic", **dict(cfg.get("tokenizer") or {})},
        "device_space": {"racks": space.R, "nodes_per_rack": space.N, "gpus_per_node": space.G},
        "hardware": {"gpu_type": (cfg.get("hardware") or {}).get("gpu_type", "B200"),
                     "memory_per_gpu_bytes": int(hw.memory_per_gpu), "memory_reserve_fraction": policy.runtime_overhead_fraction,
                     "worker_overhead_bytes": int(policy.worker_overhead_bytes),
                     "semantic_activation_cache_bytes": int(policy.semantic_activation_cache_bytes),
                     "max_worker_groups_per_gpu": policy.max_worker_groups_per_gpu,
                     "kv_cache_budget_bytes": int(policy.kv_cache_budget_bytes),
                     "activation_token_cap": int(policy.activation_token_cap)},
        "cluster": {"scheduler": "local", "launcher": {"type": "local"}, **dict(cfg.get("cluster") or {})},
        "runtime": runtime, "data": {"synthetic": True, **dict(cfg.get("data") or {})}, "optimizer_runtime": opt_rt,
        "checkpoints": {"output_dir": "checkpoints", **dict(cfg.get("checkpoints") or {})}, "monitoring": monitoring,
    }


def launch_script(run_file: Path, space: DeviceSpace) -> str:
    return ("#!/bin/bash\n# Launches the planned job on one node: one process per GPU, rendezvous on the loopback address.\n"
            f"exec python -m torch.distributed.run --nnodes=1 --nproc-per-node {space.G} --master-addr 127.0.0.1 "
            f"--master-port 29511 -m rpeg_b200.runtime.run --config {run_file}\n")


def sbatch_script(run_file: Path, space: DeviceSpace, cfg: dict) -> str:
    """A Slurm batch file for the planned job: one task per node, each starting one process per GPU with torchrun;
    the first node of the allocation is the rendezvous host. ``slurm: {partition, account, time, job_name,
    extra: [...]}`` of the job file fills the directives (reference: RPEG/runtime/job_plan.py:240-327, which
    emits ``submit.sbatch`` for its srun launcher). Nothing is submitted."""
    sl = dict(cfg.get("slurm") or {})
    nodes = space.R * space.N
    lines = ["#!/bin/bash", f"#SBATCH --job-name={sl.get('job_name', cfg.get('run_id', 'rpeg'))}", f"#SBATCH --nodes={nodes}",
             "#SBATCH --ntasks-per-node=1", f"#SBATCH --gpus-per-node={space.G}", f"#SBATCH --time={sl.get('time', '02:00:00')}",
             f"#SBATCH --output={run_file.parent}/slurm-%j.out"]
    for key in ("partition", "account", "qos", "constraint"):
        if sl.get(key):
            lines.append(f"#SBATCH --{key}={sl[key]}")
    lines += [f"#SBATCH {x}" for x in sl.get("extra", ())]
    lines += ["", "set -euo pipefail",
              'MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)',
              "export MASTER_ADDR MASTER_PORT=${MASTER_PORT:-29511}",
              *_preflight_lines(run_file, space, nodes, sl),
              f"srun --ntasks-per-node=1 python -m torch.distributed.run --nnodes={nodes} --nproc-per-node {space.G} \\",
              '     --node-rank "$SLURM_NODEID" --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \\',
              f"     -m rpeg_b200.runtime.run --config {run_file}", ""]
    if nodes > 1:
        lines.insert(7, "# the engine backend executes plans of ONE NVSwitch node; multi-node plans run with the metadata backend only")
    return "\n".join(lines)


def _preflight_lines(run_file: Path, space: DeviceSpace, nodes: int, sl: dict) -> List[str]:
    """GPU health of every node and the cluster contract, before the ranks start (``slurm.preflight: false`` drops it);
    ``slurm.engine_validate: true`` adds the engine's smoke worker on a single-node job."""
    if not sl.get("preflight", True):
        return []
    d = run_file.parent
    lines = [f"srun --ntasks-per-node=1 python -m rpeg_b200.runtime.slurm_preflight --expected-gpus {space.G} > {d}/preflight.jsonl",
             f"python -m rpeg_b200.runtime.slurm_preflight --contract-from {d}/preflight.jsonl --contract-output {d}/cluster_contract.json "
             f"--expected-nodes {nodes}" + (" --strict" if sl.get("preflight_strict", False) else "")]
    if sl.get("engine_validate", False) and nodes == 1:
        # the engine's smoke worker on all GPUs of the node: training step, two-token PPO exercise, checkpoint round trip
        lines.append(f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {space.G} --master-addr 127.0.0.1 --master-port 29513 "
                     f"-m rpeg_b200.runtime.engine_validate --ppo-exercise --checkpoint-dir {d}/validate_ckpt --json > {d}/engine_validate.json")
    return lines


# ------------------------------------------------------------------------------ driver
def plan_runtime_job(config_path, out_dir=None, *, emit_launch: bool = False, emit_sbatch: bool = False,
                     quiet: bool = False) -> Dict[str, Any]:
    cfg_path = Path(config_path).resolve()
    cfg = load_mapping(cfg_path)
    base = cfg_path.parent
    root = Path(out_dir or cfg.get("out_dir") or cfg_path.with_suffix("")).resolve()
    for sub in ("plots", "metrics"):
        (root / sub).mkdir(parents=True, exist_ok=True)
    pol = cfg.get("policy") or {}
    algorithm = str(pol.get("algorithm") or (cfg.get("algorithm") or {}).get("name") or "ppo").lower()
    if algorithm not in ("ppo", "grpo", "dpo"):
        raise RuntimeConfigError(f"unknown algorithm {algorithm!r}")
    ac_share = bool(pol.get("ac_share", False)) and algorithm == "ppo"
    workload, space, hw, suite = job_workload(cfg, base), job_device_space(cfg), job_hardware(cfg, base), job_suite(cfg)
    policy = job_memory_policy(cfg)
    transfer_policy = job_transfer_policy(cfg)
    fusion = bool((cfg.get("runtime") or {}).get("intra_stage_fusion", False))
    tau = {_MODEL_NAMES[k]: int(v) for k, v in (pol.get("tau") or {}).items() if k in _MODEL_NAMES}
    rpeg = build_rpeg("ac_share" if ac_share else algorithm, suite, workload, tau=tau or None)
    horizon = int((cfg.get("training") or {}).get("max_steps", 1))
    seed0 = int((cfg.get("outputs") or {}).get("seed", (cfg.get("algorithm") or {}).get("seed", 0)))
    options = cfg.get("optimizer") or {}
    attempts = max(1, int(options.get("feasibility_attempts", 3)))
    k_eval = int(options.get("k_eval", 1))

    baseline = fastest_at_origin_baseline(rpeg, suite, workload, hw, space, policy)
    seed_plan = validated_seed_plan(cfg, base, rpeg, space, algorithm, ac_share)
    start_plan = seed_plan if seed_plan is not None else (baseline.plan if baseline is not None else None)
    if start_plan is None:
        raise RuntimeConfigError("no memory-feasible starting plan exists for this job on this machine")
    start = Configuration(rpeg, start_plan, space, fusion, transfer_policy)
    t0 = time.perf_counter()
    best, feasible, reports = None, False, []
    # ``optimizer.plan_family``: "search" explores placements and (dp, pp, tp) per vertex; "data_parallel" emits the
    # all-data-parallel plan (the default for engine jobs on more than one GPU); "pipeline_train" the plan with
    # pipeline-parallel training vertices, which the engine backend executes for GRPO; "engine" the better of the two;
    # "disaggregated" generation on ``optimizer.gen_gpus`` GPUs and the rest elsewhere (what ``policy.tau > 0`` needs).
    engine_job = str((cfg.get("runtime") or {}).get("default_backend", "")) == "engine"
    family = str(options.get("plan_family", "data_parallel" if engine_job and space.num_devices() > 1 else "search"))
    if family not in ("search", "data_parallel", "pipeline_train", "tp_generation", "engine", "disaggregated"):
        raise RuntimeConfigError(f"[optimizer] unknown plan_family {family!r}")
    if family == "disaggregated":
        best = disaggregated_configuration(rpeg, space, suite, workload, hw, k_eval, policy, fusion, transfer_policy,
                                           options.get("gen_gpus"))
        if best is None:
            raise RuntimeConfigError("the disaggregated plan does not fit into memory on this machine")
        feasible, attempts = True, 0
    if family in ("data_parallel", "pipeline_train", "tp_generation", "engine"):
        # "engine": whichever of the executable families fits into memory and is predicted fastest. "tp_generation":
        # generation tensor parallel over all GPUs of the node, everything else data parallel (GRPO).
        if family in ("pipeline_train", "tp_generation") and algorithm != "grpo":
            raise RuntimeConfigError(f"[optimizer] plan_family {family}: the engine backend runs it for GRPO only")
        cands = []
        kinds = (("dp", "pp", "tp") if family == "engine" else ({"data_parallel": "dp", "pipeline_train": "pp", "tp_generation": "tp"}[family],))
        for kind in kinds:
            if kind != "dp" and (algorithm != "grpo" or space.num_devices() < 2):
                continue
            # generation layout (G / t, 1, t): t = G unless optimizer.generation_tp names a divisor of G, or "auto" (the
            # default of plan_family engine) lets the cost model choose among the divisors that also divide the attention heads
            g_all = space.num_devices()
            widths = [0]
            if kind == "tp":
                want = options.get("generation_tp", "auto" if family == "engine" else g_all)
                actor_spec = suite.specs.get(Model.ACTOR) or suite.specs.get(Model.AC_SHARE)
                heads = 0 if actor_spec is None else actor_spec.d // max(1, actor_spec.d_head)
                if str(want) == "auto":
                    widths = [t for t in range(2, g_all + 1) if g_all % t == 0 and (heads == 0 or heads % t == 0)] or [g_all]
                else:
                    if int(want) < 2 or g_all % int(want):
                        raise RuntimeConfigError(f"[optimizer] generation_tp={want} must be a divisor (>= 2) of the {g_all} GPUs")
                    widths = [int(want)]
            for t in widths:
                c = data_parallel_configuration(rpeg, space, suite, workload, hw, k_eval, policy, fusion, transfer_policy,
                                                pipeline_train=kind == "pp", tp_generation=t)
                if c is not None:
                    cands.append((predicted_schedule(c, suite, workload, hw, horizon, policy)[0].makespan(), len(cands), c))
        best = min(cands)[2] if cands else None
        if best is None:
            raise RuntimeConfigError(f"no plan of family {family!r} fits into memory on this machine")
        feasible, attempts = True, 0
    for attempt in range(attempts):
        oc = job_optimizer_config(cfg, algorithm, policy, ac_share, seed0 + attempt)
        cache, rep = EvalCache(), []
        cand = optimize(start, suite, workload, hw, k_eval, oc, cache, rep)
        _, _, feasible, _ = evaluate_cached(cand, cache, suite, workload, hw, k_eval, policy)
        if feasible and not oc.no_polish:
            cand = polish(cand, suite, workload, hw, k_eval, oc, cache, ac_share=Model.AC_SHARE in cand.rpeg.trainable)
        reports.extend(rep)
        best = cand
        if feasible:
            break
    if not feasible:
        raise RuntimeConfigError(f"plan search found no memory-feasible plan in {attempts} attempt(s)")
    search_s = time.perf_counter() - t0

    from ..utils.visualize import trace_to_gantt_svg
    base_cfg = Configuration(rpeg, start_plan, space, fusion, transfer_policy)
    base_trace, _ = predicted_schedule(base_cfg, suite, workload, hw, horizon, policy)
    opt_trace, _ = predicted_schedule(best, suite, workload, hw, horizon, policy)
    dump_mapping(plan_to_dict(base_cfg), root / "baseline_plan.yaml")
    source_hash = hashlib.sha256(cfg_path.read_bytes()).hexdigest()
    plan_dict = optimized_plan_to_dict(best, algorithm, workload, source_hash,
                                       execution_schedule_to_dict(opt_trace, horizon=horizon))
    dump_mapping(plan_dict, root / "optimized_plan.yaml")
    trace_to_gantt_svg(base_trace, str(root / "plots" / "optimizer_input.gantt.svg"), space, "optimizer input")
    trace_to_gantt_svg(opt_trace, str(root / "plots" / "optimizer_output.gantt.svg"), space, "optimizer output")
    w_step = workload.B * workload.K * (workload.S + workload.T)
    run_id = str(cfg.get("run_id") or root.name)
    comparison = {
        "schema_version": COMPARISON_SCHEMA, "run_id": run_id, "algorithm": algorithm, "horizon": horizon,
        "search_wall_s": search_s, "evaluations": sum(r.evaluations for r in reports),
        "input": {"makespan_s": base_trace.makespan(), "tokens_per_s": base_trace.throughput(w_step, horizon),
                  "utilization": base_trace.utilization(), "seconds_by_kind": base_trace.seconds_by_kind(),
                  "seconds_by_vertex": base_trace.seconds_by_vertex()},
        "output": {"makespan_s": opt_trace.makespan(), "tokens_per_s": opt_trace.throughput(w_step, horizon),
                   "utilization": opt_trace.utilization(), "plan_hash": plan_dict["plan_hash"],
                   "seconds_by_kind": opt_trace.seconds_by_kind(), "seconds_by_vertex": opt_trace.seconds_by_vertex()},
        "speedup": base_trace.makespan() / opt_trace.makespan(),
    }
    (root / "metrics" / "analytical_comparison.json").write_text(json.dumps(comparison, indent=2))
    run_map = run_config_mapping(cfg, run_id=run_id, algorithm=algorithm, workload=workload, space=space, hw=hw, policy=policy,
                                 plan_file="optimized_plan.yaml", plan_hash=plan_dict["plan_hash"],
                                 fusion=bool(plan_dict.get("structure", {}).get("intra_stage_fusion", fusion)))
    dump_mapping(run_map, root / "run.yaml")
    from .compiler import compile_runtime_plan
    compiled = compile_runtime_plan(root / "run.yaml", dry_run=True)
    if emit_launch or bool((cfg.get("outputs") or {}).get("emit_launch", False)):
        (root / "submit.sh").write_text(launch_script(root / "run.yaml", space))
    if emit_sbatch or bool((cfg.get("outputs") or {}).get("emit_sbatch", False)):
        (root / "submit.sbatch").write_text(sbatch_script(root / "run.yaml", space, cfg))
    if not quiet:
        print(f"job planned in {root}: {comparison['input']['makespan_s']:.3f} s -> {comparison['output']['makespan_s']:.3f} s "
              f"({comparison['speedup']:.2f}x), plan {plan_dict['plan_hash'][:12]}, {len(compiled.lowered.nodes)} runtime nodes")
    return {"out_dir": root, "run_file": root / "run.yaml", "plan_file": root / "optimized_plan.yaml",
            "plan_hash": plan_dict["plan_hash"], "comparison": comparison, "compiled": compiled}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Plan an RPEG runtime job: search a plan and emit the plan/run pair")
    ap.add_argument("--config", required=True)
    ap.add_argument("--out-dir", default=None)
    ap.add_argument("--emit-launch", action="store_true", help="also write submit.sh (a torchrun line; nothing is launched)")
    ap.add_argument("--emit-sbatch", action="store_true", help="also write submit.sbatch (a Slurm batch file; nothing is submitted)")
    args = ap.parse_args(argv)
    try:
        plan_runtime_job(args.config, args.out_dir, emit_launch=args.emit_launch, emit_sbatch=args.emit_sbatch)
    except (RuntimeConfigError, ValueError, KeyError) as exc:
        print(f"job planning error: {exc}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
