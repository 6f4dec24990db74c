"""Plan files. Same layouts as the reference (RPEG/ir/serialize.py:63-340) so files written by
either tool load in the other:

  plain plan       ``device_space`` / ``structure`` {ac_share, intra_stage_fusion, tau, trainable,
                   transfer_resource_policy} / ``plan`` {vertex: model, role, placement, parallelism,
                   microbatch}
  optimized plan   the above plus ``schema_version: rpeg.optimized_plan.v1``, algorithm, workload,
                   ``source_config_hash`` and ``plan_hash = "sha256:" + sha256(canonical JSON of
                   everything except plan_hash)``; optionally an ``execution_schedule`` with policy
                   ``rpeg_critical_path_list_v1`` and, per node, its dispatch index and predicted
                   start/finish.
"""
from __future__ import annotations

import hashlib
import json
from typing import Optional

import yaml

from ..analytic.workload import Workload
from ..core.types import Allocation, DeviceSpace, Model, TransferResourcePolicy
from ..ir.plan import ExecutionPlan
from ..ir.rpeg import RPEG
from ..schedule.trace import Trace

SCHEMA = "rpeg.optimized_plan.v1"
SCHEDULE_POLICY = "rpeg_critical_path_list_v1"
MODEL_NAME = {Model.ACTOR: "actor", Model.CRITIC: "critic", Model.REFERENCE: "reference", Model.REWARD: "reward",
              Model.AC_SHARE: "ac_share"}
MODEL_BY_NAME = {v: k for k, v in MODEL_NAME.items()}


def _is_yaml(path: str) -> bool:
    return str(path).endswith((".yaml", ".yml"))


def _dump(d: dict, path: str) -> None:
    with open(path, "w") as f:
        if _is_yaml(path):
            yaml.dump(d, f, default_flow_style=False, sort_keys=False, allow_unicode=True)
        else:
            json.dump(d, f, indent=2)
            f.write("\n")


def _load(path: str) -> dict:
    with open(path) as f:
        return yaml.safe_load(f) if _is_yaml(path) else json.load(f)


def plan_to_dict(config) -> dict:
    rpeg, plan, ds = config.rpeg, config.plan, config.device_space
    structure = {
        "ac_share": Model.AC_SHARE in rpeg.trainable,
        "intra_stage_fusion": bool(config.intra_stage_fusion),
        "tau": {MODEL_NAME[m]: int(t) for m, t in rpeg.tau.items()},
        "trainable": [MODEL_NAME[m] for m in sorted(rpeg.trainable, key=lambda m: m.value)],
    }
    if config.transfer_resource_policy is not None:
        structure["transfer_resource_policy"] = config.transfer_resource_policy.to_dict()
    vertices = {}
    for v in rpeg.vertices:
        a, (dp, pp, tp) = plan.sigma[v.id], plan.pi[v.id]
        vertices[v.id] = {"model": MODEL_NAME[v.kind.model], "role": v.kind.role.value,
                          "placement": {"origin": list(a.origin), "extent": list(a.extent)},
                          "parallelism": {"dp": dp, "pp": pp, "tp": tp}, "microbatch": plan.mb[v.id]}
    return {"device_space": {"racks": ds.R, "nodes_per_rack": ds.N, "gpus_per_node": ds.G}, "structure": structure,
            "plan": vertices}


def plan_from_dict(d: dict, rpeg: Optional[RPEG] = None) -> ExecutionPlan:
    known = None if rpeg is None else set(rpeg.vertex_ids())
    plan = ExecutionPlan()
    for vid, info in d["plan"].items():
        if known is not None and vid not in known:
            continue
        p, par = info["placement"], info["parallelism"]
        plan.sigma[vid] = Allocation(tuple(p["origin"]), tuple(p["extent"]))
        plan.pi[vid] = (int(par["dp"]), int(par["pp"]), int(par["tp"]))
        plan.mb[vid] = int(info["microbatch"])
    return plan


def device_space_from_dict(d: dict) -> DeviceSpace:
    ds = d["device_space"]
    return DeviceSpace(int(ds["racks"]), int(ds["nodes_per_rack"]), int(ds["gpus_per_node"]))


def load_plan(path: str, rpeg: RPEG) -> ExecutionPlan:
    return plan_from_dict(_load(path), rpeg)


def save_plan(config, path: str, quiet: bool = False) -> None:
    _dump(plan_to_dict(config), path)
    if not quiet:
        print(f"  Saved plan to -> {path}")


def compute_plan_hash(d: dict) -> str:
    canonical = json.dumps({k: v for k, v in d.items() if k != "plan_hash"}, sort_keys=True, separators=(",", ":"))
    return "sha256:" + hashlib.sha256(canonical.encode()).hexdigest()


def optimized_plan_to_dict(config, algorithm: str, workload: Workload, source_config_hash: Optional[str] = None,
                           execution_schedule: Optional[dict] = None) -> dict:
    d = plan_to_dict(config)
    d.update({
        "schema_version": SCHEMA, "source_config_hash": source_config_hash, "algorithm": algorithm.lower(),
        "workload": {"batch_size": workload.B, "samples_per_prompt": workload.K, "context_length": workload.S,
                     "generation_length": workload.T,
                     "gen_quantiles": [list(q) for q in workload.gen_quantiles] if workload.gen_quantiles else None},
    })
    if execution_schedule is not None:
        d["execution_schedule"] = execution_schedule
    d["plan_hash"] = compute_plan_hash(d)
    keys = ["schema_version", "plan_hash", "source_config_hash", "algorithm", "workload", "device_space", "structure", "plan"]
    out = {k: d[k] for k in keys}
    if execution_schedule is not None:
        out["execution_schedule"] = execution_schedule
    return out


def execution_schedule_to_dict(trace: Trace, *, horizon: int) -> dict:
    if horizon < 1:
        raise ValueError("execution schedule horizon must be >= 1")
    nodes = [{"node_id": n.id, "dispatch_index": i, "predicted_start_s": float(trace.start[n]),
              "predicted_finish_s": float(trace.finish[n])} for i, n in enumerate(trace.ordered())]
    return {"policy": SCHEDULE_POLICY, "horizon": horizon, "predicted_makespan_s": float(trace.makespan()), "nodes": nodes}


def save_optimized_plan(config, path: str, algorithm: str, workload: Workload, source_config_hash: Optional[str] = None,
                        execution_schedule: Optional[dict] = None) -> dict:
    d = optimized_plan_to_dict(config, algorithm, workload, source_config_hash, execution_schedule)
    _dump(d, path)
    return d


def load_optimized_plan(path: str, verify_hash: bool = True) -> dict:
    d = _load(path)
    if d.get("schema_version") != SCHEMA:
        raise ValueError(f"optimized plan must use schema_version {SCHEMA}")
    if verify_hash and d.get("plan_hash") != compute_plan_hash(d):
        raise ValueError("optimized plan hash mismatch: the file was edited after it was written")
    return d
