"""Strict run configuration ``rpeg.run.v1`` and the optimized-plan wrapper.

Every section is a dataclass built by ``from_mapping`` which rejects unknown keys and bad values with
``RuntimeConfigError``; the optimized plan is re-hashed on load. Section and field names follow the
reference (RPEG/runtime/schema.py:117-932, RPEG/runtime/configuration.md:35-51). Options that
select transports the reference needs between worker processes (TCP, UCX, Gloo, files) are accepted
for compatibility and normalised to the single NVLink peer-memory path this runtime has.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..ir.serialize import SCHEMA as PLAN_SCHEMA, compute_plan_hash
from .errors import RuntimeConfigError
from .io import load_mapping

RUN_SCHEMA = "rpeg.run.v1"
ALGORITHMS = ("ppo", "grpo", "dpo")
BACKENDS = ("metadata", "engine", "torch_ppo", "torch_dpo", "megatron")
ACTIVATION_TRANSPORTS = ("auto", "peer_memory", "tcp_direct", "torch_dist", "gloo_direct", "nccl_direct", "ucx_direct",
                         "kernel", "stream", "copy")
WEIGHT_TRANSPORTS = ("auto", "peer_memory", "torch_dist", "gloo_direct", "nccl_direct", "ucx_direct")
DIST_OPTIMIZERS = ("none", "zero1", "zero2")


def _build(cls, raw: Optional[Mapping[str, Any]], section: str):
    raw = dict(raw or {})
    known = {f.name for f in fields(cls)}
    unknown = sorted(set(raw) - known)
    if unknown:
        raise RuntimeConfigError(f"[{section}] unknown keys: {unknown}")
    try:
        obj = cls(**raw)
    except TypeError as exc:
        raise RuntimeConfigError(f"[{section}] {exc}") from None
    if hasattr(obj, "validate"):
        obj.validate()
    return obj


def _choice(value, options, what):
    if value not in options:
        raise RuntimeConfigError(f"{what} must be one of {list(options)}, got {value!r}")


@dataclass
class AlgorithmConfig:
    name: str = "ppo"
    beta: float = 0.1
    kl_coef: float = 0.0
    clip: float = 0.2
    gamma: float = 1.0
    gae_lambda: float = 0.95
    value_coef: float = 0.5
    entropy_coef: float = 0.0
    epochs: int = 1
    minibatch_size: Optional[int] = None
    normalize_advantages: bool = True
    seed: int = 1234
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    greedy: bool = False
    generation_backend: str = "static_kv"

    def validate(self):
        _choice(self.name, ALGORITHMS, "algorithm.name")
        _choice(self.generation_backend, ("static_kv", "full_sequence", "paged_kv"), "algorithm.generation_backend")
        if self.epochs < 1 or self.clip <= 0 or not 0 < self.top_p <= 1 or self.temperature <= 0:
            raise RuntimeConfigError("[algorithm] epochs >= 1, clip > 0, 0 < top_p <= 1, temperature > 0 required")


@dataclass
class TrainingConfig:
    max_steps: int = 1
    save_every_steps: int = 1
    eval_every_steps: int = 1
    log_every_steps: int = 1

    def validate(self):
        if self.max_steps < 1:
            raise RuntimeConfigError("[training] max_steps must be >= 1")


@dataclass
class WorkloadConfig:
    batch_size: int = 0
    samples_per_prompt: int = 1
    context_length: int = 0
    generation_length: int = 0
    gen_quantiles: Optional[List[List[float]]] = None

    def validate(self):
        if min(self.batch_size, self.samples_per_prompt, self.context_length, self.generation_length) < 1:
            raise RuntimeConfigError("[workload] batch_size, samples_per_prompt, context_length, generation_length must be >= 1")
        if self.gen_quantiles:
            prev_f, prev_t = 0.0, 0
            for q in self.gen_quantiles:
                if len(q) != 2:
                    raise RuntimeConfigError("[workload.gen_quantiles] entries are [fraction, tokens]")
                f, t = float(q[0]), int(q[1])
                if not (prev_f < f <= 1.0) or not (prev_t < t <= self.generation_length):
                    raise RuntimeConfigError("[workload.gen_quantiles] fractions and lengths must strictly increase within bounds")
                prev_f, prev_t = f, t
            if abs(prev_f - 1.0) > 1e-9:
                raise RuntimeConfigError("[workload.gen_quantiles] the last fraction must be 1.0")

    def quantile_tuples(self) -> Optional[Tuple[Tuple[float, int], ...]]:
        return tuple((float(a), int(b)) for a, b in self.gen_quantiles) if self.gen_quantiles else None


@dataclass
class RuntimeModelConfig:
    source: str = "random_init"          # random_init | checkpoint
    checkpoint_path: Optional[str] = None
    dtype: str = "bfloat16"
    layers: int = 0
    hidden_dim: int = 0
    ffn_dim: int = 0
    vocab_size: int = 0
    head_dim: int = 128
    num_heads: Optional[int] = None
    num_kv_heads: Optional[int] = None
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5

    def validate(self):
        _choice(self.source, ("random_init", "checkpoint", "hf"), "models.*.source")
        _choice(self.dtype, ("bfloat16", "bf16"), "models.*.dtype")
        if min(self.layers, self.hidden_dim, self.ffn_dim, self.vocab_size) < 1:
            raise RuntimeConfigError("[models] layers, hidden_dim, ffn_dim, vocab_size must be >= 1")
        if self.source != "random_init" and not self.checkpoint_path:
            raise RuntimeConfigError("[models] checkpoint_path is required unless source is random_init")


@dataclass
class TokenizerConfig:
    source: str = "synthetic"
    path: Optional[str] = None
    eos_token_id: int = 2
    pad_token_id: int = 0


@dataclass
class DeviceSpaceConfig:
    racks: int = 1
    nodes_per_rack: int = 1
    gpus_per_node: int = 1

    def validate(self):
        if min(self.racks, self.nodes_per_rack, self.gpus_per_node) < 1:
            raise RuntimeConfigError("[device_space] all extents must be >= 1")


@dataclass
class HardwareConfig:
    gpu_type: str = "B200"
    memory_per_gpu_bytes: int = 180_000_000_000
    worker_overhead_bytes: int = 0
    semantic_activation_cache_bytes: int = 0
    max_worker_groups_per_gpu: int = 0
    kv_cache_budget_bytes: int = 0
    activation_token_cap: int = 0
    memory_reserve_fraction: float = 0.10
    calibration_path: Optional[str] = None

    def validate(self):
        if self.memory_per_gpu_bytes <= 0 or not 0 <= self.memory_reserve_fraction < 1:
            raise RuntimeConfigError("[hardware] memory_per_gpu_bytes > 0 and 0 <= memory_reserve_fraction < 1 required")


@dataclass
class LauncherConfig:
    type: str = "local"
    shared_step: bool = False
    mpi: Optional[str] = None
    ready_timeout_s: float = 120.0

    def validate(self):
        _choice(self.type, ("local", "slurm", "torchrun"), "cluster.launcher.type")


@dataclass
class ClusterConfig:
    scheduler: str = "local"
    launcher: LauncherConfig = field(default_factory=LauncherConfig)
    inventory: Optional[str] = None


@dataclass
class RuntimeConfig:
    default_backend: str = "metadata"
    intra_stage_fusion: bool = False
    dry_run: bool = False
    log_dir: str = "logs"
    store_dir: str = "store"
    trace_path: str = "traces/run.jsonl"
    activation_transport: str = "auto"
    activation_store: str = "auto"
    weight_transport: str = "auto"
    direct_channel_reuse: bool = True
    direct_source_overlap: bool = False
    semantic_control_transport: str = "tcp"
    semantic_weight_keep_latest: int = 8
    require_optimized_schedule: bool = True
    critic_pipeline_device_order: str = "reverse"
    fusion_sync_backend: str = "stream_events"
    node_timeout_s: float = 600.0
    gen_slots: int = 64
    micro_tokens: int = 16384
    recompute: str = "full"
    use_cuda_graphs: bool = True

    def validate(self):
        _choice(self.default_backend, BACKENDS, "runtime.default_backend")
        _choice(self.activation_transport, ACTIVATION_TRANSPORTS, "runtime.activation_transport")
        _choice(self.weight_transport, WEIGHT_TRANSPORTS, "runtime.weight_transport")
        _choice(self.activation_store, ("auto", "memory", "filesystem", "hybrid"), "runtime.activation_store")
        _choice(self.semantic_control_transport, ("tcp", "file", "inproc"), "runtime.semantic_control_transport")
        _choice(self.fusion_sync_backend, ("stream_events", "cuda_ipc", "filesystem"), "runtime.fusion_sync_backend")
        _choice(self.recompute, ("full", "none"), "runtime.recompute")
        if self.semantic_weight_keep_latest < 1 or self.node_timeout_s <= 0:
            raise RuntimeConfigError("[runtime] semantic_weight_keep_latest >= 1 and node_timeout_s > 0 required")

    def effective_transports(self) -> Tuple[str, str]:
        """All tensor movement between GPUs of the node goes through peer memory."""
        return "peer_memory", "peer_memory"


@dataclass
class DataConfig:
    train_prompts: Optional[str] = None
    preferences: Optional[str] = None
    synthetic: bool = True
    data_seed: int = 0
    shuffle: bool = False
    # "cap": synthetic rows generate until EOS or the length cap (random weights: the cap); "quantiles": every row is
    # ended at a length drawn from workload.gen_quantiles, the distribution the planner assumes
    synthetic_response_lengths: str = "cap"

    def validate(self):
        _choice(self.synthetic_response_lengths, ("cap", "quantiles"), "data.synthetic_response_lengths")


@dataclass
class OptimizerRuntimeConfig:
    learning_rate_actor: float = 1e-6
    learning_rate_critic: float = 5e-6
    weight_decay: float = 0.0
    grad_clip: float = 1.0
    activation_checkpointing: bool = True
    distributed_optimizer: str = "zero1"
    zero2_bucket_bytes: int = 64 * 1024 * 1024
    zero2_max_inflight_buckets: int = 2
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8

    def validate(self):
        _choice(self.distributed_optimizer, DIST_OPTIMIZERS, "optimizer_runtime.distributed_optimizer")
        if self.learning_rate_actor <= 0 or self.learning_rate_critic <= 0 or self.grad_clip < 0:
            raise RuntimeConfigError("[optimizer_runtime] learning rates must be > 0 and grad_clip >= 0")


@dataclass
class CheckpointConfig:
    output_dir: str = "checkpoints"
    interval_steps: int = 100
    resume_from: Optional[str] = None
    keep_last_interval_steps: Optional[int] = None
    save_final: bool = True
    portable_weight_versions: bool = True
    format: str = "flat_shards"

    def validate(self):
        if self.interval_steps < 1:
            raise RuntimeConfigError("[checkpoints] interval_steps must be >= 1")


@dataclass
class MonitoringConfig:
    summary_path: Optional[str] = None
    metrics_path: Optional[str] = None
    alert_path: Optional[str] = None
    dashboard_path: Optional[str] = None
    alert_rules: Dict[str, Any] = field(default_factory=dict)
    graph_replay_retries: int = 0
    worker_ready_timeout_s: float = 120.0
    operation_timeout_s: float = 600.0
    test_inject_failure_after_checkpoint_step: Optional[int] = None
    test_inject_failure_attempt: int = 0
    test_inject_failure_node_contains: Optional[str] = None

    def validate(self):
        if self.graph_replay_retries < 0:
            raise RuntimeConfigError("[monitoring] graph_replay_retries must be >= 0")


@dataclass
class OptimizedPlanRef:
    path: str = ""
    expected_hash: Optional[str] = None
    require_exact_match: bool = True


@dataclass
class RuntimeRunConfig:
    run_id: str
    optimized_plan: OptimizedPlanRef
    algorithm: AlgorithmConfig
    training: TrainingConfig
    workload: WorkloadConfig
    models: Dict[str, RuntimeModelConfig]
    tokenizer: TokenizerConfig
    device_space: DeviceSpaceConfig
    hardware: HardwareConfig
    cluster: ClusterConfig
    runtime: RuntimeConfig
    data: DataConfig
    optimizer_runtime: OptimizerRuntimeConfig
    checkpoints: CheckpointConfig
    monitoring: MonitoringConfig
    base_dir: Path = field(default_factory=Path)

    SECTIONS = ("schema_version", "run_id", "optimized_plan", "algorithm", "training", "workload", "models", "tokenizer",
                "device_space", "hardware", "cluster", "runtime", "data", "optimizer_runtime", "checkpoints", "monitoring")

    @classmethod
    def from_mapping(cls, raw: Mapping[str, Any], base_dir=".") -> "RuntimeRunConfig":
        if raw.get("schema_version") != RUN_SCHEMA:
            raise RuntimeConfigError(f"run file must declare schema_version: {RUN_SCHEMA}")
        unknown = sorted(set(raw) - set(cls.SECTIONS))
        if unknown:
            raise RuntimeConfigError(f"unknown top-level sections: {unknown}")
        cluster_raw = dict(raw.get("cluster") or {})
        launcher = _build(LauncherConfig, cluster_raw.pop("launcher", None), "cluster.launcher")
        cluster = _build(ClusterConfig, {**cluster_raw, "launcher": launcher}, "cluster")
        models_raw = raw.get("models") or {}
        if "actor" not in models_raw:
            raise RuntimeConfigError("[models] an 'actor' entry is required")
        models = {name: _build(RuntimeModelConfig, m, f"models.{name}") for name, m in models_raw.items()}
        cfg = cls(
            run_id=str(raw.get("run_id") or "run"),
            optimized_plan=_build(OptimizedPlanRef, raw.get("optimized_plan"), "optimized_plan"),
            algorithm=_build(AlgorithmConfig, raw.get("algorithm"), "algorithm"),
            training=_build(TrainingConfig, raw.get("training"), "training"),
            workload=_build(WorkloadConfig, raw.get("workload"), "workload"),
            models=models, tokenizer=_build(TokenizerConfig, raw.get("tokenizer"), "tokenizer"),
            device_space=_build(DeviceSpaceConfig, raw.get("device_space"), "device_space"),
            hardware=_build(HardwareConfig, raw.get("hardware"), "hardware"), cluster=cluster,
            runtime=_build(RuntimeConfig, raw.get("runtime"), "runtime"), data=_build(DataConfig, raw.get("data"), "data"),
            optimizer_runtime=_build(OptimizerRuntimeConfig, raw.get("optimizer_runtime"), "optimizer_runtime"),
            checkpoints=_build(CheckpointConfig, raw.get("checkpoints"), "checkpoints"),
            monitoring=_build(MonitoringConfig, raw.get("monitoring"), "monitoring"), base_dir=Path(base_dir))
        if not cfg.optimized_plan.path:
            raise RuntimeConfigError("[optimized_plan] path is required")
        need = {"ppo": ("actor", "critic", "reward"), "grpo": ("actor",), "dpo": ("actor",)}[cfg.algorithm.name]
        for name in need:
            if name not in cfg.models:
                raise RuntimeConfigError(f"[models] algorithm {cfg.algorithm.name} needs a '{name}' model")
        return cfg

    @classmethod
    def load(cls, path) -> "RuntimeRunConfig":
        p = Path(path)
        return cls.from_mapping(load_mapping(p), base_dir=p.parent)

    def resolve(self, rel: str) -> Path:
        p = Path(rel)
        return p if p.is_absolute() else self.base_dir / p


@dataclass
class PlanVertex:
    vertex_id: str
    model: str
    role: str
    origin: Tuple[int, int, int]
    extent: Tuple[int, int, int]
    dp: int
    pp: int
    tp: int
    microbatch: int


@dataclass
class OptimizedExecutionSchedule:
    policy: str
    horizon: int
    predicted_makespan_s: float
    nodes: List[dict]

    def order(self) -> List[str]:
        return [n["node_id"] for n in sorted(self.nodes, key=lambda n: n["dispatch_index"])]


@dataclass
class OptimizedPlan:
    raw: dict
    plan_hash: str
    algorithm: str
    vertices: Dict[str, PlanVertex]
    schedule: Optional[OptimizedExecutionSchedule]

    @classmethod
    def from_mapping(cls, raw: Mapping[str, Any], expected_hash: Optional[str] = None) -> "OptimizedPlan":
        if raw.get("schema_version") != PLAN_SCHEMA:
            raise RuntimeConfigError(f"optimized plan must declare schema_version: {PLAN_SCHEMA}")
        actual = compute_plan_hash(dict(raw))
        if raw.get("plan_hash") != actual:
            raise RuntimeConfigError("optimized plan hash mismatch: file content does not match its plan_hash")
        if expected_hash and expected_hash != actual:
            raise RuntimeConfigError(f"optimized plan hash {actual} differs from the run file's expected_hash {expected_hash}")
        verts = {}
        for vid, info in (raw.get("plan") or {}).items():
            try:
                p, par = info["placement"], info["parallelism"]
                verts[vid] = PlanVertex(vid, info["model"], info["role"], tuple(p["origin"]), tuple(p["extent"]),
                                        int(par["dp"]), int(par["pp"]), int(par["tp"]), int(info["microbatch"]))
            except (KeyError, TypeError) as exc:
                raise RuntimeConfigError(f"[plan.{vid}] malformed entry: {exc}") from None
        sched = None
        s = raw.get("execution_schedule")
        if s is not None:
            if s.get("policy") != "rpeg_critical_path_list_v1":
                raise RuntimeConfigError(f"unsupported execution schedule policy {s.get('policy')!r}")
            sched = OptimizedExecutionSchedule(s["policy"], int(s["horizon"]), float(s["predicted_makespan_s"]), list(s["nodes"]))
        return cls(dict(raw), actual, str(raw.get("algorithm", "ppo")), verts, sched)

    @classmethod
    def load(cls, path, expected_hash: Optional[str] = None) -> "OptimizedPlan":
        return cls.from_mapping(load_mapping(path), expected_hash)
