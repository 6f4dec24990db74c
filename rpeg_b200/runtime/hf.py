"""Hugging Face helpers that need no network: locating a local snapshot, reading ``config.json`` into
the planner's ``ModelSpec``, counting parameters from safetensors headers without loading tensors, and
importing / exporting weights between the safetensors naming and this engine's flat layout.

Remote repositories must be pinned to a 40-character commit hash; nothing is downloaded here (local
paths only), so a repo id without a local ``checkpoint_path`` is a configuration error.
Reference: RPEG/runtime/hf.py:26-170; the weight import replaces the reference's HF -> Megatron name
mapping with TP slicing (RPEG/runtime/workers/megatron_worker.py:4807-4964).
"""
from __future__ import annotations

import json
import re
import struct
from pathlib import Path
from typing import Any, Dict, Iterable, Optional, Tuple

from ..analytic.models import ModelSpec
from .errors import RuntimeConfigError

_COMMIT = re.compile(r"^[0-9a-f]{40}$")


def require_pinned_revision(repo: str, revision: Optional[str]) -> str:
    if not revision or not _COMMIT.fullmatch(str(revision)):
        raise RuntimeConfigError(f"model {repo!r} needs a 40-character commit hash as revision, got {revision!r} "
                                 "(branches and tags move)")
    return str(revision)


def resolve_model_path(source: str, repo: Optional[str] = None, checkpoint_path: Optional[str] = None,
                       revision: Optional[str] = None) -> Path:
    """``source`` is ``local`` / ``checkpoint`` (use ``checkpoint_path``) or ``hf`` (a pinned repo whose
    snapshot must already be on disk at ``checkpoint_path``)."""
    if source in ("hf", "huggingface"):
        require_pinned_revision(repo or "?", revision)
    if not checkpoint_path:
        raise RuntimeConfigError(f"model source {source!r} needs checkpoint_path: snapshots are not downloaded by the runtime")
    p = Path(checkpoint_path)
    if not p.exists():
        raise RuntimeConfigError(f"model path {p} does not exist")
    return p


def load_hf_config(model_dir) -> Dict[str, Any]:
    p = Path(model_dir) / "config.json"
    if not p.exists():
        raise RuntimeConfigError(f"{p} not found")
    return json.loads(p.read_text())


def model_spec_from_hf_config(cfg: Dict[str, Any], parameter_count: Optional[int] = None) -> ModelSpec:
    hidden, heads = int(cfg["hidden_size"]), int(cfg["num_attention_heads"])
    return ModelSpec(int(cfg["num_hidden_layers"]), hidden, int(cfg["intermediate_size"]), int(cfg["vocab_size"]), 2,
                     int(cfg.get("head_dim") or hidden // heads), parameter_count)


def safetensors_header(path) -> Dict[str, Any]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n <= 0 or n > 100 * 1024 * 1024:
            raise RuntimeConfigError(f"{path}: implausible safetensors header length {n}")
        return json.loads(f.read(n))


def safetensors_parameter_count(model_dir) -> int:
    """Sum of tensor sizes over all ``*.safetensors`` files, read from the headers only."""
    total = 0
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise RuntimeConfigError(f"no safetensors files in {model_dir}")
    for f in files:
        for name, meta in safetensors_header(f).items():
            if name == "__metadata__":
                continue
            n = 1
            for s in meta["shape"]:
                n *= int(s)
            total += n
    return total


def infer_model_spec(model_dir) -> ModelSpec:
    cfg = load_hf_config(model_dir)
    try:
        count = safetensors_parameter_count(model_dir)
    except RuntimeConfigError:
        count = None
    return model_spec_from_hf_config(cfg, count)


# ------------------------------------------------------------------------------ weights
def _hf_names(cfg, i: int) -> Dict[str, str]:
    pre = f"model.layers.{i}."
    out = {"attn_norm": pre + "input_layernorm.weight", "q": pre + "self_attn.q_proj.weight", "k": pre + "self_attn.k_proj.weight",
           "v": pre + "self_attn.v_proj.weight", "wo": pre + "self_attn.o_proj.weight", "mlp_norm": pre + "post_attention_layernorm.weight",
           "gate": pre + "mlp.gate_proj.weight", "up": pre + "mlp.up_proj.weight", "w_down": pre + "mlp.down_proj.weight"}
    if cfg.qk_norm:
        out.update(q_norm=pre + "self_attn.q_norm.weight", k_norm=pre + "self_attn.k_norm.weight")
    return out


def _open_shards(model_dir):
    from safetensors import safe_open
    index: Dict[str, Any] = {}
    for f in sorted(Path(model_dir).glob("*.safetensors")):
        h = safe_open(str(f), framework="pt", device="cpu")
        for k in h.keys():
            index[k] = h
    if not index:
        raise RuntimeConfigError(f"no safetensors files in {model_dir}")
    return index


def load_hf_weights(model, model_dir) -> int:
    """Copy a Hugging Face checkpoint (llama / qwen3 naming) into ``model``'s flat bf16 buffer: q, k, v
    projections are stacked into ``wqkv`` and gate, up into ``w_gate_up``. The rotary convention is the
    same rotate-half pairing as Hugging Face uses, so no permutation is needed. Returns the number of
    parameters copied."""
    import torch
    cfg = model.cfg
    idx = _open_shards(model_dir)

    def get(name: str):
        if name not in idx:
            raise RuntimeConfigError(f"tensor {name} is missing from {model_dir}")
        return idx[name].get_tensor(name)

    copied = 0

    def put(dst, src) -> None:
        nonlocal copied
        if tuple(dst.shape) != tuple(src.shape):
            raise RuntimeConfigError(f"shape mismatch: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
        dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
        copied += src.numel()

    put(model.p["embed"], get("model.embed_tokens.weight"))
    for i in range(cfg.n_layers):
        n = _hf_names(cfg, i)
        put(model.p[f"l{i}.attn_norm"], get(n["attn_norm"]))
        put(model.p[f"l{i}.wqkv"], torch.cat([get(n["q"]), get(n["k"]), get(n["v"])], 0))
        put(model.p[f"l{i}.wo"], get(n["wo"]))
        put(model.p[f"l{i}.mlp_norm"], get(n["mlp_norm"]))
        put(model.p[f"l{i}.w_gate_up"], torch.cat([get(n["gate"]), get(n["up"])], 0))
        put(model.p[f"l{i}.w_down"], get(n["w_down"]))
        if cfg.qk_norm:
            put(model.p[f"l{i}.q_norm"], get(n["q_norm"]))
            put(model.p[f"l{i}.k_norm"], get(n["k_norm"]))
    put(model.p["final_norm"], get("model.norm.weight"))
    if cfg.lm_head and not cfg.tie_embeddings:
        put(model.p["lm_head"], get("lm_head.weight" if "lm_head.weight" in idx else "model.embed_tokens.weight"))
    return copied


def save_hf_weights(model, model_dir, shard_bytes: int = 4 << 30) -> None:
    """Write ``model`` as a Hugging Face style directory (``config.json`` + safetensors shards)."""
    from safetensors.torch import save_file
    from ..models.registry import hf_config_dict
    cfg = model.cfg
    out = Path(model_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(hf_config_dict(cfg), indent=1))
    tensors: Dict[str, Any] = {"model.embed_tokens.weight": model.p["embed"], "model.norm.weight": model.p["final_norm"]}
    q, kv = cfg.q_width, cfg.kv_width
    for i in range(cfg.n_layers):
        n = _hf_names(cfg, i)
        w = model.p[f"l{i}.wqkv"]
        gu = model.p[f"l{i}.w_gate_up"]
        tensors.update({n["attn_norm"]: model.p[f"l{i}.attn_norm"], n["q"]: w[:q], n["k"]: w[q:q + kv], n["v"]: w[q + kv:],
                        n["wo"]: model.p[f"l{i}.wo"], n["mlp_norm"]: model.p[f"l{i}.mlp_norm"], n["gate"]: gu[:cfg.d_ff],
                        n["up"]: gu[cfg.d_ff:], n["w_down"]: model.p[f"l{i}.w_down"]})
        if cfg.qk_norm:
            tensors.update({n["q_norm"]: model.p[f"l{i}.q_norm"], n["k_norm"]: model.p[f"l{i}.k_norm"]})
    if cfg.lm_head and not cfg.tie_embeddings:
        tensors["lm_head.weight"] = model.p["lm_head"]
    shard, size, k = {}, 0, 0
    items = list(tensors.items())
    for j, (name, t) in enumerate(items):
        shard[name] = t.detach().cpu().contiguous()
        size += t.numel() * 2
        if size >= shard_bytes or j == len(items) - 1:
            k += 1
            save_file(shard, str(out / f"model-{k:05d}.safetensors"))
            shard, size = {}, 0
