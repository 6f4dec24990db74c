"""Model families: Hugging Face ``config.json`` -> this engine's ``LlamaConfig``.

Two decoder families are supported, both pre-norm transformers with RMSNorm, rotary embeddings,
SwiGLU and (grouped-query) attention with head_dim 128:

  llama   Llama 2 / 3 (``model_type: llama``); optional llama3 rope scaling (low_freq_factor 1,
          high_freq_factor 4, original context 8192 are the only accepted parameters); optional tied
          embeddings
  qwen3   Qwen3 dense models (``model_type: qwen3``): as llama plus per-head RMSNorm on queries and keys

Anything the kernels do not implement is rejected here with a clear message (linear biases, attention
dropout, other rope scaling types, head_dim != 128, sliding windows). Reference:
RPEG/runtime/models/base.py:19-58, llama.py:17-79, qwen3.py:17-60, registry.py:23-52.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping

from ..runtime.errors import RuntimeConfigError
from .llama import LlamaConfig

FAMILIES = ("llama", "qwen3")


def _llama3_rope_factor(cfg: Mapping[str, Any]) -> float:
    raw = cfg.get("rope_scaling")
    if raw is None:
        return 1.0
    if not isinstance(raw, Mapping):
        raise RuntimeConfigError("rope_scaling must be a JSON object when provided")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        return 1.0
    if kind != "llama3":
        raise RuntimeConfigError(f"unsupported rope_scaling type {kind!r}; only llama3 scaling is implemented")
    if float(raw.get("low_freq_factor", 1.0)) != 1.0 or float(raw.get("high_freq_factor", 4.0)) != 4.0 \
            or int(raw.get("original_max_position_embeddings", 8192)) != 8192:
        raise RuntimeConfigError("unsupported llama3 rope_scaling factors (need low_freq_factor=1, high_freq_factor=4, "
                                 "original_max_position_embeddings=8192)")
    return max(1.0, float(raw.get("factor", 1.0)))


def config_from_hf(hf: Mapping[str, Any], *, max_pos: int | None = None, lm_head: bool = True, scalar_head: bool = False) -> LlamaConfig:
    family = hf.get("model_type")
    if family not in FAMILIES:
        raise RuntimeConfigError(f"unsupported model_type {family!r}; supported: {', '.join(FAMILIES)}")
    hidden, heads = int(hf["hidden_size"]), int(hf["num_attention_heads"])
    head_dim = int(hf.get("head_dim") or hidden // heads)
    if head_dim != 128:
        raise RuntimeConfigError(f"head_dim {head_dim} is not supported (the attention kernels are built for 128)")
    if hf.get("attention_bias") or hf.get("mlp_bias"):
        raise RuntimeConfigError("linear biases are not supported")
    if float(hf.get("attention_dropout", 0.0)) != 0.0:
        raise RuntimeConfigError("attention dropout is not supported")
    if hf.get("use_sliding_window") or (hf.get("sliding_window") and family != "qwen3"):
        raise RuntimeConfigError("sliding-window attention is not supported")
    if str(hf.get("hidden_act", "silu")) != "silu":
        raise RuntimeConfigError("only the SiLU-gated MLP is supported")
    return LlamaConfig(
        n_layers=int(hf["num_hidden_layers"]), d_model=hidden, d_ff=int(hf["intermediate_size"]), n_heads=heads,
        n_kv_heads=int(hf.get("num_key_value_heads", heads)), head_dim=head_dim, vocab=int(hf["vocab_size"]),
        rms_eps=float(hf.get("rms_norm_eps", 1e-6 if family == "qwen3" else 1e-5)),
        rope_theta=float(hf.get("rope_theta", 1e6 if family == "qwen3" else 5e5)),
        max_pos=int(max_pos or min(int(hf.get("max_position_embeddings", 8192)), 32768)),
        lm_head=lm_head, scalar_head=scalar_head, qk_norm=family == "qwen3",
        tie_embeddings=bool(hf.get("tie_word_embeddings", False)),
        rope_scaling_factor=_llama3_rope_factor(hf) if family == "llama" else 1.0, family=family)


def config_from_hf_path(path, **kw) -> LlamaConfig:
    p = Path(path)
    cfg_file = p / "config.json" if p.is_dir() else p
    if not cfg_file.exists():
        raise RuntimeConfigError(f"{cfg_file} does not exist")
    return config_from_hf(json.loads(cfg_file.read_text()), **kw)


def hf_config_dict(cfg: LlamaConfig) -> Dict[str, Any]:
    """The inverse mapping (used when exporting a checkpoint next to its architecture)."""
    out: Dict[str, Any] = {
        "model_type": cfg.family, "hidden_size": cfg.d_model, "intermediate_size": cfg.d_ff, "num_hidden_layers": cfg.n_layers,
        "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab,
        "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": cfg.max_pos, "hidden_act": "silu",
        "tie_word_embeddings": cfg.tie_embeddings, "attention_bias": False, "torch_dtype": "bfloat16"}
    if cfg.rope_scaling_factor > 1.0:
        out["rope_scaling"] = {"rope_type": "llama3", "factor": cfg.rope_scaling_factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192}
    return out
