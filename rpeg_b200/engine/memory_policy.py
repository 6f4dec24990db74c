"""How much of the backward pass's recomputation the free device memory can buy.

A training microbatch either keeps a layer's activations for the backward pass (``(7 d + 3 d_ff)`` bf16 values per token plus
the attention statistics) or recomputes the layer from its saved input. ``choose_kept_layers`` turns the memory that is
free after the models, the optimizer state and the KV pool are allocated into the number of layers to keep, and halves
the microbatch when that lets more layers fit (same tokens per step, twice the launches). Reference: activation
checkpointing is all-or-nothing there (``optimizer_runtime.activation_checkpointing``, RPEG/runtime/schema.py:667 region).
"""
from __future__ import annotations

from typing import Tuple

ACTIVATION_SLACK = 1.15          # attention statistics, norm statistics, allocator rounding
FIXED_RESERVE_BYTES = 8e9        # LM-head chunk, backward temporaries, fragmentation
RESERVE_LAYERS = 3.0             # one layer being recomputed plus the backward pass's per-layer temporaries


def layer_activation_bytes(micro_tokens: int, d_model: int, d_ff: int) -> float:
    return ACTIVATION_SLACK * micro_tokens * (7 * d_model + 3 * d_ff) * 2


def layers_that_fit(free_bytes: float, n_layers: int, d_model: int, d_ff: int, micro_tokens: int) -> int:
    per_layer = layer_activation_bytes(micro_tokens, d_model, d_ff)
    reserve = FIXED_RESERVE_BYTES + RESERVE_LAYERS * per_layer
    return max(0, min(n_layers, int((free_bytes - reserve) // per_layer)))


def choose_kept_layers(free_bytes: float, n_layers: int, d_model: int, d_ff: int, micro_tokens: int,
                       min_micro_tokens: int = 8192) -> Tuple[int, int]:
    """``(layers whose activations are kept, microbatch tokens)``: the requested microbatch if every layer fits with it,
    else half of it if more layers fit then (never below ``min_micro_tokens``)."""
    fit = layers_that_fit(free_bytes, n_layers, d_model, d_ff, micro_tokens)
    if fit < n_layers and micro_tokens // 2 >= min_micro_tokens:
        half = layers_that_fit(free_bytes, n_layers, d_model, d_ff, micro_tokens // 2)
        if half > fit:
            return half, micro_tokens // 2
    return fit, micro_tokens
