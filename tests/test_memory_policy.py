"""How many layers' activations the free memory pays for (``engine/memory_policy.py``), at the sizes the benchmark met."""
from rpeg_b200.engine.memory_policy import choose_kept_layers, layer_activation_bytes, layers_that_fit

L, D, F = 32, 4096, 11008      # Llama-7B


def test_activation_bytes_of_one_layer():
    assert abs(layer_activation_bytes(16384, D, F) - 2.325e9) < 5e6        # (7 d + 3 d_ff) bf16 values per token + 15 %
    assert layer_activation_bytes(8192, D, F) * 2 == layer_activation_bytes(16384, D, F)


def test_choices_at_the_memory_the_benchmark_found_free():
    assert choose_kept_layers(104.7e9, L, D, F, 16384) == (32, 16384)      # 4 GPUs: everything fits, microbatch stays
    assert choose_kept_layers(59.1e9, L, D, F, 16384) == (32, 8192)        # 2 GPUs: all layers only with the halved microbatch
    keep, micro = choose_kept_layers(25.9e9, L, D, F, 16384)               # 1 GPU: 12 of 32 layers, halved microbatch
    assert (keep, micro) == (12, 8192)
    assert choose_kept_layers(5e9, L, D, F, 16384) == (0, 16384)           # nothing fits: recompute everything, microbatch stays


def test_never_below_the_minimum_microbatch_and_monotone_in_memory():
    assert choose_kept_layers(30e9, L, D, F, 8192)[1] == 8192
    fits = [layers_that_fit(g * 1e9, L, D, F, 8192) for g in range(0, 80, 4)]
    assert fits == sorted(fits) and fits[0] == 0 and fits[-1] == L
