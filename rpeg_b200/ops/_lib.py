"""ctypes loader for the in-tree native library ``rpeg_b200/librpeg_kernels.so``.

The library is never optional on a GPU machine: ``lib()`` raises if it is missing or fails to
load, so no op can silently fall back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "librpeg_kernels.so"
_lib = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

_SIGNATURES = {
    "rpeg_gemm_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, LL, P, P],
    "rpeg_gemm_bf16_gated": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, LL, P, I, c_uint, c_ulonglong, P, P],
    "rpeg_publish_version": [P, I, I, c_uint, P],
    "rpeg_wait_flags": [P, I, c_uint, c_ulonglong, P, P],
    "rpeg_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "rpeg_rmsnorm_bwd": [P, P, P, P, P, P, P, I, I, P],
    "rpeg_rope": [P, P, P, P, I, I, I, I, I, I, P],
    "rpeg_swiglu_fwd": [P, P, LL, I, P],
    "rpeg_swiglu_bwd": [P, P, P, LL, I, P],
    "rpeg_add_bf16": [P, P, P, LL, P],
    "rpeg_embed_fwd": [P, P, P, I, I, P],
    "rpeg_embed_bwd": [P, P, P, I, I, P],
    "rpeg_token_logprob_fwd": [P, P, P, P, I, I, I, F, P],
    "rpeg_token_logprob_bwd": [P, P, P, P, I, I, I, F, P],
    "rpeg_token_entropy": [P, P, P, I, I, I, F, P],
    "rpeg_token_logprob_entropy_bwd": [P, P, P, P, P, P, I, I, I, F, P],
    "rpeg_policy_loss": [P, P, P, P, P, P, P, LL, F, F, F, P],
    "rpeg_masked_rowsum": [P, P, P, I, I, P],
    "rpeg_dpo_loss": [P, P, P, P, I, F, P],
    "rpeg_expand_seq_coef": [P, P, P, I, I, P],
    "rpeg_value_loss": [P, P, P, P, P, LL, F, P],
    "rpeg_gae": [P, P, P, P, P, P, P, I, I, F, F, F, I, P],
    "rpeg_group_advantage": [P, P, I, I, P],
    "rpeg_sample": [P, I, I, I, F, I, c_ulonglong, P, P, P, P, P],
    "rpeg_head_gemv": [P, P, P, P, I, I, P],
    "rpeg_head_gemv_bwd": [P, P, P, P, P, P, I, I, P],
    "rpeg_adamw": [P, P, P, P, P, LL, F, F, F, F, F, I, F, P, I, F, P],
    "rpeg_sumsq": [P, LL, P, P],
    "rpeg_flag_barrier": [P, I, I, I, c_uint, P, P, c_ulonglong, P, P],
    "rpeg_dp_reduce_norm": [P, I, LL, LL, F, P, P, P],
    "rpeg_dp_adam_push": [P, P, P, P, P, I, LL, LL, F, F, F, F, F, I, P, I, F, P],
    "rpeg_copy16": [P, P, LL, P],
    "rpeg_gemm_bf16_partials": [P, P, I, I, I, I, I, P, c_longlong, P, P, P],
    "rpeg_rmsnorm_fwd_partials": [P, I, c_longlong, P, P, P, P, I, I, F, P],
    "rpeg_swiglu_fwd_partials": [P, I, c_longlong, P, c_longlong, I, P],
    "rpeg_rope_kv_append_partials": [P, I, c_longlong, P, I, I, I, I, P, P, P, P, P, I, P, P, I, I, I, I, P],
    "rpeg_headnorm_fwd": [P, I, I, I, I, P, P, I, F, P],
    "rpeg_headnorm_bwd": [P, I, P, I, I, I, I, P, P, P, I, P],
    "rpeg_ag_gemm": [P, P, P, P, I, I, I, I, I, I, I, I, c_uint, P, P],
    "rpeg_copy2d": [P, c_longlong, P, c_longlong, c_longlong, c_longlong, P],
    "rpeg_scatter_rows_by_index": [P, c_longlong, c_longlong, P, c_longlong, P, I, P],
    "rpeg_sample_filtered": [P, I, I, I, F, I, F, c_ulonglong, P, P, P, P, P],
    "rpeg_gemm_rs": [P, P, I, I, I, I, I, P, P, P, I, I, I, c_uint, I, P, P],
    "rpeg_kv_append": [P, I, I, I, P, P, P, I, P, P, I, I, I, P],
    "rpeg_rope_kv_append": [P, I, I, I, I, P, P, P, P, P, I, P, P, I, I, I, I, P],
    "rpeg_paged_decode_attn": [P, I, I, P, P, P, I, P, P, P, I, I, I, I, I, F, P],
    "rpeg_paged_decode_attn_grouped": [P, I, I, P, P, P, I, P, P, P, I, I, I, I, I, F, P, P, P, P],
    "rpeg_tp_allreduce_rmsnorm": [P, P, I, I, LL, P, P, LL, LL, I, I, F, LL, P, c_ulonglong, P, P],
    "rpeg_tp_allgather_cols": [P, P, I, I, LL, I, I, I, LL, P, c_ulonglong, P, P],
    "rpeg_tp_allreduce_rmsnorm_ll": [P, P, I, I, LL, P, I, LL, P, P, LL, LL, I, I, F, LL, I, P, c_ulonglong, P, P],
    "rpeg_tp_trace": [I, P],
    "rpeg_paged_decode_attn_grouped_tc": [P, I, I, P, P, LL, P, I, P, P, P, I, I, I, I, I, F, P, P, P, P, P],
    "rpeg_gemm_swiglu": [P, P, P, I, I, I, I, I, I, P, P],
    "rpeg_symm_alloc": [c_ulonglong, P],
    "rpeg_symm_free": [P],
    "rpeg_ipc_export": [P, P],
    "rpeg_ipc_open": [P, P],
    "rpeg_ipc_close": [P],
    "rpeg_memset_async": [P, I, c_ulonglong, P],
    "rpeg_decode_prepare": [P, P, P, P, I, I, P],
    "rpeg_decode_advance": [P, P, P, P, P, P, P, P, P, I, I, I, P, P, P],
    "rpeg_gather_rows": [P, P, P, I, I, P],
    "rpeg_scatter_rows": [P, P, P, I, I, I, P],
    "rpeg_splitk_reduce": [P, P, I, I, I, I, P],
    "rpeg_flash_attn_fwd": [P, I, I, I, I, P, I, I, I, I, I, I, F, P, P, P, P],
    "rpeg_flash_attn_bwd": [P, I, I, I, I, P, P, P, P, I, I, I, I, I, I, F, P, P, P, I, P, P],
}


def lib_path() -> Path:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    """Load (once) and return the native library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m rpeg_b200.build_ext` "
                "(the CUDA kernels are mandatory; there is no eager fallback)"
            )
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue  # symbol added by a newer source than the built library
            fn.argtypes = argtypes
            fn.restype = c_int
        if hasattr(handle, "rpeg_decode_attn_scratch_bytes"):
            handle.rpeg_decode_attn_scratch_bytes.argtypes = [I, I, I]
            handle.rpeg_decode_attn_scratch_bytes.restype = c_longlong
        _lib = handle
    return _lib


_launches = 0


def launch_count() -> int:
    """Number of native kernel launches issued so far by this process (graph replays included:
    a replay adds the number of launches recorded while that graph was captured)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def check(rc: int, what: str) -> None:
    global _launches
    if rc != 0:
        raise RuntimeError(f"{what} failed with native error code {rc}")
    _launches += 1
