"""Checked mode for the kernel wrappers: validate every DATA-DEPENDENT index a kernel is about to follow.

The kernels index memory with values they read from tensors: token ids into the embedding table, positions into the
rotary tables, (sequence, position) pairs through the page table into the KV pool, global row numbers into a peer's
buffer. Shapes and dtypes are always validated on the host; the VALUES are on the device, and a wrong one makes the
kernel read or write somewhere else without any error (or with a fault that ends the CUDA context). With
``RPEG_CHECK_ARGS=1`` in the environment (or ``set_enabled(True)``) every wrapper in ``ops/kernels.py`` that passes
such a tensor first reduces it on the device (min / max, a few masked comparisons) and raises
``KernelArgumentError`` naming the kernel, the argument, the offending value and the allowed range, BEFORE the launch.
Each check synchronises, so the mode is for debugging and tests, not for timed runs; inside a CUDA graph capture the
checks are skipped (run the generator with ``use_graphs=False`` to cover the decode step).

The validators are plain torch code and work on CPU tensors as well, which is how they are unit tested.

This takes the place of a memory checker on machines where none may be run; the reference has neither
(its closest pieces are shape asserts in RPEG/runtime/workers/megatron_worker.py:2370-2628 around generation).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

KV_PAGE = 64
ENABLED = os.environ.get("RPEG_CHECK_ARGS", "0") not in ("", "0", "false", "False")


class KernelArgumentError(ValueError):
    """A tensor argument holds an index outside the memory the kernel may touch."""


def set_enabled(on: bool) -> bool:
    """Switch checked mode; returns the previous setting."""
    global ENABLED
    prev, ENABLED = ENABLED, bool(on)
    return prev


def active() -> bool:
    """Checks run now: the mode is on and the current stream is not being captured into a graph."""
    if not ENABLED:
        return False
    return not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())


def index_range(kernel: str, name: str, t: Optional[torch.Tensor], lo: int, hi: int) -> None:
    """Every element of ``t`` must lie in ``[lo, hi)``."""
    if t is None or t.numel() == 0:
        return
    mn, mx = int(t.min()), int(t.max())
    if mn < lo or mx >= hi:
        bad = mn if mn < lo else mx
        where = int(((t < lo) | (t >= hi)).reshape(-1).nonzero()[0])
        raise KernelArgumentError(f"{kernel}: {name}[{where}] = {bad} outside [{lo}, {hi}) ({t.numel()} elements, min {mn}, max {mx})")


def rows(kernel: str, name: str, t: torch.Tensor, n: int) -> None:
    if t.numel() < n:
        raise KernelArgumentError(f"{kernel}: {name} has {t.numel()} elements, the kernel reads {n}")


def embed(kernel: str, ids: torch.Tensor, table_rows: int) -> None:
    index_range(kernel, "ids", ids, 0, table_rows)


def rope(kernel: str, pos: torch.Tensor, n_rows: int, cos_t: torch.Tensor) -> None:
    rows(kernel, "pos", pos, n_rows)
    index_range(kernel, "pos", pos.reshape(-1)[:n_rows], 0, cos_t.shape[0])


def pool_pages(kcache: torch.Tensor, n_kv_heads: int, head_dim: int) -> int:
    return kcache.numel() // (n_kv_heads * KV_PAGE * head_dim)


def kv_append(kernel: str, n_tokens: int, seq_id: torch.Tensor, pos: torch.Tensor, page_table: torch.Tensor, kcache: torch.Tensor,
              n_kv_heads: int, head_dim: int, cos_t: Optional[torch.Tensor] = None) -> None:
    """Tokens ``t < n_tokens`` are stored at ``page_table[seq_id[t], pos[t] // 64]``: the sequence must be a row of the
    table, the position inside the table's span (and inside the rotary tables), the page inside the pool."""
    rows(kernel, "seq_id", seq_id, n_tokens)
    rows(kernel, "pos", pos, n_tokens)
    if n_tokens == 0:
        return
    sid, p = seq_id.reshape(-1)[:n_tokens].long(), pos.reshape(-1)[:n_tokens].long()
    index_range(kernel, "seq_id", sid, 0, page_table.shape[0])
    index_range(kernel, "pos", p, 0, page_table.shape[1] * KV_PAGE)
    if cos_t is not None:
        index_range(kernel, "pos (rotary table)", p, 0, cos_t.shape[0])
    index_range(kernel, "page_table[seq_id, pos // 64]", page_table[sid, p // KV_PAGE], 0, pool_pages(kcache, n_kv_heads, head_dim))


def paged_attention(kernel: str, n_rows: int, seq_lens: torch.Tensor, page_table: torch.Tensor, kcache: torch.Tensor, n_kv_heads: int,
                    head_dim: int) -> None:
    """Row ``b`` reads the pages ``page_table[b, 0 .. ceil(seq_lens[b] / 64))``."""
    rows(kernel, "seq_lens", seq_lens, n_rows)
    if n_rows > page_table.shape[0]:
        raise KernelArgumentError(f"{kernel}: {n_rows} rows but the page table has {page_table.shape[0]}")
    if n_rows == 0:
        return
    lens = seq_lens.reshape(-1)[:n_rows].long()
    index_range(kernel, "seq_lens", lens, 0, page_table.shape[1] * KV_PAGE + 1)
    used = torch.arange(page_table.shape[1], device=page_table.device)[None, :] < ((lens + KV_PAGE - 1) // KV_PAGE)[:, None]
    index_range(kernel, "page_table (pages in use)", page_table[:n_rows][used], 0, pool_pages(kcache, n_kv_heads, head_dim))


def packed_sequences(kernel: str, cu_seqlens: torch.Tensor, n_tokens: int, max_seqlen: int) -> None:
    """``cu_seqlens``: starts at 0, never decreases, ends inside the packed buffer (tensor-parallel callers pad the
    token dimension, so the last boundary may lie before the buffer's end), no sequence longer than ``max_seqlen`` (the
    kernel sizes its grid from it)."""
    cu = cu_seqlens.reshape(-1).long()
    if cu.numel() < 2:
        raise KernelArgumentError(f"{kernel}: cu_seqlens needs at least two entries")
    d = cu[1:] - cu[:-1]
    if int(cu[0]) != 0 or int(cu[-1]) > n_tokens or int(d.min()) < 0:
        raise KernelArgumentError(f"{kernel}: cu_seqlens must rise from 0 to at most {n_tokens}, got {cu[:4].tolist()} ... {int(cu[-1])}")
    if int(d.max()) > max_seqlen:
        raise KernelArgumentError(f"{kernel}: a sequence of {int(d.max())} tokens exceeds max_seqlen = {max_seqlen}")


def row_indices(kernel: str, rows_t: torch.Tensor, n_rows: int) -> None:
    index_range(kernel, "rows", rows_t, 0, n_rows)


def global_rows(kernel: str, global_idx: torch.Tensor, rows_per_rank: int, world: int) -> None:
    index_range(kernel, "global_idx", global_idx, 0, rows_per_rank * world)
