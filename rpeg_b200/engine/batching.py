"""Packing of (prompt, response) rows into variable-length token streams for the packed kernels.

A rollout batch is ``prompt_ids [N, S]`` (+ ``prompt_lens``), ``resp_ids [N, T]`` (+ ``resp_lens``).
Row ``i`` becomes the sequence ``prompt_i[:pl_i] ++ resp_i[:rl_i]``; sequences are concatenated with
``cu_seqlens`` offsets (no padding tokens are ever computed). The hidden state at sequence index
``pl_i - 1 + t`` predicts response token ``t``, so those rows (``sel``) are the only ones that reach
the LM / value head. ``flat`` maps each selected row back to ``i * T + t`` in ``[N, T]`` arrays
(old log-probs, advantages, masks).

The reference pads to ``[N, S+T]`` and slices ``prompt_len-1`` onward
(RPEG/runtime/algorithms/ppo_graph.py:980, RPEG/runtime/workers/megatron_worker.py:1879-1928).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch


@dataclass
class PackedBatch:
    rows: List[int]            # original row indices in this microbatch, in order
    tokens: torch.Tensor       # [Ttot] int32
    pos: torch.Tensor          # [Ttot] int32
    cu_seqlens: torch.Tensor   # [n+1] int32
    max_seqlen: int
    sel: torch.Tensor          # [n_sel] int32 rows of the packed stream feeding the heads
    targets: torch.Tensor      # [n_sel] int32 response token predicted by each selected row
    flat: torch.Tensor         # [n_sel] int64 index into [N, T] row-major arrays
    last: torch.Tensor         # [n] int32 packed index of each sequence's last token
    n_tokens: int


def split_microbatches(total_lens: Sequence[int], max_tokens: int, group: int = 1) -> List[List[int]]:
    """Greedy split of row indices into microbatches of at most ``max_tokens`` packed tokens, never
    separating the ``group`` consecutive rows of one prompt/pair."""
    out, cur, cur_tok = [], [], 0
    for g0 in range(0, len(total_lens), group):
        idx = list(range(g0, min(len(total_lens), g0 + group)))
        tok = sum(total_lens[i] for i in idx)
        if cur and cur_tok + tok > max_tokens:
            out.append(cur)
            cur, cur_tok = [], 0
        cur.extend(idx)
        cur_tok += tok
    if cur:
        out.append(cur)
    return out


def pack_rows(prompt_ids: torch.Tensor, prompt_lens: Sequence[int], resp_ids: torch.Tensor, resp_lens: Sequence[int],
              rows: Sequence[int]) -> PackedBatch:
    dev = prompt_ids.device
    T = resp_ids.shape[1]
    pieces, pos, sel, flat, cu, last = [], [], [], [], [0], []
    off = 0
    for i in rows:
        pl, rl = int(prompt_lens[i]), int(resp_lens[i])
        pieces.append(prompt_ids[i, :pl])
        pieces.append(resp_ids[i, :rl])
        n = pl + rl
        pos.append(torch.arange(n, dtype=torch.int32))
        if rl > 0:
            sel.append(torch.arange(off + pl - 1, off + pl - 1 + rl, dtype=torch.int32))
            flat.append(torch.arange(i * T, i * T + rl, dtype=torch.int64))
        off += n
        cu.append(off)
        last.append(off - 1)
    tokens = torch.cat(pieces).to(torch.int32)
    sel_t = torch.cat(sel) if sel else torch.zeros(0, dtype=torch.int32)
    flat_t = torch.cat(flat) if flat else torch.zeros(0, dtype=torch.int64)
    flat_dev = flat_t.to(dev)
    targets = resp_ids.reshape(-1)[flat_dev].to(torch.int32)
    return PackedBatch(list(rows), tokens.contiguous(), torch.cat(pos).to(dev), torch.tensor(cu, dtype=torch.int32, device=dev),
                       max(int(prompt_lens[i]) + int(resp_lens[i]) for i in rows), sel_t.to(dev), targets.contiguous(),
                       flat_dev, torch.tensor(last, dtype=torch.int32, device=dev), off)
