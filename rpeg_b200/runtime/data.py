"""Batch and minibatch index selection (pure functions, same result on every rank).

``dataset_batch_indices`` picks the prompts of one logical step from a dataset of ``n_items`` rows: consecutive
windows that wrap around, optionally over a permutation that is reshuffled every pass (reference:
RPEG/runtime/data.py:16-52). ``minibatch_indices`` cuts the rows of a rollout into the minibatches of the
policy / critic update epochs (reference: RPEG/runtime/ppo_math.py:93-112): every epoch visits every row once, in
a fresh order when ``shuffle`` is set; the last minibatch of an epoch may be short unless ``drop_last``.
``quantile_lengths`` draws synthetic response lengths from the workload's quantile phases.
"""
from __future__ import annotations

import random
from typing import List, Optional, Sequence, Tuple


def dataset_batch_indices(n_items: int, batch_size: int, step: int, *, seed: int = 0, shuffle: bool = False) -> List[int]:
    """Row indices of logical step ``step`` (1-based)."""
    if n_items < 1 or batch_size < 1 or step < 1:
        raise ValueError("n_items, batch_size and step must be >= 1")
    out: List[int] = []
    pos = (step - 1) * batch_size
    while len(out) < batch_size:
        epoch, off = divmod(pos, n_items)
        if shuffle:
            perm = list(range(n_items))
            random.Random(seed * 1000003 + epoch).shuffle(perm)
            out.append(perm[off])
        else:
            out.append(off)
        pos += 1
    return out


def minibatch_indices(n_rows: int, minibatch_size: Optional[int], epochs: int = 1, *, seed: int = 0, shuffle: bool = True,
                      drop_last: bool = False) -> List[List[int]]:
    """The sequence of minibatches (lists of row indices) of all ``epochs``; ``minibatch_size=None`` means one
    minibatch with every row per epoch (a single optimizer step per epoch)."""
    if n_rows < 1 or epochs < 1:
        raise ValueError("n_rows and epochs must be >= 1")
    size = n_rows if not minibatch_size else int(minibatch_size)
    if size < 1:
        raise ValueError("minibatch_size must be >= 1")
    out: List[List[int]] = []
    for e in range(epochs):
        rows = list(range(n_rows))
        if shuffle and size < n_rows:
            random.Random(seed * 1000003 + e).shuffle(rows)
        for s in range(0, n_rows, size):
            mb = rows[s:s + size]
            if len(mb) < size and drop_last and out:
                continue
            out.append(sorted(mb))
    return out


def quantile_lengths(n_rows: int, quantiles: Sequence[Tuple[float, int]], *, seed: int = 0) -> List[int]:
    """One generation length per row of a logical batch, following ``workload.gen_quantiles``: a row ends in
    phase ``q`` with that phase's probability mass and at a length uniform in ``(previous bound, bound]``. This
    is the length distribution the planner's quantile split assumes (reference: RPEG/analytic/workload.py:30-62
    describes the phases; synthetic runs of the reference reach the cap instead)."""
    if n_rows < 0:
        raise ValueError("n_rows must be >= 0")
    rng = random.Random(seed)
    out: List[int] = []
    for _ in range(n_rows):
        u = rng.random()
        lo = 0
        for frac, bound in quantiles:
            if u < frac or frac >= 1.0:
                out.append(lo + 1 + rng.randrange(max(1, int(bound) - lo)))
                break
            lo = int(bound)
        else:   # fractions that do not reach 1.0: the rest runs to the last bound
            out.append(int(quantiles[-1][1]))
    return out
