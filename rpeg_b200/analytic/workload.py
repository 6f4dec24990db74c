"""Workload description: B prompts per step, K samples per prompt, prompt length S, generation
length T and optional cumulative generation-length quantiles ((fraction, tokens), ...)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class Workload:
    B: int
    K: int
    S: int
    T: int
    gen_quantiles: Optional[Tuple[Tuple[float, int], ...]] = None
