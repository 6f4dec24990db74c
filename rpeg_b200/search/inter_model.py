"""Structural search space: which template (PPO with or without actor/critic stage fusion, PPO
with a shared actor-critic trunk, GRPO, DPO) and which staleness budget per trainable model.
Enumeration order follows the reference (RPEG/search/inter_model.py:26-121)."""
from __future__ import annotations

import dataclasses
import itertools
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Set, Tuple

from ..analytic.models import ModelSuite
from ..analytic.workload import Workload
from ..core.types import Model
from ..ir.rpeg import RPEG
from ..ir.templates import build_AC_share_RPEG, build_DPO_RPEG, build_GRPO_RPEG, build_PPO_RPEG, is_AC_share_applicable

DEFAULT_T_CAND: Dict[Model, Set[int]] = {Model.ACTOR: {0, 1}, Model.CRITIC: {0, 1}, Model.AC_SHARE: {0, 1}}


@dataclass
class InterModelConfig:
    ac_share: bool
    tau: Dict[Model, int]
    algorithm: str = "ppo"
    intra_stage_fusion: bool = False

    def family(self) -> Tuple[bool, bool]:
        return (self.ac_share, self.intra_stage_fusion)


def iter_staleness(trainable, T_cand) -> Iterator[Dict[Model, int]]:
    models = sorted(trainable, key=lambda m: m.value)
    for combo in itertools.product(*[sorted(T_cand[m]) for m in models]):
        yield dict(zip(models, combo))


def Iter_inter_model_candidates(suite: ModelSuite, workload: Workload, T_cand: Optional[Dict[Model, Set[int]]] = None,
                                algorithm: str = "ppo") -> Iterator[Tuple[RPEG, InterModelConfig]]:
    T_cand = {m: set(s) for m, s in (T_cand or DEFAULT_T_CAND).items()}
    for m, s in DEFAULT_T_CAND.items():
        T_cand.setdefault(m, set(s))
    if algorithm in ("dpo", "grpo"):
        base = (build_DPO_RPEG if algorithm == "dpo" else build_GRPO_RPEG)(suite, workload)
        for tau in iter_staleness(base.trainable, T_cand):
            yield dataclasses.replace(base, tau=tau), InterModelConfig(False, tau, algorithm)
        return
    ppo = build_PPO_RPEG(suite, workload)
    for tau in iter_staleness(ppo.trainable, T_cand):
        for fusion in (False, True):
            yield dataclasses.replace(ppo, tau=tau), InterModelConfig(False, tau, "ppo", fusion)
    if is_AC_share_applicable(ppo) and Model.AC_SHARE in suite.specs:
        ac = build_AC_share_RPEG(suite, workload)
        for tau in iter_staleness(ac.trainable, T_cand):
            yield dataclasses.replace(ac, tau=tau), InterModelConfig(True, tau, "ppo", False)
