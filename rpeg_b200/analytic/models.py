"""Model shapes used by the planner. Parameter count of a dense Llama-style transformer:
``L * (4 d^2 + 2 d d_ff) + V d`` plus ``d`` for a scalar head on critic / reward / shared
actor-critic models (reference: RPEG/model/models.py:38-63)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

from ..core.types import Model


@dataclass(frozen=True)
class ModelSpec:
    L: int
    d: int
    d_ff: int
    V: int
    dtype_bytes: int = 2
    d_head: int = 128
    parameter_count: Optional[int] = None


# Stand-in for a reward that is a rule, not a network (length penalties, exact-match checkers, host-provided scores):
# the algorithm graph still has a reward vertex, but it must cost (almost) nothing in time and memory.
RULE_REWARD_SPEC = ModelSpec(1, 128, 128, 128)


def base_transformer_params(spec: ModelSpec) -> int:
    if spec.parameter_count is not None:
        return int(spec.parameter_count)
    return spec.L * (4 * spec.d * spec.d + 2 * spec.d * spec.d_ff) + spec.V * spec.d


def transformer_parameter_count(spec: ModelSpec, m: Model) -> int:
    scalar_head = spec.d if m in (Model.CRITIC, Model.REWARD, Model.AC_SHARE) else 0
    return base_transformer_params(spec) + scalar_head


@dataclass(frozen=True)
class ModelSuite:
    specs: Dict[Model, ModelSpec]

    def n_params(self, m: Model) -> int:
        return transformer_parameter_count(self.specs[m], m)
