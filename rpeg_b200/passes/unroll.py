"""Unroll the steady-state template over ``K_eval`` consecutive iterations.

Node ``(v, k)`` is vertex ``v`` in iteration ``k``. Data edges are replicated per iteration.
A publication edge of model ``m`` with staleness ``tau_m`` reaches iteration ``k`` from the
training node of iteration ``s_m(k) = max(0, k - (tau_m + 1))`` and only exists for ``k > tau_m``
(the first ``tau_m + 1`` iterations run on the initial weights). Same semantics as the
reference's RPEG/passes/unroll.py:62-152.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from ..core.types import Container, EdgeKind, Model, TemplateVertex
from ..ir.rpeg import RPEG


@dataclass(frozen=True)
class UnrolledNode:
    template_vertex: TemplateVertex
    k: int
    i: Optional[int] = None

    @property
    def id(self) -> str:
        base = f"{self.template_vertex.id}@{self.k}"
        return base if self.i is None else f"{base}:{self.i}"


@dataclass(frozen=True)
class UnrolledEdge:
    src: UnrolledNode
    dst: UnrolledNode
    container: Container
    kind: EdgeKind


@dataclass(frozen=True)
class UnrolledRPEG:
    nodes: Tuple[UnrolledNode, ...]
    data_edges: Tuple[UnrolledEdge, ...]
    pub_edges: Tuple[UnrolledEdge, ...]


def publisher_selection(model: Model, tau: Dict[Model, int], k: int) -> int:
    """Iteration whose training output iteration ``k`` consumes."""
    if model not in tau:
        raise ValueError(f"no staleness budget for trainable model {model.value}")
    t = tau[model]
    if isinstance(t, bool) or not isinstance(t, int) or t < 0:
        raise ValueError(f"staleness budget of {model.value} must be a non-negative integer")
    return max(0, k - (t + 1))


def unroll(rpeg: RPEG, K_eval: int, verbose: bool = False) -> UnrolledRPEG:
    if K_eval < 1:
        raise ValueError(f"K_eval must be >= 1, got {K_eval}")
    rpeg.well_formed()
    at = {(v.id, k): UnrolledNode(v, k) for k in range(K_eval) for v in rpeg.vertices}
    nodes = tuple(at[(v.id, k)] for k in range(K_eval) for v in rpeg.vertices)
    data = tuple(UnrolledEdge(at[(e.src.id, k)], at[(e.dst.id, k)], e.container, EdgeKind.DATA)
                 for k in range(K_eval) for e in rpeg.data_edges)
    pub = []
    for k in range(1, K_eval):
        for e in rpeg.pub_edges:
            m = e.src.kind.model
            if k <= rpeg.tau[m]:
                continue
            src_k = publisher_selection(m, rpeg.tau, k)
            assert src_k < k
            pub.append(UnrolledEdge(at[(e.src.id, src_k)], at[(e.dst.id, k)], e.container, EdgeKind.PUB))
    out = UnrolledRPEG(nodes, data, tuple(pub))
    if verbose:
        print(f"unrolled {K_eval} steps: {len(nodes)} nodes, {len(data)} data edges, {len(pub)} publication edges")
    return out
