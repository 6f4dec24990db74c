"""The RPEG template graph: one steady-state RLHF iteration as vertices, data edges and
publication edges, plus the staleness budget per trainable model.

``well_formed`` enforces the same structural rules as the reference's ``RPEG.well_formed``
(RPEG/ir/rpeg.py:37-186): unique ids, edges between known vertices, tau defined exactly for the
trainable models, publication edges leaving a TRAIN vertex of the model they publish, containers
present on both interfaces of an edge, a publication per trainable model, consistent container
definitions, matching step boundary, and an acyclic data-edge graph.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, Set, Tuple

from ..core.types import Container, EdgeKind, Model, Role, TemplateEdge, TemplateVertex


class IllFormedRPEG(ValueError):
    pass


@dataclass
class RPEG:
    vertices: Tuple[TemplateVertex, ...]
    data_edges: Tuple[TemplateEdge, ...]
    pub_edges: Tuple[TemplateEdge, ...]
    containers: Tuple[Container, ...]
    in_containers: Tuple[Container, ...]
    out_containers: Tuple[Container, ...]
    tau: Dict[Model, int] = field(default_factory=dict)
    trainable: Set[Model] = field(default_factory=set)

    def vertex(self, vid: str) -> TemplateVertex:
        for v in self.vertices:
            if v.id == vid:
                return v
        raise KeyError(vid)

    def vertex_ids(self) -> Tuple[str, ...]:
        return tuple(v.id for v in self.vertices)

    def topological_vertices(self) -> Tuple[TemplateVertex, ...]:
        """Kahn order over data edges; ties resolved by declaration order."""
        indeg = {v.id: 0 for v in self.vertices}
        succ = defaultdict(list)
        for e in self.data_edges:
            indeg[e.dst.id] += 1
            succ[e.src.id].append(e.dst.id)
        order, ready = [], [v.id for v in self.vertices if indeg[v.id] == 0]
        while ready:
            vid = ready.pop(0)
            order.append(vid)
            for nxt in succ[vid]:
                indeg[nxt] -= 1
                if indeg[nxt] == 0:
                    ready.append(nxt)
        if len(order) != len(self.vertices):
            raise IllFormedRPEG("data edges contain a cycle")
        return tuple(self.vertex(v) for v in order)

    def well_formed(self, verbose: bool = False) -> bool:
        ids = [v.id for v in self.vertices]
        if len(set(ids)) != len(ids):
            raise IllFormedRPEG("duplicate vertex ids")
        known = set(ids)
        for e in (*self.data_edges, *self.pub_edges):
            if e.src.id not in known or e.dst.id not in known:
                raise IllFormedRPEG(f"edge {e.src.id}->{e.dst.id} references an unknown vertex")
        if set(self.tau) != set(self.trainable):
            raise IllFormedRPEG("tau must be defined exactly for the trainable models")
        for m, t in self.tau.items():
            if not isinstance(t, int) or isinstance(t, bool) or t < 0:
                raise IllFormedRPEG(f"tau[{m.value}] must be a non-negative integer")
        for e in self.data_edges:
            if e.kind is not EdgeKind.DATA:
                raise IllFormedRPEG("data edge list holds a non-data edge")
            self._check_interface(e)
        published = set()
        for e in self.pub_edges:
            if e.kind is not EdgeKind.PUB:
                raise IllFormedRPEG("publication edge list holds a non-publication edge")
            if e.src.kind.role is not Role.TRAINING or e.src.kind.model not in self.trainable:
                raise IllFormedRPEG(f"publication edge {e.src.id}->{e.dst.id} must leave a TRAIN vertex of a trainable model")
            if e.dst.kind.model is not e.src.kind.model:
                raise IllFormedRPEG(f"publication edge {e.src.id}->{e.dst.id} crosses models")
            self._check_interface(e)
            published.add(e.src.kind.model)
        if published != set(self.trainable):
            raise IllFormedRPEG("every trainable model needs a publication edge")
        by_name: Dict[str, Container] = {}
        for v in self.vertices:
            for c in (*v.kind.read, *v.kind.write):
                if by_name.setdefault(c.name, c) != c:
                    raise IllFormedRPEG(f"container {c.name} is defined inconsistently")
        for c in (*self.containers, *self.in_containers, *self.out_containers):
            if by_name.setdefault(c.name, c) != c:
                raise IllFormedRPEG(f"container {c.name} is defined inconsistently")
        # step boundary: what a step needs from the previous one (weights of trainable models that
        # are read before being written) is exactly what it hands to the next one.
        if self._boundary_in() != self._boundary_out():
            raise IllFormedRPEG("step boundary mismatch between consumed and produced weights")
        self.topological_vertices()
        if verbose:
            print(f"RPEG well formed: {len(self.vertices)} vertices, {len(self.data_edges)} data edges, "
                  f"{len(self.pub_edges)} publication edges")
        return True

    @staticmethod
    def _check_interface(e: TemplateEdge) -> None:
        if e.container not in e.src.kind.write:
            raise IllFormedRPEG(f"{e.container.name} is not written by {e.src.id}")
        if e.container not in e.dst.kind.read:
            raise IllFormedRPEG(f"{e.container.name} is not read by {e.dst.id}")

    def _boundary_in(self) -> Set[str]:
        return {e.container.name for e in self.pub_edges}

    def _boundary_out(self) -> Set[str]:
        return {c.name for v in self.vertices if v.kind.role is Role.TRAINING and v.kind.model in self.trainable
                for c in v.kind.write if c.name.startswith("W_")}
