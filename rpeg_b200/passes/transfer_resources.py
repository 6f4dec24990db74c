"""Which device allocations a transfer node (COMM / RESHARD) keeps busy while it runs.

A weight transfer (label ``W_*``) or an activation transfer reserves only its destination when
the policy for its class says ``destination_only``; activations additionally need the producing
and consuming operators to use the same data-parallel degree (otherwise rows are repartitioned and
both sides take part). Everything else reserves both endpoints. Reference:
RPEG/passes/transfer_resources.py:18-148.
"""
from __future__ import annotations

from typing import Mapping, Set, Tuple

from ..core.types import Allocation, TransferResourcePolicy
from .lower import ExecNode, ExecNodeType


def is_weight_transfer(node: ExecNode) -> bool:
    return str(node.label or "").startswith("W_")


def _adjacent_op(ids, by_id):
    for i in sorted(ids):
        n = by_id.get(i)
        if n is not None and n.kind is ExecNodeType.OP and n.pi is not None:
            return n
    return None


def transfer_preserves_data_parallelism(node, *, predecessors: Mapping[str, Set[str]], successors: Mapping[str, Set[str]],
                                        by_id: Mapping[str, ExecNode]) -> bool:
    src = _adjacent_op(predecessors.get(node.id, ()), by_id)
    dst = _adjacent_op(successors.get(node.id, ()), by_id)
    return src is not None and dst is not None and int(src.pi[0]) == int(dst.pi[0])


def transfer_reserves_destination_only(node, *, policy: TransferResourcePolicy, predecessors, successors, by_id) -> bool:
    if node.kind not in (ExecNodeType.COMM, ExecNodeType.RESHARD) or len(node.allocs) < 2:
        return False
    weight = is_weight_transfer(node)
    if policy.for_weight(weight) != "destination_only":
        return False
    return weight or transfer_preserves_data_parallelism(node, predecessors=predecessors, successors=successors, by_id=by_id)


def reserved_allocations(node, *, policy: TransferResourcePolicy, predecessors, successors, by_id) -> Tuple[Allocation, ...]:
    if transfer_reserves_destination_only(node, policy=policy, predecessors=predecessors, successors=successors, by_id=by_id):
        chosen = node.allocs[-1:]
    else:
        chosen = node.allocs
    return tuple(dict.fromkeys(chosen))
