"""Alias checks for in-place pointwise ops (``relu_``, ``add_``, ``mul_``, ``sigmoid_``).

A fused kernel never writes into the tensor an in-place op would have mutated: it
keeps the value in registers and writes only the chain's output.  Absorbing an
in-place op is therefore only sound when nobody outside the group can observe the
mutation — neither through the mutated tensor itself nor through a tensor it is a
view of.  Same API as the reference (fuseml/passes/mutation_safety.py:27-223):
``IN_PLACE_OPS``, ``MutationFinding``, ``is_safe_inplace``,
``check_group_mutation_safety``.  Nodes are duck-typed (``target``, ``args``, ``users``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterable

import torch

from .._logging import logger
from .topology import TRANSPARENT_OPS

_aten = torch.ops.aten

IN_PLACE_OPS: dict[Any, str] = {
    _aten.relu_.default: "elementwise",
    _aten.add_.Tensor: "elementwise",
    _aten.mul_.Tensor: "elementwise",
    _aten.sigmoid_.default: "elementwise",
}


@dataclass
class MutationFinding:
    node_name: str
    description: str
    safe: bool


def _has_external_users(node: Any, group_node_set: set, exclude: set | None = None) -> bool:
    skip = exclude or set()
    return any(u not in group_node_set and u not in skip for u in node.users)


def _view_ancestors(node: Any) -> Iterable[Any]:
    """The tensors ``node`` is (transitively) a view of."""
    cur = node
    while (hasattr(cur, "target") and cur.target in TRANSPARENT_OPS and getattr(cur, "args", None)
           and hasattr(cur.args[0], "users")):
        cur = cur.args[0]
        yield cur


def is_safe_inplace(node: Any, group_node_set: set) -> bool:
    """True when absorbing the in-place op ``node`` hides no mutation from outside users."""
    if node.target not in IN_PLACE_OPS or not node.args:
        return True
    mutated = node.args[0]
    if not hasattr(mutated, "users"):
        return True  # python scalar etc.
    me = {node}
    if _has_external_users(mutated, group_node_set, me):
        logger.debug("in-place %s: %s is read outside the group", node.name, getattr(mutated, "name", mutated))
        return False
    for base in _view_ancestors(mutated):
        if _has_external_users(base, group_node_set, me):
            logger.debug("in-place %s: mutates a view of %s, which is read outside the group",
                         node.name, getattr(base, "name", base))
            return False
    return True


def check_group_mutation_safety(group_nodes: list, group_node_set: set) -> list[MutationFinding]:
    """One finding per in-place node of the group."""
    findings: list[MutationFinding] = []
    for node in group_nodes:
        if getattr(node, "target", None) not in IN_PLACE_OPS:
            continue
        ok = is_safe_inplace(node, group_node_set)
        verdict = ("safe to fuse: no external aliasing detected" if ok
                   else "UNSAFE to fuse: the mutated tensor has external consumers")
        findings.append(MutationFinding(node_name=getattr(node, "name", str(node)),
                                        description=f"In-place op {node.target} is {verdict}.", safe=ok))
    return findings
