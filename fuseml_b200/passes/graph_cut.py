"""Cut a fusion group at the first op the epilogue program cannot express.

Everything before the cut stays a (shorter) fused group, the offending op and what
follows run as ordinary PyTorch ops; if an ``addmm`` shows up later in the tail it may
seed a second group.  Same API as the reference (fuseml/passes/graph_cut.py:37-390):
``SUPPORTED_TRITON_OPS`` (kept under that name; it now lists what the sm_100a epilogue
VM implements — also exported as ``SUPPORTED_EPILOGUE_OPS``), ``GraphSegment``,
``validate_fusion_group``, ``split_fusion_group``.  Nodes are duck-typed so tests can
pass light stand-ins.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Literal

import torch

from .._logging import logger
from ..codegen.kernel_cache import _materialize_ints
from ..fusion_group import FusionGroup
from .topology import TRANSPARENT_OPS

_aten = torch.ops.aten

SUPPORTED_EPILOGUE_OPS: dict[Any, str] = {
    _aten.addmm.default: "gemm",
    _aten.mm.default: "gemm",
    _aten.relu.default: "elementwise",
    _aten.relu_.default: "elementwise",
    _aten.gelu.default: "elementwise",
    _aten.sigmoid.default: "elementwise",
    _aten.sigmoid_.default: "elementwise",
    _aten.add.Tensor: "elementwise",
    _aten.add_.Tensor: "elementwise",
    _aten.mul.Tensor: "elementwise",
    _aten.mul_.Tensor: "elementwise",
    _aten.gelu_backward.default: "elementwise",   # absorbed only when discovery runs with backward_ops=True
    _aten.sum.dim_IntList: "reduction",
    _aten.amax.default: "reduction",
    _aten.mean.dim: "reduction",
}
SUPPORTED_TRITON_OPS = SUPPORTED_EPILOGUE_OPS  # historical name, same object


@dataclass
class GraphSegment:
    kind: Literal["fused", "native"]
    group: FusionGroup | None = None
    nodes: list = field(default_factory=list)

    def __repr__(self) -> str:
        return f"GraphSegment(kind={self.kind!r}, nodes={[n.name for n in self.nodes]})"


def validate_fusion_group(group: FusionGroup) -> list:
    """Nodes of ``group`` with no epilogue translation (views are fine: they are no-ops)."""
    return [n for n in group.all_nodes
            if n.op == "call_function" and n.target not in SUPPORTED_EPILOGUE_OPS
            and n.target not in TRANSPARENT_OPS]


def _extract_tensor_metadata(node: Any) -> dict:
    meta = node.meta.get("tensor_meta")
    if meta is not None and not hasattr(meta, "shape"):
        meta = meta[0] if isinstance(meta, (tuple, list)) and len(meta) > 0 else None
    if meta is None or not hasattr(meta, "shape"):
        return {}
    return {"shape": _materialize_ints(meta.shape), "stride": _materialize_ints(meta.stride), "dtype": meta.dtype}


def _wire(sub: FusionGroup, parent_bindings: dict) -> None:
    """Recompute inputs, escape nodes, output metadata and parameter bindings of ``sub``."""
    members = set(sub.all_nodes)
    for node in sub.all_nodes:
        for arg in node.args:
            if hasattr(arg, "op") and arg not in members and arg not in sub.inputs:
                sub.inputs.append(arg)
    for node in sub.all_nodes:
        if node is not sub.output_node and any(u not in members for u in node.users):
            sub.intermediate_outputs.append(node)
    sub.output_metadata = _extract_tensor_metadata(sub.output_node)
    sub.original_inputs = list(sub.inputs)
    if parent_bindings:
        wanted = set()
        for inp in sub.inputs:
            if getattr(inp, "op", None) == "get_attr":
                wanted.add(inp.target)
            for arg in getattr(inp, "args", ()) or ():
                if getattr(arg, "op", None) == "get_attr":
                    wanted.add(arg.target)
        sub.param_bindings = {k: v for k, v in parent_bindings.items() if k in wanted}


def _build_sub_group(original: FusionGroup, fused_subset: list) -> FusionGroup:
    sub = FusionGroup(base_node=original.base_node)
    sub.fused_nodes = list(fused_subset)
    sub.output_node = fused_subset[-1] if fused_subset else original.base_node
    _wire(sub, original.param_bindings)
    return sub


def split_fusion_group(group: FusionGroup) -> list[GraphSegment]:
    bad = validate_fusion_group(group)
    if not bad:
        return [GraphSegment("fused", group, list(group.all_nodes))]
    first_bad = bad[0]
    logger.warning("Unsupported op %s (node %r) found in %s — splitting.", first_bad.target, first_bad.name, group)
    if first_bad is group.base_node:
        return [GraphSegment("native", nodes=list(group.all_nodes))]

    cut = next(i for i, n in enumerate(group.fused_nodes) if n is first_bad)
    segments: list[GraphSegment] = []
    head = group.fused_nodes[:cut]
    if head:
        a = _build_sub_group(group, head)
        segments.append(GraphSegment("fused", a, list(a.all_nodes)))
    else:
        segments.append(GraphSegment("native", nodes=[group.base_node]))  # a lone GEMM gains nothing

    tail = group.fused_nodes[cut:]  # starts with the unsupported node
    reseed = next((j for j, n in enumerate(tail)
                   if j > 0 and n.op == "call_function" and n.target is _aten.addmm.default), None)
    if reseed is None:
        segments.append(GraphSegment("native", nodes=tail))
        return segments
    segments.append(GraphSegment("native", nodes=tail[:reseed]))
    rest = [n for n in tail[reseed + 1:] if n.op == "call_function" and n.target in SUPPORTED_EPILOGUE_OPS]
    if rest:
        b = FusionGroup(base_node=tail[reseed])
        b.fused_nodes = rest
        b.output_node = rest[-1]
        _wire(b, group.param_bindings)
        segments.append(GraphSegment("fused", b, list(b.all_nodes)))
    else:
        segments.append(GraphSegment("native", nodes=tail[reseed:]))
    return segments
