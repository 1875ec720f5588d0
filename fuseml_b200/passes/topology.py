"""Node classification for fusion discovery, and the roofline router's Python face.

Classification looks only at ``node.target`` (the ATen overload object) and at graph
connectivity, never at node names, so graphs from ``make_fx``, Dynamo or AOT Autograd
are treated alike.  Public names follow the reference (fuseml/passes/topology.py:36-139,
153-277): ``NodeRole``, the canonical op sets, ``classify_node``, ``is_trigger``,
``canonicalize_target``, ``build_op_signature``, ``resolve_to_defining_node`` and the
SymInt-safe helpers.

The reference's cost model (``:300-571``) chose between Triton, cuBLAS Lt and eager
from per-architecture tables that end at sm_90.  Here there is one tier, so
:func:`is_compute_bound_gemm` only reports which roof bounds a GEMM on the current
device; the tile / stage decision is made by ``fuseml_sm100_plan`` in the native library.
"""
from __future__ import annotations

from enum import Enum, auto
from typing import Any, Callable, Iterable

import torch

from .._logging import logger

_aten = torch.ops.aten


class NodeRole(Enum):
    TRIGGER = auto()       # seeds a group (addmm / mm)
    ABSORBABLE = auto()    # pointwise, joins the epilogue
    REDUCTION = auto()     # joins as the last op
    BARRIER = auto()       # stops absorption
    TRANSPARENT = auto()   # view / metadata op, absorbed when it keeps the [M, N] shape
    INPLACE = auto()       # in-place pointwise, absorbed when alias-safe
    UNKNOWN = auto()


TRIGGER_OPS: set[Callable] = {_aten.addmm.default, _aten.mm.default}

BARRIER_OPS: set[Callable] = {
    _aten._softmax.default, _aten._log_softmax.default, _aten.native_layer_norm.default,
    _aten.addmm.default, _aten.mm.default, _aten.bmm.default, _aten.convolution.default,
}

ABSORBABLE_OPS: set[Callable] = {
    _aten.relu.default, _aten.gelu.default, _aten.sigmoid.default, _aten.add.Tensor, _aten.mul.Tensor,
}

# Pointwise ops of backward graphs whose first argument is the incoming gradient (the chain value)
# and whose other tensor argument is a saved activation: absorbed only when the pass is asked to
# (backward_ops=True); the forward-only default set above stays what the reference's is.
BACKWARD_ABSORBABLE_OPS: set[Callable] = {_aten.gelu_backward.default}

REDUCTION_OPS: set[Callable] = {_aten.sum.dim_IntList, _aten.amax.default, _aten.mean.dim}

# Whole-tensor reductions: only fused when the pass is asked to (global_reductions=True).
GLOBAL_REDUCTION_OPS: set[Callable] = {_aten.sum.default, _aten.mean.default, _aten.max.default}

TRANSPARENT_OPS: set[Callable] = {
    _aten.view.default, _aten._unsafe_view.default, _aten.reshape.default, _aten.unsqueeze.default,
    _aten.squeeze.dim, _aten.expand.default, _aten.permute.default, _aten.slice.Tensor, _aten.select.int,
    # aten.t is deliberately absent: it swaps M and N and would confuse operand identification
}

INPLACE_OPS: set[Callable] = {
    _aten.relu_.default, _aten.add_.Tensor, _aten.mul_.Tensor, _aten.sigmoid_.default,
}

_ROLE_ORDER: tuple[tuple[set, NodeRole], ...] = (
    (INPLACE_OPS, NodeRole.INPLACE),
    (REDUCTION_OPS, NodeRole.REDUCTION),
    (TRANSPARENT_OPS, NodeRole.TRANSPARENT),
    (ABSORBABLE_OPS, NodeRole.ABSORBABLE),
    (BARRIER_OPS, NodeRole.BARRIER),
)


def classify_node(node: torch.fx.Node) -> NodeRole:
    """Role of ``node`` as a *successor* in a chain (a second addmm is a BARRIER; whether a
    node may *start* a chain is :func:`is_trigger`)."""
    if node.op != "call_function":
        return NodeRole.UNKNOWN
    target = node.target
    for ops, role in _ROLE_ORDER:
        if target in ops:
            return role
    return NodeRole.UNKNOWN


def is_trigger(node: torch.fx.Node) -> bool:
    return node.op == "call_function" and node.target in TRIGGER_OPS


def canonicalize_target(target: Any) -> str:
    """Stable string for an FX target (``"aten.addmm.default"`` for ATen overloads)."""
    text = str(target)
    if text and text != "<unknown>":
        return text
    return getattr(target, "__qualname__", None) or repr(target)


def build_op_signature(nodes: Iterable[torch.fx.Node]) -> tuple[str, ...]:
    return tuple(canonicalize_target(n.target) for n in nodes if n.op == "call_function")


def resolve_to_defining_node(node: torch.fx.Node) -> torch.fx.Node:
    """Walk back through view / metadata ops (``args[0]``) to the node that produced the data."""
    seen: set = set()
    cur = node
    while cur.op == "call_function" and cur.target in TRANSPARENT_OPS and cur not in seen:
        seen.add(cur)
        if not cur.args or not isinstance(cur.args[0], torch.fx.Node):
            break
        cur = cur.args[0]
    return cur


# Views that only regroup dimensions: element order in memory is what it was.
RESHAPE_OPS: set[Callable] = {_aten.view.default, _aten._unsafe_view.default, _aten.reshape.default}


def resolve_through_reshapes(node: torch.fx.Node) -> torch.fx.Node:
    """Like :func:`resolve_to_defining_node`, but only through pure reshapes.  A group input
    found this way can be handed to the kernel in place of the view: flattening it again gives
    the same elements in the same order.  (Behind a permute, slice, select or expand the
    defining tensor holds *different* elements per position, so those views stay the input.)"""
    seen: set = set()
    cur = node
    while cur.op == "call_function" and cur.target in RESHAPE_OPS and cur not in seen:
        seen.add(cur)
        if not cur.args or not isinstance(cur.args[0], torch.fx.Node):
            break
        cur = cur.args[0]
    return cur


def reduction_axis_code(dims: Any, rank: int) -> str | None:
    """Which kernel reduction a ``dim`` argument means for an input of ``rank`` dimensions whose
    leading dimensions are the flattened rows: 'n' (over the last dimension: one result per
    row), 'm' (2-D only: one result per column), 'all', or None (not a reduction the kernel runs,
    e.g. over the sequence dimension of a [B, S, N] tensor)."""
    if rank < 1:
        return None
    if dims is None or dims == [] or dims == ():
        return "all"
    if isinstance(dims, int):
        dims = [dims]
    try:
        norm = tuple(sorted({int(d) % rank for d in dims}))
    except (TypeError, ValueError):
        return None
    if norm == tuple(range(rank)):
        return "all"
    if norm == (rank - 1,):
        return "n"
    if rank == 2 and norm == (0,):
        return "m"
    return None


def classify_epilogue_operand(shape: Any, rows: int, n_cols: int) -> str | None:
    """How an outside operand of ``shape`` lines up with chain values of ``rows`` flattened rows
    and ``n_cols`` columns (visible shape ``[..., n_cols]``, any grouping of the rows):
    'scalar', 'row' (one value per column), 'col' (one value per row), 'full', or None when it
    broadcasts some other way (e.g. ``[S, N]`` against ``[B, S, N]``)."""
    try:
        s = tuple(int(v) for v in shape)
        rows, n_cols = int(rows), int(n_cols)
    except (TypeError, ValueError):
        return None
    one_d = len(s) == 1
    numel = 1
    for v in s:
        numel *= v
    if numel == 1:
        return "scalar"
    while len(s) > 1 and s[0] == 1:
        s = s[1:]
    if s == (n_cols,):
        return "row"
    if one_d:
        # the reference's 1-D rule: length N runs along N, else length M along M
        return "col" if s == (rows,) else None
    lead = 1
    for v in s[:-1]:
        lead *= v
    if lead == rows and s[-1] == n_cols:
        return "full"
    if lead == rows and s[-1] == 1:
        return "col"
    return None


# ---- SymInt-safe helpers ------------------------------------------------------------

def symint_safe_eq(a: Any, b: Any) -> bool:
    """``a == b`` that answers False instead of raising on unresolved symbolic ints."""
    try:
        return bool(a == b)
    except Exception:
        return False


def symint_safe_len(shape: Any) -> int | None:
    try:
        return len(shape)
    except Exception:
        return None


def symint_safe_materialize(vals: Any) -> tuple[int, ...] | None:
    """Concrete ints for a shape / stride tuple, or None if any entry is still symbolic."""
    try:
        return tuple(int(v) for v in vals)
    except Exception:
        return None


# ---- roofline router (Python face) -----------------------------------------------------

_BYTES_PER_ELEM = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.int8: 1}

# Published dense figures for the parts this package targets; used when no device is present.
_B200_TENSOR_FLOPS = 2.25e15
_B200_HBM_BYTES_PER_S = 7.7e12

_cached_gpu_specs: Any = False  # False = not queried yet


def _get_gpu_specs() -> tuple[float, float] | None:
    """``(dense bf16 FLOP/s, HBM bytes/s)`` of the current device, or None without CUDA."""
    global _cached_gpu_specs
    if _cached_gpu_specs is not False:
        return _cached_gpu_specs
    specs = None
    try:
        if torch.cuda.is_available():
            props = torch.cuda.get_device_properties(torch.cuda.current_device())
            if props.major == 10:
                # scale the published 148-SM figures by the SM count actually exposed
                frac = props.multi_processor_count / 148.0
                specs = (_B200_TENSOR_FLOPS * frac, _B200_HBM_BYTES_PER_S)
            else:
                specs = (2.0e12 * props.multi_processor_count, 1.0e12)
    except Exception:  # pragma: no cover - defensive
        specs = None
    _cached_gpu_specs = specs
    return specs


def gemm_roofline(M: int, N: int, K: int, dtype: Any = torch.bfloat16, num_epilogue_ops: int = 1,
                  specs: tuple[float, float] | None = None) -> dict:
    """Roofline figures of one fused GEMM: flops, algorithmic bytes, both times, the bound."""
    flops_rate, bw = specs or _get_gpu_specs() or (_B200_TENSOR_FLOPS, _B200_HBM_BYTES_PER_S)
    bpe = _BYTES_PER_ELEM.get(dtype, 2)
    flops = 2.0 * M * N * K
    if dtype == torch.float32:
        flops_rate = flops_rate / 2.0 / 3.0   # TF32 at half rate, three products per fp32 product
    nbytes = float(bpe) * (M * K + K * N + M * N)
    t_tensor = flops / flops_rate
    t_hbm = nbytes / bw
    # what unfused execution would add: one [M,N] round trip per absorbed op
    saved = 2.0 * M * N * bpe * max(num_epilogue_ops, 0) / bw
    return {"flops": flops, "bytes": nbytes, "t_tensor": t_tensor, "t_hbm": t_hbm,
            "bound": "tensor" if t_tensor >= t_hbm else "hbm", "t_saved_by_fusion": saved}


def is_compute_bound_gemm(M: int, N: int, K: int, dtype: Any = torch.bfloat16, num_epilogue_ops: int = 1,
                          min_penalty: float = 0.0) -> bool:
    """True when the tensor roof, not HBM, bounds this GEMM on the current device.

    Same signature as the reference's cost-model entry (fuseml/passes/topology.py:479-571).
    There it decided "hand the matmul to cuBLAS"; here both answers run the same fused kernel,
    the answer only tells which roofline the launch is measured against.  ``min_penalty`` is
    accepted for compatibility and ignored (there is no per-tier dispatch penalty).
    """
    r = gemm_roofline(M, N, K, dtype, num_epilogue_ops)
    logger.debug("roofline M=%d N=%d K=%d: tensor %.1f us, hbm %.1f us -> %s",
                 M, N, K, r["t_tensor"] * 1e6, r["t_hbm"] * 1e6, r["bound"])
    return r["bound"] == "tensor"
