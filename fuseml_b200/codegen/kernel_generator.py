"""From a FusionGroup to a kernel specification.

The reference's generator emitted ``@triton.jit`` source for every group
(fuseml/codegen/kernel_generator.py:326-2043) and compiled it from a temp file.  Here
the kernels are precompiled sm_100a code, so "code generation" reduces to *lowering*:
walk the group's nodes in execution order and produce a :class:`KernelSpec` — which
inputs are the GEMM operands, the epilogue program as ``(opcode, input index | immediate)``
steps, the reductions, what is stored.  The launcher binds live tensors to that spec at
call time.  Names the reference exports are kept: ``TensorDescriptor``, ``ReductionInfo``,
``next_power_of_2``, ``_classify``, ``_identify_matmul_operands`` and the generator class
(``Sm100KernelGenerator``, also importable as ``TritonKernelGenerator``).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch

from .. import _native as N
from .._logging import logger
from ..passes.topology import GLOBAL_REDUCTION_OPS, REDUCTION_OPS, TRANSPARENT_OPS, reduction_axis_code

_aten = torch.ops.aten


@dataclass(frozen=True)
class ReductionInfo:
    """``axis``: tile axis that is collapsed (0 = M, 1 = N, 2 = both); ``op``: sum | max | mean."""
    axis: int
    op: str
    keepdim: bool = False


@dataclass(frozen=True)
class TensorDescriptor:
    """Name, concrete shape / stride, dtype and 16-byte alignment of one kernel argument
    (same fields as the reference's, fuseml/codegen/kernel_generator.py:165-186)."""
    name: str
    shape: tuple
    stride: tuple
    dtype: torch.dtype
    aligned: bool = True


def next_power_of_2(val: int) -> int:
    val = int(val)
    return 1 if val <= 1 else 1 << (val - 1).bit_length()


def _classify(tensors: Sequence[TensorDescriptor]):
    """Split descriptors into 2-D matrices and 1-D vectors."""
    return [t for t in tensors if len(t.shape) == 2], [t for t in tensors if len(t.shape) == 1]


def _identify_matmul_operands(matrices: Sequence[TensorDescriptor]):
    """(left[M,K], right[K,N]) among the first two matrices, trying both orders
    (fuseml/codegen/kernel_generator.py:293-319)."""
    m0, m1 = matrices[0], matrices[1]
    if m0.shape[1] == m1.shape[0]:
        return m0, m1
    if m1.shape[1] == m0.shape[0]:
        return m1, m0
    raise ValueError(f"Contracting dimension mismatch: {m0.name}{m0.shape} vs {m1.name}{m1.shape}")


class UnsupportedChainError(ValueError):
    """The group contains something the epilogue program cannot express."""


@dataclass(frozen=True)
class EpiStep:
    opcode: int
    input_index: int = -1     # index into FusionGroup.inputs for *_T steps
    imm: float = 0.0
    aux_index: int = -1       # which intermediate output a STORE_AUX step writes


@dataclass
class KernelSpec:
    """Everything static about one fused kernel."""
    left_index: int
    right_index: int
    steps: tuple = ()
    reductions: tuple = ()            # ReductionInfo per reduction output, in output order
    store_output: bool = True
    n_inputs: int = 0
    n_aux: int = 0
    op_chain: tuple = ()

    def signature(self) -> str:
        """Stable digest of the lowering (the analogue of the reference's SHA-256 source cache,
        fuseml/codegen/kernel_generator.py:1067-1172)."""
        h = hashlib.sha256()
        h.update(repr((self.left_index, self.right_index,
                       tuple((s.opcode, s.input_index, round(s.imm, 9), s.aux_index) for s in self.steps),
                       tuple((r.axis, r.op) for r in self.reductions), self.store_output)).encode())
        return h.hexdigest()

    @property
    def uses_second_register(self) -> bool:
        return any(s.opcode in (N.OP_SAVE, N.OP_SWAP, N.OP_ADD_SAVED, N.OP_MUL_SAVED) for s in self.steps)


_UNARY = {
    _aten.relu.default: N.OP_RELU, _aten.relu_.default: N.OP_RELU,
    _aten.sigmoid.default: N.OP_SIGMOID, _aten.sigmoid_.default: N.OP_SIGMOID,
}
_ADD = (_aten.add.Tensor, _aten.add_.Tensor)
_MUL = (_aten.mul.Tensor, _aten.mul_.Tensor)
_RED_KIND = {
    _aten.sum.dim_IntList: "sum", _aten.amax.default: "max", _aten.mean.dim: "mean",
    _aten.sum.default: "sum", _aten.mean.default: "mean", _aten.max.default: "max",
}


def _args_of(group: Any, node: Any) -> tuple:
    """Node args, from the pre-surgery snapshot when the node has been erased since."""
    snap = getattr(group, "node_args_snapshot", None) or {}
    return snap.get(node.name, tuple(node.args))


class Sm100KernelGenerator:
    """Lowers FusionGroups to :class:`KernelSpec`."""

    def __init__(self) -> None:
        self._spec_cache: dict[str, KernelSpec] = {}

    # ------------------------------------------------------------------ public
    def build_spec(self, group: Any) -> KernelSpec:
        inputs = list(group.inputs)
        index_of = {id(n): i for i, n in enumerate(inputs)}
        for i, n in enumerate(getattr(group, "original_inputs", None) or []):
            index_of.setdefault(id(n), i)

        def input_index(node: Any) -> int:
            """Index of an external operand: the node itself or what it is a view of."""
            cur = node
            for _ in range(16):
                if id(cur) in index_of:
                    return index_of[id(cur)]
                if getattr(cur, "op", None) == "call_function" and cur.target in TRANSPARENT_OPS and cur.args:
                    cur = cur.args[0]
                    continue
                break
            raise UnsupportedChainError(f"operand {getattr(node, 'name', node)} is not an input of the group")

        base = group.base_node
        bargs = _args_of(group, base)
        steps: list[EpiStep] = []
        if base.target is _aten.addmm.default:
            bias, left, right = bargs[0], bargs[1], bargs[2]
            beta = float(base.kwargs.get("beta", 1))
            alpha = float(base.kwargs.get("alpha", 1))
            if beta == 0.0:
                if alpha != 1.0:
                    steps.append(EpiStep(N.OP_MUL_IMM, imm=alpha))
            else:
                # beta*bias + alpha*acc  ==  beta * (acc * alpha/beta + bias)
                if alpha / beta != 1.0:
                    steps.append(EpiStep(N.OP_MUL_IMM, imm=alpha / beta))
                steps.append(EpiStep(N.OP_ADD_T, input_index(bias)))
                if beta != 1.0:
                    steps.append(EpiStep(N.OP_MUL_IMM, imm=beta))
        elif base.target is _aten.mm.default:
            left, right = bargs[0], bargs[1]
        else:
            raise UnsupportedChainError(f"base node {base.target} is not addmm / mm")
        left_i, right_i = input_index(left), input_index(right)

        members = {id(n) for n in group.all_nodes}
        aux_nodes = list(getattr(group, "intermediate_outputs", []) or [])
        extra = list(getattr(group, "extra_outputs", []) or [])
        reductions: list[ReductionInfo] = []
        # value tracking for diamonds: which node's value sits in `acc` / `saved`
        acc_of: Any = base
        saved_of: Any = None
        pending = [n for n in group.fused_nodes]
        # readers of each value inside the group, counted from the recorded args (the nodes may
        # already have been erased from the graph, which empties ``node.users``)
        fork_users: dict[int, int] = {id(n): 0 for n in group.all_nodes}
        for n in group.all_nodes:
            if n is base or n.target in _RED_KIND or n.target in TRANSPARENT_OPS:
                continue
            seen_here = set()
            for a in _args_of(group, n):
                while getattr(a, "op", None) == "call_function" and a.target in TRANSPARENT_OPS and id(a) in members:
                    a = _args_of(group, a)[0]
                if hasattr(a, "op") and id(a) in members and id(a) not in seen_here:
                    seen_here.add(id(a))
                    fork_users[id(a)] += 1

        def emit_aux_if_needed(node: Any) -> None:
            if node in aux_nodes:
                steps.append(EpiStep(N.OP_STORE_AUX, aux_index=aux_nodes.index(node)))

        emit_aux_if_needed(base)
        if fork_users.get(id(base), 0) >= 2:
            steps.append(EpiStep(N.OP_SAVE))
            saved_of = base

        def resolve(v: Any) -> Any:
            """look through views absorbed into the group"""
            while getattr(v, "op", None) == "call_function" and v.target in TRANSPARENT_OPS and id(v) in members:
                v = _args_of(group, v)[0]
            return v

        for node in pending:
            tgt = node.target
            if tgt in TRANSPARENT_OPS:
                continue
            if tgt in _RED_KIND:
                reductions.append(self._reduction_info(group, node))
                continue
            args = _args_of(group, node)
            tensor_args = [resolve(a) for a in args if hasattr(a, "op")]
            inside = [a for a in tensor_args if id(a) in members]
            # make sure the value this op consumes is in `acc`
            if inside and all(a is not acc_of for a in inside):
                if saved_of is not None and any(a is saved_of for a in inside):
                    steps.append(EpiStep(N.OP_SWAP))
                    acc_of, saved_of = saved_of, acc_of
                else:
                    raise UnsupportedChainError(f"{node.name}: operand order needs more than two value registers")
            if tgt in _UNARY:
                steps.append(EpiStep(_UNARY[tgt]))
            elif tgt is _aten.gelu.default:
                approx = node.kwargs.get("approximate", "none")
                steps.append(EpiStep(N.OP_GELU_TANH if approx == "tanh" else N.OP_GELU_ERF))
            elif tgt is _aten.gelu_backward.default:
                # gelu_backward(grad, self, approximate): grad is the chain value, self a saved activation
                approx = node.kwargs.get("approximate", args[2] if len(args) > 2 else "none")
                if approx != "none":
                    raise UnsupportedChainError(f"{node.name}: gelu_backward(approximate={approx!r}) has no epilogue op")
                if len(inside) != 1 or resolve(args[0]) is not acc_of:
                    raise UnsupportedChainError(f"{node.name}: the chain value must be the gradient argument")
                steps.append(EpiStep(N.OP_GELU_ERF_BWD_T, input_index(args[1])))
            elif tgt in _ADD or tgt in _MUL:
                is_add = tgt in _ADD
                alpha = float(node.kwargs.get("alpha", 1)) if is_add else 1.0
                scalars = [a for a in args if isinstance(a, (int, float)) and not isinstance(a, bool)]
                if len(inside) == 2:
                    a0, a1 = inside
                    if a0 is a1:
                        if is_add:
                            steps.append(EpiStep(N.OP_MUL_IMM, imm=1.0 + alpha))
                        else:
                            steps += [EpiStep(N.OP_SAVE), EpiStep(N.OP_MUL_SAVED)]
                            saved_of = acc_of
                    else:
                        other = a1 if a0 is acc_of else a0
                        if other is not saved_of:
                            raise UnsupportedChainError(f"{node.name}: second operand is not in the saved register")
                        if is_add and alpha != 1.0:
                            raise UnsupportedChainError(f"{node.name}: add with alpha between two chain values")
                        steps.append(EpiStep(N.OP_ADD_SAVED if is_add else N.OP_MUL_SAVED))
                elif scalars:
                    c = float(scalars[0]) * (alpha if is_add else 1.0)
                    steps.append(EpiStep(N.OP_ADD_IMM if is_add else N.OP_MUL_IMM, imm=c))
                else:
                    ext = [a for a in tensor_args if id(a) not in members]
                    if len(ext) != 1:
                        raise UnsupportedChainError(f"{node.name}: cannot identify the external operand")
                    if is_add and alpha != 1.0:
                        # acc + alpha*t  ==  alpha * (acc/alpha + t)
                        steps.append(EpiStep(N.OP_MUL_IMM, imm=1.0 / alpha))
                        steps.append(EpiStep(N.OP_ADD_T, input_index(ext[0])))
                        steps.append(EpiStep(N.OP_MUL_IMM, imm=alpha))
                    else:
                        steps.append(EpiStep(N.OP_ADD_T if is_add else N.OP_MUL_T, input_index(ext[0])))
            else:
                raise UnsupportedChainError(f"no epilogue translation for {tgt}")
            acc_of = node
            emit_aux_if_needed(node)
            if fork_users.get(id(node), 0) >= 2:
                steps.append(EpiStep(N.OP_SAVE))
                saved_of = node

        if len(steps) > N.MAX_EPI_OPS:
            raise UnsupportedChainError(f"epilogue of {len(steps)} steps exceeds {N.MAX_EPI_OPS}")
        axes = {r.axis for r in reductions}
        if len(axes) > 1:
            raise UnsupportedChainError("reductions over different axes in one group")
        spec = KernelSpec(left_index=left_i, right_index=right_i, steps=tuple(steps),
                          reductions=tuple(reductions),
                          store_output=bool(getattr(group, "store_output", True)),
                          n_inputs=len(inputs), n_aux=len(aux_nodes), op_chain=tuple(group.op_signature))
        # a classic single-reduction group never stores the matrix
        if reductions and not extra and group.output_node.target in _RED_KIND:
            spec.store_output = False
        self._spec_cache.setdefault(spec.signature(), spec)
        logger.debug("lowered %s -> %d epilogue step(s), %d reduction(s)", group, len(steps), len(reductions))
        return spec

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _reduction_info(group: Any, node: Any) -> ReductionInfo:
        kind = _RED_KIND[node.target]
        if node.target in GLOBAL_REDUCTION_OPS:
            return ReductionInfo(axis=2, op=kind)
        args = _args_of(group, node)
        dims = args[1] if len(args) > 1 else []
        # rows are the flattened leading dimensions of the reduced tensor ([B, S, N] -> [B*S, N])
        src = args[0] if args else None
        shape = None
        for key in ("tensor_meta", "val"):
            m = getattr(src, "meta", {}).get(key) if src is not None else None
            if m is not None and hasattr(m, "shape"):
                shape = m.shape
                break
        rank = len(shape) if shape is not None else 2
        axis = {"n": 1, "m": 0, "all": 2}.get(reduction_axis_code(dims, rank))
        if axis is None:
            raise UnsupportedChainError(f"{node.name}: reduction dims {dims} of a rank-{rank} tensor")
        keepdim = bool(args[2]) if len(args) > 2 else False
        if keepdim:
            raise UnsupportedChainError(f"{node.name}: keepdim=True reductions are not fused")
        return ReductionInfo(axis=axis, op=kind)


# historical name kept importable
TritonKernelGenerator = Sm100KernelGenerator
