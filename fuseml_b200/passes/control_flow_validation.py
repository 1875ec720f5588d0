"""Refuse graphs whose trace baked in a data-dependent branch.

Tracing evaluates Python ``if`` / ``while`` on tensors once and records a single path;
compiling that path into fused kernels would be silently wrong for other inputs.  Two
tiers, as in the reference (fuseml/passes/control_flow_validation.py:158-401):

1. the FX graph: higher-order control-flow ops (``cond``, ``while_loop``, ``map_impl``),
   scalar extraction (``.item()``, ``.tolist()``, ``.bool()``), boolean reductions feeding
   one; ``where(comparison, ...)`` is only a warning;
2. the source of the original callable (when given): ``if`` / ``while`` / ``for`` whose
   condition calls a tensor reduction or extraction method.

Errors raise :class:`ControlFlowError`; the compiler then leaves the module to eager.
"""
from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass
from typing import Any, Callable, Literal, Sequence

import torch

from .._logging import logger

_aten = torch.ops.aten


@dataclass
class ControlFlowViolation:
    node_name: str
    description: str
    severity: Literal["error", "warning"] = "error"

    def __str__(self) -> str:
        return f"[{self.severity.upper()}] {self.node_name}: {self.description}"


class ControlFlowError(Exception):
    def __init__(self, violations: Sequence[ControlFlowViolation],
                 warnings: Sequence[ControlFlowViolation] | None = None) -> None:
        self.violations = list(violations)
        self.warnings = list(warnings or [])
        joined = "; ".join(str(v) for v in self.violations)
        super().__init__(f"Data-dependent control flow detected in traced graph — "
                         f"{len(self.violations)} violation(s): {joined}")


_SCALAR_EXTRACTION_METHODS = frozenset({"item", "tolist", "bool"})
_COMPARISON_OPS: frozenset[Callable] = frozenset(
    getattr(getattr(_aten, name), overload)
    for name in ("gt", "lt", "ge", "le", "eq", "ne") for overload in ("Scalar", "Tensor"))
_BOOLEAN_REDUCTION_OPS: frozenset[Callable] = frozenset(
    {_aten.any.default, _aten.any.dim, _aten.all.default, _aten.all.dim})
_WHERE_OPS: frozenset[Callable] = frozenset({_aten.where.self, _aten.where.ScalarSelf, _aten.where.ScalarOther})
_HIGHER_ORDER_CF_NAMES = frozenset({"cond", "while_loop", "map_impl"})

_TENSOR_REDUCTION_ATTRS = frozenset({
    "item", "tolist", "bool", "sum", "mean", "max", "min", "prod", "any", "all", "argmax", "argmin",
    "norm", "count_nonzero"})
_SAFE_CONDITION_ATTRS = frozenset({"training"})


def _check_graph_nodes(gm: torch.fx.GraphModule):
    """Tier 1.  Returns ``(errors, warnings)``."""
    errors: list[ControlFlowViolation] = []
    warnings: list[ControlFlowViolation] = []
    for node in gm.graph.nodes:
        if node.op == "call_function":
            name = getattr(node.target, "__name__", str(node.target))
            if name in _HIGHER_ORDER_CF_NAMES:
                errors.append(ControlFlowViolation(
                    node.name, f"Higher-order control flow op '{name}' detected — the graph contains an "
                               f"explicit conditional branch that cannot be compiled to one static path."))
                continue
            if node.target in _BOOLEAN_REDUCTION_OPS:
                for user in node.users:
                    if user.op == "call_method" and user.target in _SCALAR_EXTRACTION_METHODS:
                        errors.append(ControlFlowViolation(
                            node.name, f"Boolean reduction '{name}' feeds scalar extraction method "
                                       f"'.{user.target}()' — likely used in data-dependent control flow."))
            if node.target in _WHERE_OPS:
                cond = node.args[0] if node.args else None
                if (isinstance(cond, torch.fx.Node) and cond.op == "call_function"
                        and cond.target in _COMPARISON_OPS):
                    warnings.append(ControlFlowViolation(
                        node.name, "torch.where with a comparison condition detected — may be a flattened "
                                   "data-dependent if/else; check the original source.", "warning"))
        elif node.op == "call_method" and node.target in _SCALAR_EXTRACTION_METHODS:
            if not any(v.node_name == node.name for v in errors):
                errors.append(ControlFlowViolation(
                    node.name, f"Tensor scalar extraction method '.{node.target}()' found in the traced graph "
                               f"— the value was probably used in Python control flow that is now baked in."))
    return errors, warnings


class _ControlFlowVisitor(ast.NodeVisitor):
    """Tier 2: flags if / while / for whose condition involves a tensor-derived value."""

    def __init__(self) -> None:
        self.violations: list[ControlFlowViolation] = []

    @staticmethod
    def _is_safe_receiver(node: ast.AST) -> bool:
        return isinstance(node, ast.Attribute) and node.attr in _SAFE_CONDITION_ATTRS

    def _involves_tensor_op(self, node: ast.AST) -> bool:
        if isinstance(node, ast.Call):
            f = node.func
            if isinstance(f, ast.Attribute) and f.attr in _TENSOR_REDUCTION_ATTRS and not self._is_safe_receiver(f.value):
                return True
            return any(self._involves_tensor_op(a) for a in node.args) or \
                any(self._involves_tensor_op(k.value) for k in node.keywords)
        if isinstance(node, ast.Compare):
            return self._involves_tensor_op(node.left) or any(self._involves_tensor_op(c) for c in node.comparators)
        if isinstance(node, ast.BoolOp):
            return any(self._involves_tensor_op(v) for v in node.values)
        if isinstance(node, ast.UnaryOp):
            return self._involves_tensor_op(node.operand)
        if isinstance(node, ast.BinOp):
            return self._involves_tensor_op(node.left) or self._involves_tensor_op(node.right)
        if isinstance(node, ast.Attribute):
            return node.attr in _TENSOR_REDUCTION_ATTRS and not self._is_safe_receiver(node.value)
        return False

    def _record(self, stmt: ast.stmt, kind: str) -> None:
        line = getattr(stmt, "lineno", "?")
        self.violations.append(ControlFlowViolation(
            f"source:L{line}", f"Data-dependent '{kind}' statement at line {line} — its condition involves "
                               f"tensor-derived value(s) that tracing bakes into a single path."))

    def visit_If(self, node: ast.If) -> None:
        if self._involves_tensor_op(node.test):
            self._record(node, "if")
        self.generic_visit(node)

    def visit_While(self, node: ast.While) -> None:
        if self._involves_tensor_op(node.test):
            self._record(node, "while")
        self.generic_visit(node)

    def visit_For(self, node: ast.For) -> None:
        if self._involves_tensor_op(node.iter):
            self._record(node, "for")
        self.generic_visit(node)


def _check_source_ast(callable_obj: Any) -> list[ControlFlowViolation]:
    target = callable_obj
    if hasattr(target, "forward") and callable(target.forward):
        target = target.forward
    try:
        tree = ast.parse(textwrap.dedent(inspect.getsource(target)))
    except (OSError, TypeError, SyntaxError):
        return []
    visitor = _ControlFlowVisitor()
    visitor.visit(tree)
    return visitor.violations


def validate_graph_control_flow(gm: torch.fx.GraphModule, original_callable: Any | None = None) -> None:
    """Raise :class:`ControlFlowError` if ``gm`` (or the source of ``original_callable``) shows
    data-dependent control flow; log warnings otherwise."""
    errors, warnings = _check_graph_nodes(gm)
    if original_callable is not None:
        errors.extend(_check_source_ast(original_callable))
    for w in warnings:
        logger.warning("Control flow advisory: %s", w)
    if errors:
        raise ControlFlowError(errors, warnings)
    logger.debug("control-flow validation passed")
