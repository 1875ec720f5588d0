"""The three "library epilogue" patterns of the reference, as ordinary epilogue programs.

The reference routed compute-bound GEMMs to cuBLAS Lt when the chain was exactly
``addmm -> gelu``, ``addmm -> relu`` or ``addmm -> add(residual)``
(fuseml/codegen/cublas_epilogue.py:166-258; launchers ``:586-679``; the inline cublasLt
extension ``:355-571``).  No cuBLAS runs on a fused path here: the same patterns are just
short programs of the sm_100a kernel.  The matcher and the pattern dataclass are kept
(structural only: no availability gating), the launcher names resolve to the one launcher.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from .kernel_launcher import KernelLauncher

_aten = torch.ops.aten


def cublas_epilogue_available() -> bool:
    """Always False: fused paths never call cuBLAS Lt in this package."""
    return False


@dataclass
class CublasEpiloguePattern:
    epilogue_type: str                 # "GELU_BIAS" | "RELU_BIAS" | "BIAS_RESIDUAL"
    trigger_node: Any
    absorbed_nodes: list = field(default_factory=list)
    output_node: Any = None
    has_bias: bool = True
    use_gelu: bool = True
    residual_arg_index: int | None = None

    def program(self) -> tuple[str, ...]:
        """The epilogue program this pattern lowers to (op names of the sm_100a kernel)."""
        return {"GELU_BIAS": ("add_t", "gelu_erf"), "RELU_BIAS": ("add_t", "relu"),
                "BIAS_RESIDUAL": ("add_t", "add_t")}[self.epilogue_type]


def match_cublas_epilogue(trigger_node: torch.fx.Node) -> CublasEpiloguePattern | None:
    """Structural match of ``addmm`` followed by exactly one gelu (erf) / relu / add(residual)."""
    if trigger_node.target is not _aten.addmm.default or len(trigger_node.args) < 3:
        return None
    if len(trigger_node.users) != 1:
        return None
    nxt = next(iter(trigger_node.users))
    if nxt.op != "call_function":
        return None
    if nxt.target is _aten.gelu.default:
        if nxt.kwargs.get("approximate", "none") not in ("none", None):
            return None
        return CublasEpiloguePattern("GELU_BIAS", trigger_node, [nxt], nxt, True, True)
    if nxt.target in (_aten.relu.default, _aten.relu_.default):
        return CublasEpiloguePattern("RELU_BIAS", trigger_node, [nxt], nxt, True, False)
    if nxt.target in (_aten.add.Tensor, _aten.add_.Tensor) and len(nxt.args) >= 2:
        a0, a1 = nxt.args[0], nxt.args[1]
        if isinstance(a0, torch.fx.Node) and isinstance(a1, torch.fx.Node) and (a0 is trigger_node) != (a1 is trigger_node):
            return CublasEpiloguePattern("BIAS_RESIDUAL", trigger_node, [nxt], nxt, True, False,
                                         residual_arg_index=1 if a0 is trigger_node else 0)
    return None


# The reference had one launcher class per library call; both are the fused launcher now.
CublasEpilogueLauncher = KernelLauncher
CublasResidualLauncher = KernelLauncher
