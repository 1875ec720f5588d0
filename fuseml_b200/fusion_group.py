"""FusionGroup: one ``trigger -> pointwise... [-> reduction]`` chain cut out of an FX graph.

Field names and meaning follow the reference's dataclass (fuseml/fusion_group.py:18-122)
because graph surgery, the compiler and user code read them: ``inputs`` is ordered and
becomes the fused kernel's argument order; ``output_metadata`` carries
``shape/stride/dtype`` of the chain's result.  Two fields are new and default to "off":
``extra_reductions`` (more than one reduction of the same tensor in one pass) and
``store_output`` (whether the matrix itself is still needed).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class FusionGroup:
    base_node: torch.fx.Node
    fused_nodes: list = field(default_factory=list)
    inputs: list = field(default_factory=list)
    output_node: torch.fx.Node = None  # type: ignore[assignment]
    output_metadata: dict = field(default_factory=dict)
    intermediate_outputs: list = field(default_factory=list)
    param_bindings: dict = field(default_factory=dict)
    node_args_snapshot: dict = field(default_factory=dict)
    fusion_strategy: str = "sm100"
    cublas_pattern: Any = None
    # extensions (see FuseMLFusionPass options)
    extra_outputs: list = field(default_factory=list)   # further reduction nodes fed by the same tensor
    store_output: bool = True                           # False: only reductions leave the kernel
    # inputs as discovery saw them; surgery later swaps entries of ``inputs`` for the fused
    # nodes that replaced them, while recorded node args still name the originals
    original_inputs: list = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.output_node is None:
            self.output_node = self.base_node

    @property
    def all_nodes(self) -> list:
        return [self.base_node, *self.fused_nodes]

    @property
    def op_signature(self) -> tuple[str, ...]:
        """Canonical op names in execution order; independent of node names."""
        from .passes.topology import canonicalize_target

        return tuple(canonicalize_target(n.target) for n in self.all_nodes if n.op == "call_function")

    def __len__(self) -> int:
        return 1 + len(self.fused_nodes)

    def __repr__(self) -> str:
        chain = " -> ".join(n.name for n in self.all_nodes)
        return f"FusionGroup({chain}, inputs={len(self.inputs)})"
