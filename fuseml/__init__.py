"""Drop-in import name: ``import fuseml`` resolves to :mod:`fuseml_b200`.

Existing code written against the reference (``from fuseml import FuseMLCompiler``,
``from fuseml.passes.fusion_pass import FuseMLFusionPass`` ...) keeps working: every
sub-module path of the reference package is aliased to the module of the same role here.
"""
import importlib
import sys

import fuseml_b200 as _impl

_SUBMODULES = (
    "_logging", "registry", "fusion_group", "compiler",
    "passes", "passes.topology", "passes.fusion_pass", "passes.graph_cut", "passes.mutation_safety",
    "passes.control_flow_validation",
    "codegen", "codegen.kernel_generator", "codegen.kernel_launcher", "codegen.kernel_cache",
    "codegen.sram_autotuner", "codegen.cublas_epilogue", "codegen.eager_fallback",
)
for _name in _SUBMODULES:
    _mod = importlib.import_module(f"fuseml_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    if "." not in _name:
        globals()[_name] = _mod

for _k, _v in vars(_impl).items():
    if not _k.startswith("__"):
        globals().setdefault(_k, _v)

__all__ = [k for k in vars(_impl) if not k.startswith("_")]
