"""fuseml_b200 — B200-native (sm_100a) fused-kernel backend with FuseML's API.

``torch.compile(model, backend=FuseMLCompiler())`` keeps working; matched
``addmm``/``mm`` + epilogue chains run as hand-written TMA + tcgen05 kernels
through the C ABI in ``include/fuseml_sm100.h``.  The names the reference package
exports (fuseml/__init__.py:59-98) are exported here too.
"""
from . import _native  # noqa: F401
from .codegen import (CublasEpilogueLauncher, CublasEpiloguePattern, CublasResidualLauncher, EagerFallbackGuard,  # noqa: F401
                      KernelCache, KernelCacheKey, KernelLauncher, KernelSpec, LaunchParams, ReductionInfo,
                      Sm100KernelGenerator, SRAMAutotuner, TensorDescriptor, TensorFingerprint,
                      TritonKernelGenerator, TuneConfig, build_cache_key, build_op_chain,
                      compute_launch_params, compute_sram_bytes, cublas_epilogue_available,
                      generate_sram_safe_configs, match_cublas_epilogue, next_power_of_2)
from .compiler import FuseMLCompiler  # noqa: F401
from .fusion_group import FusionGroup  # noqa: F401
from .kernels import EpilogueProgram, device_status, fused_gemm, reduce_tail  # noqa: F401
from .passes.control_flow_validation import ControlFlowError, validate_graph_control_flow  # noqa: F401
from .passes.fusion_pass import FuseMLFusionPass, fuseml_fused_kernel_placeholder  # noqa: F401
from .passes.graph_cut import (SUPPORTED_EPILOGUE_OPS, SUPPORTED_TRITON_OPS, GraphSegment,  # noqa: F401
                               split_fusion_group, validate_fusion_group)
from .passes.mutation_safety import IN_PLACE_OPS, MutationFinding, is_safe_inplace  # noqa: F401
from .passes.topology import (NodeRole, build_op_signature, canonicalize_target, classify_node, is_trigger,  # noqa: F401
                              resolve_to_defining_node, symint_safe_eq, symint_safe_materialize)
from .registry import SupportedOpsRegistry, build_default_registry  # noqa: F401

__version__ = "0.1.0"
