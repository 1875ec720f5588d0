"""Back half of the compiler: lowering, launch, cache, tile chooser."""
from .cublas_epilogue import (CublasEpilogueLauncher, CublasEpiloguePattern, CublasResidualLauncher,  # noqa: F401
                              cublas_epilogue_available, match_cublas_epilogue)
from .eager_fallback import EagerFallbackGuard  # noqa: F401
from .kernel_cache import KernelCache, KernelCacheKey, TensorFingerprint, build_cache_key, build_op_chain  # noqa: F401
from .kernel_generator import (KernelSpec, ReductionInfo, Sm100KernelGenerator, TensorDescriptor,  # noqa: F401
                               TritonKernelGenerator, next_power_of_2)
from .kernel_launcher import KernelLauncher, LaunchParams, compute_launch_params  # noqa: F401
from .sram_autotuner import SRAMAutotuner, TuneConfig, compute_sram_bytes, generate_sram_safe_configs  # noqa: F401
