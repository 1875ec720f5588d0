"""fuseml_b200 — B200-native (sm_100a) fused-kernel backend with FuseML's API.

``torch.compile(model, backend=FuseMLCompiler())`` keeps working; matched
``addmm``/``mm`` + epilogue chains run as hand-written TMA + tcgen05 kernels
through the C ABI in ``include/fuseml_sm100.h``.
"""
from . import _native  # noqa: F401
from .kernels import EpilogueProgram, fused_gemm, reduce_tail, device_status  # noqa: F401

__version__ = "0.1.0"
