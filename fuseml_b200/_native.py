"""ctypes binding of ``libfuseml_sm100.so`` (the C ABI in ``include/fuseml_sm100.h``).

The structures below mirror the header field by field.  There is no Python or
PyTorch fallback: if the library cannot be loaded every launch raises
``RuntimeError`` (the reference instead falls back to eager silently,
fuseml/codegen/cublas_epilogue.py:617-626 — that behaviour is not kept).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

MAX_EPI_OPS = 16
MAX_OPERANDS = 8
ABI_VERSION = 3          # FUSEML_SM100_ABI_VERSION of include/fuseml_sm100.h

# status codes -----------------------------------------------------------------
OK = 0
E_NULL, E_SHAPE, E_DTYPE, E_LAYOUT, E_EPILOGUE, E_REDUCTION = 1, 2, 3, 4, 5, 6
E_WORKSPACE, E_PLAN, E_DEVICE, E_LAUNCH, E_TIMEOUT, E_LIMIT = 7, 8, 9, 10, 11, 12

# dtypes -------------------------------------------------------------------------
BF16, F16, F32 = 0, 1, 2

# opcodes ------------------------------------------------------------------------
OP_NOP, OP_RELU, OP_GELU_ERF, OP_SIGMOID, OP_ADD_IMM, OP_MUL_IMM = 0, 1, 2, 3, 4, 5
OP_ADD_T, OP_MUL_T, OP_SAVE, OP_SWAP, OP_ADD_SAVED, OP_MUL_SAVED = 6, 7, 8, 9, 10, 11
OP_GELU_TANH, OP_STORE_AUX, OP_SUB_T, OP_RSUB_T, OP_GELU_ERF_MUL_SIGMOID, OP_GELU_ERF_BWD_T = 12, 13, 14, 15, 16, 17
OP_NAMES = {
    OP_NOP: "nop", OP_RELU: "relu", OP_GELU_ERF: "gelu_erf", OP_SIGMOID: "sigmoid",
    OP_ADD_IMM: "add_imm", OP_MUL_IMM: "mul_imm", OP_ADD_T: "add_t", OP_MUL_T: "mul_t",
    OP_SAVE: "save", OP_SWAP: "swap", OP_ADD_SAVED: "add_saved", OP_MUL_SAVED: "mul_saved",
    OP_GELU_TANH: "gelu_tanh", OP_STORE_AUX: "store_aux", OP_SUB_T: "sub_t", OP_RSUB_T: "rsub_t",
    OP_GELU_ERF_MUL_SIGMOID: "gelu_erf_mul_sigmoid", OP_GELU_ERF_BWD_T: "gelu_erf_bwd_t",
}

# reductions ---------------------------------------------------------------------
RED_SUM, RED_MAX, RED_MEAN = 1, 2, 4
PLAN_B_EXPANSION_VALID = 1
PLAN_STREAM_K = 2
PLAN_GROUP_N = 4
MLP_WEIGHTS_EXPANDED = 1
WHERE_MMA_FULL = 0x202
AXIS_M, AXIS_N, AXIS_ALL = 0, 1, 2


class EpiOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("slot", C.c_int32), ("imm", C.c_float), ("reserved", C.c_int32)]


class Operand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_m", C.c_int64), ("stride_n", C.c_int64),
                ("dtype", C.c_int32), ("reserved", C.c_int32)]


class Reduce(C.Structure):
    _fields_ = [("kinds", C.c_int32), ("axis", C.c_int32),
                ("out_sum", C.c_void_p), ("out_max", C.c_void_p), ("out_mean", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64)]


class GemmDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("a", C.c_void_p), ("lda", C.c_int64),
        ("b", C.c_void_p), ("b_stride_k", C.c_int64), ("b_stride_n", C.c_int64),
        ("ab_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("d", C.c_void_p), ("ldd", C.c_int64),
        ("n_ops", C.c_int32), ("n_operands", C.c_int32),
        ("ops", EpiOp * MAX_EPI_OPS),
        ("operands", Operand * MAX_OPERANDS),
        ("reduce", Reduce),
        ("a_stride_k", C.c_int64),
    ]


class MlpDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("D_in", C.c_int64), ("I", C.c_int64), ("D_out", C.c_int64),
        ("x", C.c_void_p), ("ldx", C.c_int64),
        ("w1", C.c_void_p), ("ldw1", C.c_int64),
        ("w2", C.c_void_p), ("ldw2", C.c_int64),
        ("ab_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("y", C.c_void_p), ("ldy", C.c_int64),
        ("n_ops1", C.c_int32), ("n_ops2", C.c_int32), ("n_operands", C.c_int32), ("flags", C.c_int32),
        ("ops1", EpiOp * MAX_EPI_OPS), ("ops2", EpiOp * MAX_EPI_OPS),
        ("operands", Operand * MAX_OPERANDS),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
    ]


class Plan(C.Structure):
    _fields_ = [
        ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32), ("stages", C.c_int32),
        ("cluster", C.c_int32), ("acc_stages", C.c_int32), ("grid", C.c_int32), ("group_m", C.c_int32),
        ("smem_bytes", C.c_int32), ("tmem_cols", C.c_int32), ("bound", C.c_int32), ("fuse", C.c_int32),
        ("split_k", C.c_int32), ("flags", C.c_int32),
        ("flops", C.c_double), ("bytes", C.c_double), ("t_tensor_us", C.c_double),
        ("t_hbm_us", C.c_double), ("t_est_us", C.c_double),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


class WorkItem(C.Structure):
    """``fuseml_work_item_t``: one entry of a unit's schedule (``fuseml_sm100_schedule``)."""
    _fields_ = [("tile", C.c_int32), ("kb0", C.c_int32), ("kb1", C.c_int32), ("kind", C.c_int32),
                ("after", C.c_int32), ("slot", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32)]


class DeviceProps(C.Structure):
    _fields_ = [
        ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
        ("smem_per_block_optin", C.c_int32), ("tmem_cols", C.c_int32), ("l2_bytes", C.c_int32),
        ("hbm_gbs", C.c_double), ("tensor_tflops", C.c_double),
    ]


#: every symbol ``include/fuseml_sm100.h`` declares
EXPORTS = (
    "fuseml_sm100_query", "fuseml_sm100_plan", "fuseml_sm100_workspace_bytes", "fuseml_sm100_validate",
    "fuseml_sm100_gemm_epilogue", "fuseml_sm100_reduce_tail", "fuseml_sm100_device_status",
    "fuseml_sm100_strerror", "fuseml_sm100_abi_version",
    "fuseml_sm100_gemm_epilogue_noalloc", "fuseml_sm100_noalloc_scratch_bytes",
    "fuseml_sm100_set_diagnostics", "fuseml_sm100_mlp_small", "fuseml_sm100_mlp_small_workspace_bytes",
    "fuseml_sm100_schedule",
)

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfuseml_sm100.so"

_lib = None
_lock = threading.Lock()


class NativeLibraryError(RuntimeError):
    """The sm_100a library is missing or a call into it failed."""


def _declare(lib: C.CDLL) -> None:
    lib.fuseml_sm100_abi_version.restype = C.c_int
    lib.fuseml_sm100_abi_version.argtypes = []
    lib.fuseml_sm100_strerror.restype = C.c_char_p
    lib.fuseml_sm100_strerror.argtypes = [C.c_int]
    lib.fuseml_sm100_query.restype = C.c_int
    lib.fuseml_sm100_query.argtypes = [C.POINTER(DeviceProps)]
    lib.fuseml_sm100_plan.restype = C.c_int
    lib.fuseml_sm100_plan.argtypes = [C.POINTER(GemmDesc), C.POINTER(DeviceProps), C.POINTER(Plan)]
    lib.fuseml_sm100_workspace_bytes.restype = C.c_int64
    lib.fuseml_sm100_workspace_bytes.argtypes = [C.POINTER(GemmDesc), C.POINTER(Plan)]
    lib.fuseml_sm100_validate.restype = C.c_int
    lib.fuseml_sm100_validate.argtypes = [C.POINTER(GemmDesc)]
    lib.fuseml_sm100_gemm_epilogue.restype = C.c_int
    lib.fuseml_sm100_gemm_epilogue.argtypes = [C.POINTER(GemmDesc), C.POINTER(Plan), C.c_void_p]
    lib.fuseml_sm100_gemm_epilogue_noalloc.restype = C.c_int
    lib.fuseml_sm100_gemm_epilogue_noalloc.argtypes = [C.POINTER(GemmDesc), C.POINTER(Plan), C.c_void_p]
    lib.fuseml_sm100_noalloc_scratch_bytes.restype = C.c_int64
    lib.fuseml_sm100_noalloc_scratch_bytes.argtypes = []
    lib.fuseml_sm100_reduce_tail.restype = C.c_int
    lib.fuseml_sm100_reduce_tail.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                             C.POINTER(Reduce), C.c_void_p]
    lib.fuseml_sm100_mlp_small.restype = C.c_int
    lib.fuseml_sm100_mlp_small.argtypes = [C.POINTER(MlpDesc), C.c_void_p]
    lib.fuseml_sm100_mlp_small_workspace_bytes.restype = C.c_int64
    lib.fuseml_sm100_mlp_small_workspace_bytes.argtypes = [C.POINTER(MlpDesc)]
    lib.fuseml_sm100_set_diagnostics.restype = C.c_int
    lib.fuseml_sm100_set_diagnostics.argtypes = [C.c_int64, C.c_int32]
    lib.fuseml_sm100_device_status.restype = C.c_int
    lib.fuseml_sm100_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.fuseml_sm100_schedule.restype = C.c_int32
    lib.fuseml_sm100_schedule.argtypes = [C.POINTER(GemmDesc), C.POINTER(Plan), C.c_int32, C.POINTER(WorkItem),
                                          C.c_int32, C.POINTER(C.c_int32)]


def load(path: os.PathLike | str | None = None) -> C.CDLL:
    """Load (once) and return the library.  Raises :class:`NativeLibraryError` if absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    with _lock:
        if _lib is not None and path is None:
            return _lib
        # FUSEML_SM100_LIB points at an alternative build of the same ABI (A/B measurements)
        override = os.environ.get("FUSEML_SM100_LIB")
        p = Path(path) if path is not None else (Path(override) if override else LIB_PATH)
        if not p.exists():
            raise NativeLibraryError(
                f"{p} is missing: build it with `python -m fuseml_b200.build` "
                "(nvcc, sm_100a). There is no fallback path for fused kernels."
            )
        try:
            lib = C.CDLL(str(p))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise NativeLibraryError(f"cannot load {p}: {exc}") from exc
        missing = [s for s in EXPORTS if not hasattr(lib, s)]
        if missing:
            raise NativeLibraryError(f"{p} lacks symbols {missing}")
        _declare(lib)
        if lib.fuseml_sm100_abi_version() != ABI_VERSION:
            raise NativeLibraryError("ABI version mismatch between the Python binding and the library")
        if path is None:
            _lib = lib
        return lib


def strerror(code: int) -> str:
    return load().fuseml_sm100_strerror(int(code)).decode()


def check(code: int, what: str = "fuseml_sm100") -> None:
    """Raise ``RuntimeError`` for a non-zero status code."""
    if code != OK:
        raise NativeLibraryError(f"{what} failed with status {code}: {strerror(code)}")
