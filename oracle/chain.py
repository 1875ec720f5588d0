"""numpy restatement of one fused ``addmm|mm -> pointwise... [-> reduction]`` chain.

TEST INFRASTRUCTURE: the checker the CUDA path is compared against.

Arithmetic contract of the reference kernel that this follows
(paths inside the FuseML tree):

* accumulator is fp32, operands keep their storage dtype
  (fuseml/codegen/kernel_generator.py:1470, 1536);
* the addmm bias is upcast and added to the accumulator before any other op
  (fuseml/codegen/kernel_generator.py:885-901);
* every epilogue op is evaluated in fp32 (``:1599-1903``), with one cast to the
  output dtype at the store and an fp16 clamp to +-65504 (``:1575-1592``);
* reductions act on the fp32 epilogue result; mean multiplies the sum by 1/len
  (``:1959-1960, 1983-1984, 2015-2017``).

bf16 / fp16 tensors are represented as float32 arrays whose values are exactly
representable in the narrow type (see :func:`round_bf16`).
"""
from __future__ import annotations

import math
from typing import Iterable, Sequence

import numpy as np

try:  # scipy is present in the image; keep a pure-numpy erf for safety
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf, otypes=[np.float64])


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32).reshape(x.shape)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.float32(np.nan), out)
    return out


def round_f16(x: np.ndarray) -> np.ndarray:
    """Saturate to +-65504 then round to fp16 (fuseml/codegen/kernel_generator.py:1575-1581)."""
    x = np.clip(np.asarray(x, dtype=np.float32), -65504.0, 65504.0)
    return x.astype(np.float16).astype(np.float32)


def cast_out(x: np.ndarray, dtype: str) -> np.ndarray:
    """The single cast at the store (fuseml/codegen/kernel_generator.py:1583-1592)."""
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f16":
        return round_f16(x)
    return np.asarray(x, dtype=np.float32)


def gemm_acc32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``acc[M,N] = sum_k A[m,k] * B[k,n]`` with fp32 products and accumulation
    (fuseml/codegen/kernel_generator.py:1470, 1519-1541)."""
    return np.matmul(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32))


# ---- epilogue operations, fp32 in / fp32 out -----------------------------------

def relu(x):
    """``where(acc > 0, acc, 0)`` (fuseml/codegen/kernel_generator.py:1604)."""
    return np.where(x > 0, x, np.float32(0)).astype(np.float32)


def gelu_erf(x):
    """``0.5 * x * (1 + erf(x * 0.7071067811865476))`` (fuseml/codegen/kernel_generator.py:1641)."""
    x64 = x.astype(np.float64)
    return (0.5 * x64 * (1.0 + _erf(x64 * 0.7071067811865476))).astype(np.float32)


def gelu_tanh(x):
    """tanh-approximate GELU, ``aten.gelu(approximate='tanh')``."""
    x64 = x.astype(np.float64)
    u = 0.7978845608028654 * (x64 + 0.044715 * x64 ** 3)
    return (0.5 * x64 * (1.0 + np.tanh(u))).astype(np.float32)


def sigmoid(x):
    """``1 / (1 + exp(-x))`` (fuseml/codegen/kernel_generator.py:1655)."""
    x64 = x.astype(np.float64)
    return (1.0 / (1.0 + np.exp(-x64))).astype(np.float32)


def gelu_erf_grad(x):
    """d/dx of the erf-form GELU: ``Phi(x) + x * phi(x)`` (what ``aten.gelu_backward`` multiplies the
    incoming gradient by; the reference leaves backward graphs to PyTorch, fuseml/compiler.py:214-218)."""
    x64 = x.astype(np.float64)
    return (0.5 * (1.0 + _erf(x64 * 0.7071067811865476)) + x64 * np.exp(-0.5 * x64 * x64) / np.sqrt(2.0 * np.pi)).astype(np.float32)


def _bcast(t: np.ndarray, M: int, N: int) -> np.ndarray:
    """Broadcast rule for external operands: a 1-D tensor of length N runs along
    columns, of length M along rows (fuseml/codegen/kernel_generator.py:270-277);
    2-D tensors broadcast over size-1 / stride-0 dims (``:1708-1743``)."""
    t = np.asarray(t, dtype=np.float32)
    if t.ndim == 0:
        return np.broadcast_to(t, (M, N))
    if t.ndim == 1:
        if t.shape[0] == N or t.shape[0] == 1:
            return np.broadcast_to(t[None, :], (M, N))
        if t.shape[0] == M:
            return np.broadcast_to(t[:, None], (M, N))
        raise ValueError(f"1-D operand of length {t.shape[0]} does not broadcast to ({M},{N})")
    return np.broadcast_to(t, (M, N))


def run_epilogue(acc: np.ndarray, ops: Sequence[tuple], aux_dtype: str = "bf16"):
    """Apply ``ops`` in order.  Each op is a tuple:

    ``("relu",)``, ``("gelu",)``, ``("gelu_tanh",)``, ``("sigmoid",)``, ``("gelu_times_sigmoid",)``,
    ``("add_scalar", c)``, ``("mul_scalar", c)``,
    ``("add", t)``, ``("mul", t)``, ``("sub", t)``, ``("rsub", t)``, ``("gelu_bwd", t)`` with an external array,
    ``("save",)``, ``("swap",)``, ``("add_saved",)``, ``("mul_saved",)``,
    ``("store_aux",)`` (returns the value at that point, cast to ``aux_dtype``).

    Returns ``(value, aux_list)``.
    """
    M, N = acc.shape
    v = acc.astype(np.float32)
    saved = np.zeros_like(v)
    aux = []
    for op in ops:
        k = op[0]
        if k == "relu":
            v = relu(v)
        elif k == "gelu":
            v = gelu_erf(v)
        elif k == "gelu_tanh":
            v = gelu_tanh(v)
        elif k == "sigmoid":
            v = sigmoid(v)
        elif k == "gelu_times_sigmoid":
            v = (gelu_erf(v).astype(np.float64) * sigmoid(v).astype(np.float64)).astype(np.float32)
        elif k == "add_scalar":
            v = (v + np.float32(op[1])).astype(np.float32)
        elif k == "mul_scalar":
            v = (v * np.float32(op[1])).astype(np.float32)
        elif k in ("add", "bias"):
            v = (v + _bcast(op[1], M, N)).astype(np.float32)
        elif k == "mul":
            v = (v * _bcast(op[1], M, N)).astype(np.float32)
        elif k == "sub":
            v = (v - _bcast(op[1], M, N)).astype(np.float32)
        elif k == "gelu_bwd":
            v = (v.astype(np.float64) * gelu_erf_grad(_bcast(op[1], M, N)).astype(np.float64)).astype(np.float32)
        elif k == "rsub":
            v = (_bcast(op[1], M, N) - v).astype(np.float32)
        elif k == "save":
            saved = v.copy()
        elif k == "swap":
            v, saved = saved, v
        elif k == "add_saved":
            v = (v + saved).astype(np.float32)
        elif k == "mul_saved":
            v = (v * saved).astype(np.float32)
        elif k == "store_aux":
            aux.append(cast_out(v, aux_dtype))
        else:
            raise ValueError(f"unknown epilogue op {k!r}")
    return v, aux


def reduce_tail(v: np.ndarray, kinds: Iterable[str], axis) -> dict:
    """sum / max / mean of the fp32 epilogue result over ``axis`` (-1: per row, 0: per
    column, None: everything), accumulated in float64 and returned as float32
    (fuseml/codegen/kernel_generator.py:1909-2018; outputs are 1-D, keepdim=False,
    fuseml/passes/fusion_pass.py:223-241)."""
    out = {}
    v64 = v.astype(np.float64)
    for k in kinds:
        if k == "sum":
            out[k] = np.asarray(v64.sum(axis=axis), dtype=np.float32)
        elif k in ("max", "amax"):
            out["max"] = np.asarray(v.max(axis=axis), dtype=np.float32)
        elif k == "mean":
            out[k] = np.asarray(v64.mean(axis=axis), dtype=np.float32)
        else:
            raise ValueError(f"unknown reduction {k!r}")
    return out


def fused_chain(a, b, ops=(), out_dtype="bf16", reduce=(), axis=None, store=True):
    """One fused kernel: GEMM -> epilogue -> (store, reductions)."""
    acc = gemm_acc32(a, b)
    v, aux = run_epilogue(acc, ops, aux_dtype=out_dtype)
    res = {"d": cast_out(v, out_dtype) if store else None, "aux": aux}
    if reduce:
        res.update(reduce_tail(v, reduce, axis))
    return res
