"""Python face of the C ABI: epilogue programs and one-call fused GEMM launches.

``fused_gemm`` is what :class:`fuseml_b200.codegen.kernel_launcher.KernelLauncher`
calls on the hot path.  It takes CUDA tensors, fills a ``fuseml_gemm_desc_t``
with their pointers and strides and enqueues the sm_100a kernel on torch's
current stream.  Nothing here computes on the host and nothing falls back to
PyTorch ops: a tensor the kernel cannot address raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Iterable, Sequence

import torch

from . import _native as N

_DTYPE_CODE = {torch.bfloat16: N.BF16, torch.float16: N.F16, torch.float32: N.F32}
_RED_BITS = {"sum": N.RED_SUM, "max": N.RED_MAX, "amax": N.RED_MAX, "mean": N.RED_MEAN}
_AXIS = {"n": N.AXIS_N, "m": N.AXIS_M, "all": N.AXIS_ALL, 1: N.AXIS_N, -1: N.AXIS_N, 0: N.AXIS_M, -2: N.AXIS_M,
         None: N.AXIS_ALL}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise N.NativeLibraryError(f"dtype {dtype} is not supported by the sm_100a kernels") from None


@dataclass
class EpilogueProgram:
    """Ordered list of epilogue operations applied to the fp32 accumulator.

    The reference builds the same sequence as Triton source lines
    (fuseml/codegen/kernel_generator.py:912-1065); here it is data handed to a
    precompiled kernel.  ``operands`` holds the external tensors the program
    reads (bias, residual, ...), in slot order.
    """

    ops: list[tuple[int, int, float]] = field(default_factory=list)   # (opcode, slot, imm)
    operands: list[torch.Tensor] = field(default_factory=list)

    # --- unary ---------------------------------------------------------------
    def relu(self) -> "EpilogueProgram":
        return self._push(N.OP_RELU)

    def gelu(self, approximate: str = "none") -> "EpilogueProgram":
        return self._push(N.OP_GELU_TANH if approximate == "tanh" else N.OP_GELU_ERF)

    def sigmoid(self) -> "EpilogueProgram":
        return self._push(N.OP_SIGMOID)

    def gelu_times_sigmoid(self) -> "EpilogueProgram":
        """``acc = gelu(acc) * sigmoid(acc)`` as one step (what the launch rewrites the diamond
        ``save, gelu, swap, sigmoid, mul_saved`` to)."""
        return self._push(N.OP_GELU_ERF_MUL_SIGMOID)

    # --- binary with a python scalar ------------------------------------------
    def add_scalar(self, c: float) -> "EpilogueProgram":
        return self._push(N.OP_ADD_IMM, imm=float(c))

    def mul_scalar(self, c: float) -> "EpilogueProgram":
        return self._push(N.OP_MUL_IMM, imm=float(c))

    # --- binary with an external tensor (broadcastable to [M, N]) ---------------
    def add_tensor(self, t: torch.Tensor) -> "EpilogueProgram":
        return self._push(N.OP_ADD_T, slot=self._slot(t))

    def mul_tensor(self, t: torch.Tensor) -> "EpilogueProgram":
        return self._push(N.OP_MUL_T, slot=self._slot(t))

    def sub_tensor(self, t: torch.Tensor) -> "EpilogueProgram":
        return self._push(N.OP_SUB_T, slot=self._slot(t))

    def rsub_tensor(self, t: torch.Tensor) -> "EpilogueProgram":
        return self._push(N.OP_RSUB_T, slot=self._slot(t))

    def gelu_backward(self, pre: torch.Tensor) -> "EpilogueProgram":
        """``acc *= gelu'(pre)``: ``aten.gelu_backward(grad=acc, self=pre)``, erf form."""
        return self._push(N.OP_GELU_ERF_BWD_T, slot=self._slot(pre))

    def bias(self, b: torch.Tensor) -> "EpilogueProgram":
        """``acc += bias`` — the addmm bias (fuseml/codegen/kernel_generator.py:885-901)."""
        return self.add_tensor(b)

    def store_aux(self, t: torch.Tensor) -> "EpilogueProgram":
        """Write the current value to ``t[M,N]`` (escape store of an intermediate)."""
        return self._push(N.OP_STORE_AUX, slot=self._slot(t))

    # --- second value register (single-entry DAGs) -----------------------------
    def save(self) -> "EpilogueProgram":
        return self._push(N.OP_SAVE)

    def swap(self) -> "EpilogueProgram":
        return self._push(N.OP_SWAP)

    def add_saved(self) -> "EpilogueProgram":
        return self._push(N.OP_ADD_SAVED)

    def mul_saved(self) -> "EpilogueProgram":
        return self._push(N.OP_MUL_SAVED)

    # ---------------------------------------------------------------------------
    def _slot(self, t: torch.Tensor) -> int:
        for i, o in enumerate(self.operands):
            if o is t:
                return i
        if len(self.operands) >= N.MAX_OPERANDS:
            raise N.NativeLibraryError(f"epilogue uses more than {N.MAX_OPERANDS} external tensors")
        self.operands.append(t)
        return len(self.operands) - 1

    def _push(self, opcode: int, slot: int = 0, imm: float = 0.0) -> "EpilogueProgram":
        if len(self.ops) >= N.MAX_EPI_OPS:
            raise N.NativeLibraryError(f"epilogue longer than {N.MAX_EPI_OPS} operations")
        self.ops.append((opcode, slot, imm))
        return self

    def signature(self) -> tuple:
        """Hashable identity of the op sequence (without tensor addresses)."""
        return tuple((N.OP_NAMES[o], s, round(i, 9)) for o, s, i in self.ops)

    def with_operands(self, tensors: Sequence[torch.Tensor]) -> "EpilogueProgram":
        """Same ops, other tensors in the slots (used per call by the launcher)."""
        if len(tensors) != len(self.operands):
            raise ValueError(f"program has {len(self.operands)} operand slots, got {len(tensors)}")
        return EpilogueProgram(ops=self.ops, operands=list(tensors))


def _broadcast_strides(t: torch.Tensor, M: int, Ncols: int) -> tuple[int, int]:
    """Element strides of ``t`` viewed as ``[M, N]`` (0 where it broadcasts)."""
    if t.dim() == 0:
        return 0, 0
    if t.dim() == 1:
        # reference rule: a 1-D tensor of length N runs along N, of length M along M, else N
        # (fuseml/codegen/kernel_generator.py:270-277)
        n = t.shape[0]
        if n == Ncols or n == 1:
            return 0, (t.stride(0) if n != 1 else 0)
        if n == M:
            return t.stride(0), 0
        raise N.NativeLibraryError(f"1-D operand of length {n} does not broadcast to [{M}, {Ncols}]")
    if t.dim() == 2:
        rows, cols = t.shape
        if rows not in (1, M) or cols not in (1, Ncols):
            raise N.NativeLibraryError(f"operand of shape {tuple(t.shape)} does not broadcast to [{M}, {Ncols}]")
        sm = 0 if rows == 1 and M != 1 else t.stride(0)
        sn = 0 if cols == 1 and Ncols != 1 else t.stride(1)
        return sm, sn
    raise N.NativeLibraryError("epilogue operands must have at most 2 dimensions")


def addressable_left(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a`` itself when the kernel can read it in place, else a row-major copy.  K contiguous is
    the usual case.  A transposed view (stored ``[K, M]``: the ``dY^T`` of a weight gradient) is
    read in place when B is row-major ``[K, N]`` too and the pitch is a multiple of 16 bytes;
    fp32 operands are expanded by plain loads and take any strides."""
    M, K = a.shape
    if K == 1 or a.stride(1) == 1:
        return a
    if a.dtype == torch.float32:
        return a if min(a.stride()) >= 0 else a.contiguous()
    if (a.stride(0) == 1 or M == 1) and a.stride(1) >= M and (a.stride(1) * a.element_size()) % 16 == 0 \
            and a.data_ptr() % 16 == 0 and b.stride(1) == 1:
        return a
    return a.contiguous()


def fill_desc(desc: N.GemmDesc, a: torch.Tensor, b: torch.Tensor, program: EpilogueProgram | None,
              out: torch.Tensor | None, out_dtype: torch.dtype) -> tuple[int, int, int]:
    """Write the GEMM part of a descriptor; returns (M, N, K)."""
    if a.dim() != 2 or b.dim() != 2:
        raise N.NativeLibraryError("fused_gemm expects 2-D A[M,K] and B[K,N]")
    if not a.is_cuda or not b.is_cuda:
        raise N.NativeLibraryError("fused kernels run on CUDA tensors only (there is no CPU path)")
    M, K = a.shape
    K2, Ncols = b.shape
    if K != K2:
        raise N.NativeLibraryError(f"contracting dimension mismatch: A{tuple(a.shape)} B{tuple(b.shape)}")
    if a.dtype != b.dtype:
        raise N.NativeLibraryError(f"A and B dtypes differ: {a.dtype} vs {b.dtype}")
    a = addressable_left(a, b)
    desc.M, desc.N, desc.K = M, Ncols, K
    desc.a = a.data_ptr()
    desc.lda = a.stride(0)
    desc.a_stride_k = a.stride(1) if K != 1 else 1
    desc.b = b.data_ptr()
    desc.b_stride_k = b.stride(0)
    desc.b_stride_n = b.stride(1)
    desc.ab_dtype = dtype_code(a.dtype)
    desc.out_dtype = dtype_code(out_dtype)
    if out is not None:
        if out.stride(1) != 1 and Ncols != 1:
            raise N.NativeLibraryError("output must be row-major")
        desc.d = out.data_ptr()
        desc.ldd = out.stride(0)
    else:
        desc.d = None
        desc.ldd = 0
    n_ops = 0
    n_operands = 0
    if program is not None:
        for i, (opcode, slot, imm) in enumerate(program.ops):
            desc.ops[i].opcode = opcode
            desc.ops[i].slot = slot
            desc.ops[i].imm = imm
        n_ops = len(program.ops)
        for i, t in enumerate(program.operands):
            if not t.is_cuda:
                raise N.NativeLibraryError("epilogue operands must be CUDA tensors")
            sm, sn = _broadcast_strides(t, M, Ncols)
            desc.operands[i].ptr = t.data_ptr()
            desc.operands[i].stride_m = sm
            desc.operands[i].stride_n = sn
            desc.operands[i].dtype = dtype_code(t.dtype)
        n_operands = len(program.operands)
    desc.n_ops = n_ops
    desc.n_operands = n_operands
    desc._keepalive = (a, b)  # a.contiguous() copy must outlive the enqueue
    return M, Ncols, K


def plan_for(desc: N.GemmDesc, props: N.DeviceProps | None = None) -> N.Plan:
    """Ask the roofline router for tile / stage / grid shape (host only)."""
    plan = N.Plan()
    lib = N.load()
    rc = lib.fuseml_sm100_plan(C.byref(desc), C.byref(props) if props is not None else None, C.byref(plan))
    N.check(rc, "fuseml_sm100_plan")
    return plan


_props_cache: dict[int, N.DeviceProps] = {}


def device_props(device: torch.device | int | None = None) -> N.DeviceProps:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    p = _props_cache.get(idx)
    if p is None:
        p = N.DeviceProps()
        with torch.cuda.device(idx):
            rc = N.load().fuseml_sm100_query(C.byref(p))
        N.check(rc, "fuseml_sm100_query")
        _props_cache[idx] = p
    return p


def fused_gemm(a: torch.Tensor, b: torch.Tensor, program: EpilogueProgram | None = None, *,
               out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None, store: bool = True,
               reduce: Iterable[str] = (), axis=None, plan: N.Plan | None = None):
    """``epilogue(A @ B)`` in one sm_100a kernel.

    Returns ``out`` when no reduction is requested, else ``(out_or_None, {kind: fp32 tensor})``.
    ``reduce`` is any subset of ``{"sum", "max", "mean"}``; ``axis`` is ``-1``/``1``
    (per row), ``0`` (per column) or ``None`` (global).
    """
    lib = N.load()
    out_dtype = out_dtype or a.dtype
    M, K = a.shape
    Ncols = b.shape[1]
    kinds = 0
    for r in reduce:
        kinds |= _RED_BITS[r]
    if store and out is None:
        out = torch.empty_strided((M, Ncols), (Ncols, 1), dtype=out_dtype, device=a.device)
    desc = N.GemmDesc()
    fill_desc(desc, a, b, program, out if store else None, out_dtype)
    results: dict[str, torch.Tensor] = {}
    keep = []
    if kinds:
        ax = _AXIS[axis]
        length = M if ax == N.AXIS_N else (Ncols if ax == N.AXIS_M else 1)
        desc.reduce.kinds = kinds
        desc.reduce.axis = ax
        for bit, name, fld in ((N.RED_SUM, "sum", "out_sum"), (N.RED_MAX, "max", "out_max"),
                               (N.RED_MEAN, "mean", "out_mean")):
            if kinds & bit:
                t = torch.empty((length,) if ax != N.AXIS_ALL else (), dtype=torch.float32, device=a.device)
                results[name] = t
                setattr(desc.reduce, fld, t.data_ptr())
    if plan is None:
        plan = plan_for(desc, device_props(a.device))
    ws_bytes = lib.fuseml_sm100_workspace_bytes(C.byref(desc), C.byref(plan))
    if ws_bytes < 0:
        raise N.NativeLibraryError("fuseml_sm100_workspace_bytes rejected the descriptor")
    if ws_bytes > 0:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        keep.append(ws)
        desc.reduce.workspace = ws.data_ptr()
        desc.reduce.workspace_bytes = ws_bytes
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        rc = lib.fuseml_sm100_gemm_epilogue(C.byref(desc), C.byref(plan), C.c_void_p(stream))
    N.check(rc, "fuseml_sm100_gemm_epilogue")
    if kinds:
        return (out if store else None), results
    return out


_last_mlp_workspace: list = [None]


def last_mlp_workspace() -> torch.Tensor | None:
    """The workspace the most recent :func:`fused_mlp` call used (callers that launch the same block
    again pass it back in instead of allocating a new one)."""
    return _last_mlp_workspace[0]


def fused_mlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, prog1: EpilogueProgram | None = None,
              prog2: EpilogueProgram | None = None, *, out_dtype: torch.dtype | None = None,
              out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
              weights_expanded: bool = False) -> torch.Tensor:
    """``prog2(prog1(x @ w1.T) @ w2.T)`` for at most 128 rows in one kernel (plus the pass that folds
    the CTAs' partial outputs): the intermediate never reaches global memory.  ``w1[I, D_in]`` and
    ``w2[D_out, I]`` are the ``nn.Linear`` weights as stored.  ``prog1`` sees ``h[M, I]``, ``prog2``
    sees ``y[M, D_out]``.  Raises :class:`NativeLibraryError` when the block is not eligible
    (``fuseml_sm100_mlp_small_workspace_bytes`` returns -1); callers then launch the two Linears
    separately."""
    lib = N.load()
    if x.dim() != 2 or w1.dim() != 2 or w2.dim() != 2 or not (x.is_cuda and w1.is_cuda and w2.is_cuda):
        raise N.NativeLibraryError("fused_mlp expects 2-D CUDA tensors x[M, D_in], w1[I, D_in], w2[D_out, I]")
    if not (x.dtype == w1.dtype == w2.dtype):
        raise N.NativeLibraryError("x, w1 and w2 must share one dtype")
    M, D_in = x.shape
    I, D_in2 = w1.shape
    D_out, I2 = w2.shape
    if D_in != D_in2 or I != I2:
        raise N.NativeLibraryError(f"shape mismatch: x{tuple(x.shape)} w1{tuple(w1.shape)} w2{tuple(w2.shape)}")
    for t in (x, w1, w2):
        if t.stride(1) != 1:
            raise N.NativeLibraryError("x, w1 and w2 must be row-major (unit stride along their last dimension)")
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty_strided((M, D_out), (D_out, 1), dtype=out_dtype, device=x.device)
    d = N.MlpDesc()
    d.M, d.D_in, d.I, d.D_out = M, D_in, I, D_out
    d.x, d.ldx = x.data_ptr(), x.stride(0)
    d.w1, d.ldw1 = w1.data_ptr(), w1.stride(0)
    d.w2, d.ldw2 = w2.data_ptr(), w2.stride(0)
    d.ab_dtype, d.out_dtype = dtype_code(x.dtype), dtype_code(out_dtype)
    d.y, d.ldy = out.data_ptr(), out.stride(0)
    d.flags = N.MLP_WEIGHTS_EXPANDED if weights_expanded else 0
    slot = 0
    for prog, ops, cols, which in ((prog1, d.ops1, I, "n_ops1"), (prog2, d.ops2, D_out, "n_ops2")):
        n = 0
        if prog is not None:
            base = slot
            for t in prog.operands:
                if slot >= N.MAX_OPERANDS:
                    raise N.NativeLibraryError(f"the two programs use more than {N.MAX_OPERANDS} external tensors")
                sm, sn = _broadcast_strides(t, M, cols)
                o = d.operands[slot]
                o.ptr, o.stride_m, o.stride_n, o.dtype = t.data_ptr(), sm, sn, dtype_code(t.dtype)
                slot += 1
            for i, (opcode, s, imm) in enumerate(prog.ops):
                ops[i].opcode, ops[i].slot, ops[i].imm = opcode, base + s, imm
            n = len(prog.ops)
        setattr(d, which, n)
    d.n_operands = slot
    need = lib.fuseml_sm100_mlp_small_workspace_bytes(C.byref(d))
    if need < 0:
        raise N.NativeLibraryError("this MLP block cannot run as one kernel (more than 128 rows, an output wider than "
                                   "512 columns, an intermediate width that does not divide into slices, unaligned "
                                   "rows, or a first program that needs the second value register)")
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(int(need), 16), dtype=torch.uint8, device=x.device)
    _last_mlp_workspace[0] = workspace
    d.workspace, d.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = lib.fuseml_sm100_mlp_small(C.byref(d), C.c_void_p(stream))
    N.check(rc, "fuseml_sm100_mlp_small")
    return out


def reduce_tail(x: torch.Tensor, reduce: Iterable[str], axis=None) -> dict[str, torch.Tensor]:
    """Stand-alone sum / max / mean over a 2-D CUDA tensor (fp32 results)."""
    lib = N.load()
    if x.dim() != 2 or not x.is_cuda:
        raise N.NativeLibraryError("reduce_tail expects a 2-D CUDA tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    M, Ncols = x.shape
    kinds = 0
    for r in reduce:
        kinds |= _RED_BITS[r]
    ax = _AXIS[axis]
    length = M if ax == N.AXIS_N else (Ncols if ax == N.AXIS_M else 1)
    red = N.Reduce()
    red.kinds, red.axis = kinds, ax
    results: dict[str, torch.Tensor] = {}
    for bit, name, fld in ((N.RED_SUM, "sum", "out_sum"), (N.RED_MAX, "max", "out_max"),
                           (N.RED_MEAN, "mean", "out_mean")):
        if kinds & bit:
            t = torch.empty((length,) if ax != N.AXIS_ALL else (), dtype=torch.float32, device=x.device)
            results[name] = t
            setattr(red, fld, t.data_ptr())
    ws = None
    if ax != N.AXIS_N:
        ws_bytes = 2 * (max(M, 1184) * max(length, 1) * 4 + 256)
        if ax == N.AXIS_M:
            ws_bytes = 2 * (64 * Ncols * 4 + 256)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
        red.workspace = ws.data_ptr()
        red.workspace_bytes = ws_bytes
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = lib.fuseml_sm100_reduce_tail(C.c_void_p(x.data_ptr()), dtype_code(x.dtype), M, Ncols, x.stride(0),
                                          C.byref(red), C.c_void_p(stream))
    N.check(rc, "fuseml_sm100_reduce_tail")
    return results


def device_status() -> int:
    """Synchronise the current stream and return (then clear) the device status word."""
    out = C.c_int32(0)
    stream = torch.cuda.current_stream().cuda_stream
    N.load().fuseml_sm100_device_status(C.c_void_p(stream), C.byref(out))
    return int(out.value)


def set_diagnostics(wait_limit_us: int = 0, drop_last_load: bool = False) -> None:
    """Shorten the device-side wait limit and / or inject a lost operand load into the launches
    that follow (``fuseml_sm100_set_diagnostics``); ``set_diagnostics()`` restores normal operation."""
    N.check(N.load().fuseml_sm100_set_diagnostics(int(wait_limit_us), 1 if drop_last_load else 0),
            "fuseml_sm100_set_diagnostics")
