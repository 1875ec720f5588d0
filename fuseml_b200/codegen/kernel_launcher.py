"""Runtime dispatch of one fused chain: live tensors in, C-ABI launch on the current stream.

Counterpart of the reference's ``KernelLauncher`` (fuseml/codegen/kernel_launcher.py:309-847).
The call contract is unchanged — ``launcher(*input_tensors)`` with tensors in
``FusionGroup.inputs`` order, ``__name__ == "fuseml_fused_kernel"`` for FX node naming,
``ValueError`` on arity / unknown operand names, outputs allocated through torch per call,
no host synchronisation — but there is no Triton kernel object any more: ``kernel_fn`` is a
:class:`~fuseml_b200.codegen.kernel_generator.KernelSpec`, and the launch is
``fuseml_sm100_gemm_epilogue`` through ``ctypes``.

Per distinct (shape, stride) signature of the inputs the launcher keeps one prepared
descriptor, the plan the roofline router returned for it and a workspace per stream; a
call then only writes pointers into the descriptor.  Groups with several outputs
(escape stores, extra reductions) return a tuple ``(primary, *escapes, *reductions)``,
which is what graph surgery's ``getitem`` nodes index.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch

from .. import _native as N
from .. import kernels as K
from .._logging import logger
from ..passes.topology import classify_epilogue_operand
from .kernel_generator import KernelSpec, TensorDescriptor

_DEFAULT_BLOCK_SIZE_M = 128
_DEFAULT_BLOCK_SIZE_N = 256
_DEFAULT_BLOCK_SIZE_K = 64
_DEFAULT_GROUP_SIZE_M = 8

_RED_BIT = {"sum": N.RED_SUM, "max": N.RED_MAX, "mean": N.RED_MEAN}
_RED_FIELD = {"sum": "out_sum", "max": "out_max", "mean": "out_mean"}
_AXIS_CODE = {0: N.AXIS_M, 1: N.AXIS_N, 2: N.AXIS_ALL}


@dataclass(frozen=True)
class LaunchParams:
    """Frozen launch configuration: the tile the CTA computes, the K extent of one
    shared-memory stage, the rasterisation group, epilogue warps and ring depth.
    (The reference froze Triton ``BLOCK_SIZE_*`` / ``num_warps`` / ``num_stages`` here,
    fuseml/codegen/kernel_launcher.py:99-127.)"""
    block_m: int
    block_n: int
    block_k: int
    group_size_m: int
    num_warps: int
    num_stages: int


def _prod(shape) -> int:
    n = 1
    for v in shape:
        n *= int(v)
    return n


def compute_launch_params(M: int, Ncols: int, Kd: int, dtype: torch.dtype = torch.bfloat16, *,
                          block_size_m: int = _DEFAULT_BLOCK_SIZE_M, block_size_n: int = _DEFAULT_BLOCK_SIZE_N,
                          block_size_k: int = _DEFAULT_BLOCK_SIZE_K, group_size_m: int = _DEFAULT_GROUP_SIZE_M,
                          sram_autotuner: Any = None) -> LaunchParams:
    """Ask the native router (host only, no GPU needed) for the tile shape of an M x N x K problem."""
    desc = N.GemmDesc()
    desc.M, desc.N, desc.K = int(M), int(Ncols), int(Kd)
    desc.a, desc.b, desc.d = 0x1000, 0x2000, 0x3000          # layout-only query: aligned dummies
    desc.lda, desc.b_stride_k, desc.b_stride_n, desc.ldd = int(Kd), 1, int(Kd), int(Ncols)
    code = K.dtype_code(dtype)
    desc.ab_dtype = desc.out_dtype = code
    if code != N.F32 and (Kd * 2) % 16 != 0:
        desc.lda = desc.b_stride_n = (int(Kd) + 7) // 8 * 8
    plan = N.Plan()
    rc = N.load().fuseml_sm100_plan(C.byref(desc), None, C.byref(plan))
    if rc != N.OK:
        return LaunchParams(block_size_m, block_size_n, block_size_k, group_size_m, 6, 4)
    return LaunchParams(plan.tile_m, plan.tile_n, plan.tile_k, plan.group_m, 6, plan.stages)


_BUILD_ID: list = []


def _build_id() -> str:
    """Short digest of the sources the loaded library was built from (part of every plan-cache key)."""
    if not _BUILD_ID:
        from ..build import source_digest

        try:
            _BUILD_ID.append(source_digest()[:12])
        except OSError:
            _BUILD_ID.append("unknown")
    return _BUILD_ID[0]


class _Prepared:
    """One (shape, stride) signature: filled descriptor, plan, workspace size, output shapes."""
    __slots__ = ("desc", "plan", "ws_bytes", "ws", "b_tag", "tune_key", "M", "N", "K", "red_len", "left", "right",
                 "views", "out_shape", "aux_shapes", "red_shape")


class KernelLauncher:
    _POST_KERNEL_NOOP = 0
    _POST_KERNEL_CAST_ONLY = 1

    def __init__(self, kernel_fn: KernelSpec, input_descriptors: Sequence[TensorDescriptor],
                 output_descriptor: TensorDescriptor, intermediate_descriptors: Sequence[TensorDescriptor],
                 left_name: str, right_name: str, launch_params: LaunchParams | None = None,
                 block_size_m: int = _DEFAULT_BLOCK_SIZE_M, block_size_n: int = _DEFAULT_BLOCK_SIZE_N,
                 block_size_k: int = _DEFAULT_BLOCK_SIZE_K, group_size_m: int = _DEFAULT_GROUP_SIZE_M,
                 reduction_op: str | None = None, reduction_axis: int | None = None,
                 eager_fn: Callable | None = None, is_autotuned: bool = False, sram_autotuner: Any = None,
                 mean_epilogue_fused: bool = True, reduction_dtypes: Sequence[torch.dtype] | None = None,
                 reduction_shape: Sequence[int] | None = None, plan_cache: Any = None, autotune: bool = False) -> None:
        self.__name__ = "fuseml_fused_kernel"
        if not isinstance(kernel_fn, KernelSpec):
            raise TypeError("kernel_fn must be a KernelSpec (the lowered form of a FusionGroup)")
        self._spec = kernel_fn
        self._kernel_fn = kernel_fn
        self._input_descriptors = list(input_descriptors)
        self._output_descriptor = output_descriptor
        self._intermediate_descriptors = list(intermediate_descriptors)
        names = [d.name for d in self._input_descriptors]
        for label, name in (("left_name", left_name), ("right_name", right_name)):
            if name not in names:
                raise ValueError(f"{label}={name!r} not found in input_descriptors: {names}")
        self._left_idx = names.index(left_name)
        self._right_idx = names.index(right_name)
        if (self._left_idx, self._right_idx) != (kernel_fn.left_index, kernel_fn.right_index):
            raise ValueError("left/right operand names disagree with the kernel specification")
        # reductions: from the spec; the reduction_op / reduction_axis keywords describe the
        # classic single-reduction case and are checked against it
        self._reductions = list(kernel_fn.reductions)
        if reduction_op is not None and not self._reductions:
            raise ValueError(f"reduction_op={reduction_op!r} given but the kernel has no reduction")
        self._reduction_op = reduction_op or (self._reductions[0].op if self._reductions else None)
        self._reduction_axis = reduction_axis if reduction_axis is not None else (
            self._reductions[0].axis if self._reductions else 1)
        self._is_reduced = bool(self._reductions) and not kernel_fn.store_output and not intermediate_descriptors
        self._reduction_dtypes = list(reduction_dtypes) if reduction_dtypes is not None else \
            [output_descriptor.dtype] * len(self._reductions)
        # shape the graph expects of a per-row reduction when the rows are grouped ([B, S])
        self._row_reduction_shape = tuple(int(v) for v in reduction_shape) \
            if reduction_shape is not None and len(reduction_shape) != 1 else None
        self._launch_params = launch_params
        self._is_autotuned = is_autotuned
        self._sram_autotuner = sram_autotuner
        self._skip_stride_check = all(all(s >= 0 for s in d.stride) for d in self._input_descriptors)
        self._prepared: dict[tuple, _Prepared] = {}
        # measured plans (codegen/plan_cache.py): looked up per signature, filled by timing a few
        # candidate plans on the first call when `autotune` is set
        self._plan_cache = plan_cache
        self._autotune = bool(autotune)
        self.tuned_signatures = 0
        self._lib = None
        self.launch_count = 0
        # operand slots of the program: input indices in order of first use
        self._slot_inputs: list[int] = []
        self._aux_slots: dict[int, int] = {}
        for st in kernel_fn.steps:
            if st.opcode == N.OP_STORE_AUX:
                continue
            if st.input_index >= 0 and st.input_index not in self._slot_inputs:
                self._slot_inputs.append(st.input_index)
        n_in = len(self._slot_inputs)
        for st in kernel_fn.steps:
            if st.opcode == N.OP_STORE_AUX and st.aux_index not in self._aux_slots:
                self._aux_slots[st.aux_index] = n_in + len(self._aux_slots)
        if n_in + len(self._aux_slots) > N.MAX_OPERANDS:
            raise ValueError(f"chain needs more than {N.MAX_OPERANDS} operand slots")

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _has_negative_strides(t: torch.Tensor) -> bool:
        return any(s < 0 for s in t.stride())

    @staticmethod
    def _materialize_if_needed(t: torch.Tensor) -> torch.Tensor:
        return t.contiguous() if any(s < 0 for s in t.stride()) else t

    def _operand_views(self, inputs: Sequence[torch.Tensor]) -> list:
        """Per input: the 2-D (or 0-D) shape the kernel addresses it by, or None when it is used
        as it is.  A with leading batch dimensions is flattened to ``[M, K]``; epilogue operands
        are lined up with the flattened ``[M, N]`` tile (full, one per row, one per column, scalar)."""
        views: list = [None] * len(inputs)
        left, right = inputs[self._left_idx], inputs[self._right_idx]
        if left.dim() > 2:
            views[self._left_idx] = (-1, left.shape[-1])
        if left.dim() < 2 or right.dim() != 2:
            return views
        rows = left.numel() // max(1, left.shape[-1])
        n_cols = right.shape[1]
        for idx in self._slot_inputs:
            t = inputs[idx]
            if idx in (self._left_idx, self._right_idx) or t.dim() <= 2:
                continue          # 0-D, 1-D and 2-D operands are addressed by their own strides
            kind = classify_epilogue_operand(t.shape, rows, n_cols)
            if kind is None:
                raise N.NativeLibraryError(
                    f"operand of shape {tuple(t.shape)} does not broadcast to {rows} rows x {n_cols} columns "
                    f"(A {tuple(left.shape)}, B {tuple(right.shape)}, inputs {[tuple(i.shape) for i in inputs]})")
            views[idx] = {"full": (rows, n_cols), "row": (1, n_cols), "col": (rows, 1), "scalar": ()}[kind]
        return views

    @staticmethod
    def _apply_views(inputs: Sequence[torch.Tensor], views: Sequence) -> tuple:
        return tuple(t if v is None else t.reshape(v) for t, v in zip(inputs, views))

    def _output_shapes(self, M: int, Ncols: int):
        """Shapes the graph expects where they differ from the kernel's ``[M, N]`` / ``[M]``:
        (primary, [per escape store], row reductions)."""
        def grouped(desc, numel, last):
            shp = tuple(getattr(desc, "shape", ()) or ())
            n = 1
            for v in shp:
                n *= v
            if len(shp) in (0, 2 if last else 1) or n != numel or (last and shp[-1] != Ncols):
                return None
            return shp
        out_shape = grouped(self._output_descriptor, M * Ncols, True) if self._spec.store_output else None
        aux = [grouped(self._intermediate_descriptors[i], M * Ncols, True) for i in self._aux_slots]
        red_shape = None
        if self._reductions and self._reductions[0].axis == 1:
            if self._row_reduction_shape is not None and _prod(self._row_reduction_shape) == M:
                red_shape = self._row_reduction_shape
        return out_shape, (aux if any(a is not None for a in aux) else None), red_shape

    def _prepare(self, inputs: Sequence[torch.Tensor], key: tuple) -> _Prepared:
        spec = self._spec
        views = self._operand_views(inputs)
        inputs = self._apply_views(inputs, views)
        left, right = inputs[self._left_idx], inputs[self._right_idx]
        if left.dim() != 2 or right.dim() != 2:
            raise N.NativeLibraryError("fused GEMM operands must be 2-D")
        prog = K.EpilogueProgram()
        slot_tensors = [inputs[i] for i in self._slot_inputs]
        prog.operands = list(slot_tensors)
        for st in spec.steps:
            if st.opcode == N.OP_STORE_AUX:
                prog.ops.append((st.opcode, self._aux_slots[st.aux_index], 0.0))
            elif st.input_index >= 0:
                prog.ops.append((st.opcode, self._slot_inputs.index(st.input_index), 0.0))
            else:
                prog.ops.append((st.opcode, 0, st.imm))
        p = _Prepared()
        p.desc = N.GemmDesc()
        out_dtype = self._output_descriptor.dtype if spec.store_output else left.dtype
        M, Ncols, Kd = K.fill_desc(p.desc, left, right, prog, None, out_dtype)
        p.left, p.right = p.desc._keepalive
        p.M, p.N, p.K = M, Ncols, Kd
        # aux (escape-store) operands: row-major [M, N], pointer filled per call
        for aux_index, slot in self._aux_slots.items():
            d = self._intermediate_descriptors[aux_index]
            o = p.desc.operands[slot]
            o.stride_m, o.stride_n, o.dtype = Ncols, 1, K.dtype_code(d.dtype)
            o.ptr = 0x1000
        p.desc.n_operands = len(self._slot_inputs) + len(self._aux_slots)
        if spec.store_output:
            p.desc.d, p.desc.ldd = 0x1000, Ncols      # placeholder pointer for validation / planning
        p.red_len = 0
        if self._reductions:
            kinds = 0
            for r in self._reductions:
                kinds |= _RED_BIT[r.op]
                setattr(p.desc.reduce, _RED_FIELD[r.op], 0x1000)
            axis = self._reductions[0].axis
            p.desc.reduce.kinds = kinds
            p.desc.reduce.axis = _AXIS_CODE[axis]
            p.red_len = M if axis == 1 else (Ncols if axis == 0 else 1)
        p.plan = K.plan_for(p.desc, K.device_props(left.device))
        if self._launch_params is not None and not self._is_autotuned and self._launch_params.block_n in (128, 256):
            if self._launch_params.block_n != p.plan.tile_n:
                p.plan.tile_n = self._launch_params.block_n
                tiles = ((M + 127) // 128) * ((Ncols + p.plan.tile_n - 1) // p.plan.tile_n)
                p.plan.grid = max(1, min(p.plan.grid if p.plan.grid > 0 else tiles, tiles))
        p.tune_key = None
        if self._plan_cache is not None:
            from .plan_cache import apply_entry, plan_key

            key_str = plan_key(torch.cuda.get_device_name(left.device), _build_id(), M, Ncols, Kd, p.desc.ab_dtype,
                               p.desc.out_dtype, "k" if right.stride(0) == 1 else "n",
                               spec.signature()[:16] + ":" + ",".join(f"{o.stride_m and 1}{o.stride_n and 1}{o.dtype}"
                                                                       for o in p.desc.operands[:p.desc.n_operands]))
            entry = self._plan_cache.get(key_str)
            if entry is None or not apply_entry(p.plan, entry):
                p.tune_key = key_str if self._autotune else None
        p.ws_bytes = int(self._lib.fuseml_sm100_workspace_bytes(C.byref(p.desc), C.byref(p.plan)))
        if p.ws_bytes < 0:
            raise N.NativeLibraryError("fuseml_sm100_workspace_bytes rejected the descriptor")
        p.ws = {}
        p.b_tag = {}
        p.views = views if any(v is not None for v in views) else None
        p.out_shape, p.aux_shapes, p.red_shape = self._output_shapes(M, Ncols)
        self._prepared[key] = p
        logger.debug("prepared launch M=%d N=%d K=%d tile_n=%d grid=%d ws=%d B", M, Ncols, Kd,
                     p.plan.tile_n, p.plan.grid, p.ws_bytes)
        return p

    # ------------------------------------------------------------------ hot path
    def __call__(self, *input_tensors: torch.Tensor):
        if len(input_tensors) != len(self._input_descriptors):
            raise ValueError(f"Expected {len(self._input_descriptors)} input tensor(s), got {len(input_tensors)}.")
        if not self._skip_stride_check:
            input_tensors = tuple(self._materialize_if_needed(t) for t in input_tensors)
        if self._lib is None:
            self._lib = N.load()
        # TMA reads A and B in place and needs 16-byte aligned bases.  The compile-time check
        # sees shapes and strides only; a live tensor may still be a view that starts in the
        # middle of a 16-byte word (a column slice).  Such an operand is copied once into a fresh,
        # aligned buffer (as negative strides are), and the fused kernel runs on the copy.
        li, ri = self._left_idx, self._right_idx
        if (input_tensors[li].data_ptr() | input_tensors[ri].data_ptr()) & 15 and input_tensors[li].dtype != torch.float32:
            input_tensors = tuple(t.clone(memory_format=torch.contiguous_format)
                                  if i in (li, ri) and t.data_ptr() & 15 else t for i, t in enumerate(input_tensors))
        key = tuple((t.shape, t.stride()) for t in input_tensors)
        p = self._prepared.get(key)
        if p is None:
            p = self._prepare(input_tensors, key)
        spec = self._spec
        desc = p.desc
        if p.views is not None:
            input_tensors = self._apply_views(input_tensors, p.views)
        left, right = input_tensors[self._left_idx], input_tensors[self._right_idx]
        left = K.addressable_left(left, right)      # same decision as when the descriptor was prepared
        device = left.device
        desc.a = left.data_ptr()
        desc.b = right.data_ptr()
        operands = desc.operands
        for slot, idx in enumerate(self._slot_inputs):
            operands[slot].ptr = input_tensors[idx].data_ptr()
        outputs: list[torch.Tensor] = []
        primary = None
        if spec.store_output:
            primary = torch.empty_strided((p.M, p.N), (p.N, 1), dtype=self._output_descriptor.dtype, device=device)
            desc.d = primary.data_ptr()
        aux_out = []
        for aux_index, slot in self._aux_slots.items():
            d = self._intermediate_descriptors[aux_index]
            t = torch.empty_strided((p.M, p.N), (p.N, 1), dtype=d.dtype, device=device)
            operands[slot].ptr = t.data_ptr()
            aux_out.append(t)
        red_out = []
        if self._reductions:
            shape = (p.red_len,) if self._reductions[0].axis != 2 else ()
            for r in self._reductions:
                t = torch.empty(shape, dtype=torch.float32, device=device)
                setattr(desc.reduce, _RED_FIELD[r.op], t.data_ptr())
                red_out.append(t)
        stream = torch.cuda.current_stream(device).cuda_stream
        if p.ws_bytes:
            ws = p.ws.get(stream)
            if ws is None:
                ws = p.ws[stream] = torch.empty(p.ws_bytes, dtype=torch.uint8, device=device)
            desc.reduce.workspace = ws.data_ptr()
            desc.reduce.workspace_bytes = p.ws_bytes
            if left.dtype == torch.float32:
                # fp32 operands are expanded into the workspace before the MMA.  This workspace is
                # private to (signature, stream): when B is the same storage at the same version
                # as in the previous launch here (a weight), its expansion is still valid.
                # (Never while a CUDA graph is being captured: a replay cannot re-check the weight.)
                tag = (right.data_ptr(), right._version)
                reuse = p.b_tag.get(stream) == tag and not torch.cuda.is_current_stream_capturing()
                p.plan.flags = (p.plan.flags & ~N.PLAN_B_EXPANSION_VALID) | (N.PLAN_B_EXPANSION_VALID if reuse else 0)
                p.b_tag[stream] = tag
        if p.tune_key is not None and not torch.cuda.is_current_stream_capturing():
            self._tune(p, desc, device, stream)
        if device.index is not None and device.index != torch.cuda.current_device():
            with torch.cuda.device(device):
                rc = self._lib.fuseml_sm100_gemm_epilogue(C.byref(desc), C.byref(p.plan), C.c_void_p(stream))
        else:
            rc = self._lib.fuseml_sm100_gemm_epilogue(C.byref(desc), C.byref(p.plan), C.c_void_p(stream))
        if rc != N.OK:
            N.check(rc, "fuseml_sm100_gemm_epilogue")
        self.launch_count += 1
        # reductions come back in fp32; hand them over in the dtype the graph expects
        red_out = [t if t.dtype == dt else t.to(dt) for t, dt in zip(red_out, self._reduction_dtypes)]
        # the kernel works on [M, N]; the graph may see the rows grouped ([B, S, N], [B, S])
        if p.out_shape is not None and primary is not None:
            primary = primary.view(p.out_shape)
        if p.aux_shapes is not None:
            aux_out = [t if shp is None else t.view(shp) for t, shp in zip(aux_out, p.aux_shapes)]
        if p.red_shape is not None:
            red_out = [t.view(p.red_shape) for t in red_out]
        if primary is not None:
            outputs.append(primary)
        outputs.extend(aux_out)
        if primary is None and red_out and not aux_out and len(red_out) == 1:
            return red_out[0]
        if primary is None and red_out:   # the first reduction is the group's primary output
            return (red_out[0], *aux_out, *red_out[1:])
        outputs.extend(red_out)
        return outputs[0] if len(outputs) == 1 else tuple(outputs)

    def _tune(self, p: _Prepared, desc, device, stream) -> None:
        """First call of a signature with autotuning on: time the router's plan and its neighbours on
        the live tensors (the descriptor is complete at this point), keep the fastest, persist it."""
        from .plan_cache import candidate_plans, entry_of, tune_plan

        key, p.tune_key = p.tune_key, None
        cands = candidate_plans(p.plan, p.M, p.N, K.device_props(device).sm_count, bool(self._reductions))
        sizes = [int(self._lib.fuseml_sm100_workspace_bytes(C.byref(desc), C.byref(c))) for c in cands]
        cands = [c for c, n in zip(cands, sizes) if n >= 0]
        need = max([n for n in sizes if n >= 0] + [0])
        saved_ws = (desc.reduce.workspace, desc.reduce.workspace_bytes)
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
        desc.reduce.workspace, desc.reduce.workspace_bytes = scratch.data_ptr(), need

        def launch(plan) -> None:
            with torch.cuda.device(device):
                N.check(self._lib.fuseml_sm100_gemm_epilogue(C.byref(desc), C.byref(plan), C.c_void_p(stream)), "tuning launch")

        best, us, tried = tune_plan(launch, cands)
        desc.reduce.workspace, desc.reduce.workspace_bytes = saved_ws
        if best is None:
            return
        p.plan = best
        p.ws_bytes = int(self._lib.fuseml_sm100_workspace_bytes(C.byref(desc), C.byref(best)))
        p.ws, p.b_tag = {}, {}
        if p.ws_bytes:
            ws = p.ws[stream] = torch.empty(p.ws_bytes, dtype=torch.uint8, device=device)
            desc.reduce.workspace, desc.reduce.workspace_bytes = ws.data_ptr(), p.ws_bytes
        self.tuned_signatures += 1
        self._plan_cache.put(key, entry_of(best, us, tried))
        logger.info("tuned M=%d N=%d K=%d: tile_n=%d cluster=%d group_m=%d split_k=%d, %.1f us (%d candidates)",
                    p.M, p.N, p.K, best.tile_n, best.cluster, best.group_m, best.split_k, us, tried)

    def __repr__(self) -> str:
        ins = [d.name for d in self._input_descriptors]
        red = f", reductions={[(r.op, r.axis) for r in self._reductions]}" if self._reductions else ""
        lp = self._launch_params
        blk = f"block=({lp.block_m},{lp.block_n},{lp.block_k})" if lp is not None else "block=(router)"
        return (f"KernelLauncher(inputs={ins}, output={self._output_descriptor.name!r}, "
                f"intermediates={[d.name for d in self._intermediate_descriptors]}, {blk}{red})")


class FusedMLPLauncher:
    """Two chained launchers, ``h = first(...)`` and ``y = second(..., h, ...)``, run as ONE kernel
    when the batch has at most 128 rows: ``fuseml_sm100_mlp_small`` computes both Linears with the
    intermediate handed over in shared memory (decode-sized batches, small fp32 blocks).  Any other
    call (more rows, a layout the kernel does not take) runs the two fused launches one after the
    other, exactly as the graph did before the pair was merged.

    Inputs: the first launcher's inputs followed by the second's without its left operand.
    The reference has no counterpart: its two Linears are always two kernels with ``h`` in HBM
    (benchmarks/bench_mlp_block.py:160-182)."""

    def __init__(self, first: KernelLauncher, second: KernelLauncher) -> None:
        self.__name__ = "fuseml_fused_mlp"
        self.first, self.second = first, second
        self._n1 = len(first._input_descriptors)
        self._pos = second._left_idx                       # where h sits among the second launcher's inputs
        self._ws: dict = {}
        self._declined: set = set()
        self.fused_count = 0
        self.launch_count = 0

    @staticmethod
    def mergeable(first: KernelLauncher, second: KernelLauncher) -> bool:
        """Static conditions: plain stored outputs, no reductions, no escape stores on either side."""
        for L in (first, second):
            sp = L._spec
            if sp.reductions or sp.n_aux or not sp.store_output or L._aux_slots:
                return False
        return first._output_descriptor.dtype == first._input_descriptors[first._left_idx].dtype

    @staticmethod
    def _program(launcher: KernelLauncher, inputs: Sequence[torch.Tensor]) -> K.EpilogueProgram:
        prog = K.EpilogueProgram()
        for st in launcher._spec.steps:
            if st.input_index >= 0:
                prog.ops.append((st.opcode, prog._slot(inputs[st.input_index]), 0.0))
            else:
                prog.ops.append((st.opcode, 0, st.imm))
        return prog

    def __call__(self, *tensors: torch.Tensor):
        a1 = tensors[:self._n1]
        rest = tensors[self._n1:]
        x, w1v = a1[self.first._left_idx], a1[self.first._right_idx]
        w2v = rest[self.second._right_idx - (1 if self.second._right_idx > self._pos else 0)]
        key = (x.shape, x.stride(), w1v.stride(), w2v.shape, w2v.stride(), x.dtype)
        # nn.Linear weights reach the launchers as aten.t views: stride (1, K) means the storage is [N, K] row-major
        fusable = (key not in self._declined and x.dim() == 2 and x.shape[0] <= 128 and x.stride(1) == 1
                   and w1v.dim() == 2 and w2v.dim() == 2 and w1v.stride(0) == 1 and w2v.stride(0) == 1)
        if fusable:
            a2 = list(rest)
            a2.insert(self._pos, None)                      # h has no tensor in the fused form
            try:
                stream = torch.cuda.current_stream(x.device).cuda_stream
                ws = self._ws.get((key, stream))
                y = K.fused_mlp(x, w1v.t(), w2v.t(), self._program(self.first, a1), self._program(self.second, a2),
                                out_dtype=self.second._output_descriptor.dtype, workspace=ws)
                if ws is None:
                    self._ws[(key, stream)] = K.last_mlp_workspace()
                self.fused_count += 1
                self.launch_count += 1
                return y
            except N.NativeLibraryError as exc:
                self._declined.add(key)
                logger.info("MLP block runs as two launches: %s", exc)
        h = self.first(*a1)
        a2 = list(rest)
        a2.insert(self._pos, h)
        self.launch_count += 1
        return self.second(*a2)
