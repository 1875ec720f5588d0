"""``torch.compile`` backend: ``torch.compile(model, backend=FuseMLCompiler())``.

Pipeline per captured graph (same stages as the reference, fuseml/compiler.py:173-437):
Dynamo graph -> ``aot_module_simplified`` (ATen level: ``nn.Linear`` becomes ``aten.t`` +
``aten.addmm``) -> control-flow validation -> fusion discovery -> *lowering check* ->
graph surgery -> one :class:`KernelLauncher` per placeholder node.

What differs from the reference:

* one tier.  Its pre-scan sent tiny outputs to eager, "compute-bound" GEMMs to cuBLAS Lt and
  the rest to Triton (``:262-299``).  Here every discovered chain runs the sm_100a kernel; the
  roofline router only decides tile shapes.  ``fusion_strategy`` is ``"sm100"`` or ``"none"``.
* groups are lowered to a :class:`KernelSpec` and checked for TMA-addressable layouts *before*
  surgery; a group that cannot be expressed is left in the graph as ordinary ATen ops (it was
  never "matched"), instead of failing at the first launch.
* discovery runs with the DAG / multi-reduction / global-reduction / bare-trigger extensions
  switched on (keyword arguments; the pass itself defaults to the reference's behaviour): no
  ``addmm`` / ``mm`` of a compiled graph is left to a library GEMM.
* graphs whose tensors live on the CPU are not lowered at all: the fused path has no CPU
  implementation, so the module is handed back unchanged, as the reference does whenever it
  finds nothing to fuse (``:219-228``).
"""
from __future__ import annotations

import os
from typing import Any, Callable

import torch
from functorch.compile import make_boxed_func
from torch._functorch.aot_autograd import aot_module_simplified

from ._logging import logger
from .codegen.kernel_cache import KernelCache, TensorFingerprint, _materialize_ints, build_cache_key
from .codegen.kernel_generator import (_RED_KIND, KernelSpec, Sm100KernelGenerator, TensorDescriptor,
                                       UnsupportedChainError)
from .codegen.kernel_launcher import KernelLauncher
from .fusion_group import FusionGroup
from .passes.control_flow_validation import ControlFlowError, validate_graph_control_flow
from .passes.fusion_pass import FuseMLFusionPass, fuseml_fused_kernel_placeholder
from .passes.graph_cut import split_fusion_group
from .passes.topology import classify_epilogue_operand, is_trigger
from .registry import SupportedOpsRegistry, build_default_registry

_SUPPORTED_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


class _NoFusionPossible(Exception):
    """Nothing in the graph will run as a fused kernel: hand back the original forward."""


def _node_to_descriptor(node: torch.fx.Node) -> TensorDescriptor | None:
    """Descriptor from ``meta['tensor_meta']`` (ShapeProp) or ``meta['val']`` (FakeTensor)."""
    tm = node.meta.get("tensor_meta")
    if tm is not None and not hasattr(tm, "shape"):
        tm = tm[0] if isinstance(tm, (tuple, list)) and len(tm) > 0 else None
    if tm is not None and hasattr(tm, "shape"):
        return TensorDescriptor(node.name, _materialize_ints(tm.shape), _materialize_ints(tm.stride), tm.dtype)
    val = node.meta.get("val")
    if val is not None and hasattr(val, "shape"):
        shape = _materialize_ints(val.shape)
        stride = _materialize_ints(val.stride()) if callable(getattr(val, "stride", None)) else (1,) * len(shape)
        return TensorDescriptor(node.name, shape, stride, val.dtype)
    return None


def _descriptor_from_metadata(name: str, meta: dict) -> TensorDescriptor | None:
    if not meta or "shape" not in meta:
        return None
    return TensorDescriptor(name, _materialize_ints(meta["shape"]), _materialize_ints(meta["stride"]), meta["dtype"])


def _graph_device(gm: torch.fx.GraphModule, inputs) -> torch.device | None:
    for t in inputs or ():
        if isinstance(t, torch.Tensor):
            return t.device
    for n in gm.graph.nodes:
        v = n.meta.get("val")
        if isinstance(v, torch.Tensor):
            return v.device
    return None


class FuseMLCompiler:
    """Backend object; one per compiled model.  ``registry`` as in the reference.

    Attributes kept from the reference: ``fusion_candidates`` (trigger nodes seen),
    ``fusion_applied``, ``fusion_strategy``; plus ``launchers`` (the callables put into the
    graph) and ``declined`` (groups left to eager, with the reason).
    """

    def __init__(self, registry: SupportedOpsRegistry | None = None, *, dag_epilogue: bool = True,
                 multi_reduction: bool = True, global_reductions: bool = True, bare_trigger: bool = True,
                 backward: bool = True, fuse_mlp: bool = False, plan_cache: Any = None,
                 autotune: bool | None = None) -> None:
        self.registry: SupportedOpsRegistry = registry or build_default_registry()
        self.fusion_candidates: list = []
        self.fusion_applied: bool = False
        self.fusion_strategy: str = "none"
        self.launchers: list[KernelLauncher] = []
        # launchers put into backward graphs (a subset of `launchers`); `backward=False` leaves
        # backward graphs to PyTorch, as the reference does (it passes only a forward compiler,
        # fuseml/compiler.py:214-218)
        self.backward_launchers: list[KernelLauncher] = []
        self.fuse_backward = bool(backward)
        # `fuse_mlp=True`: pairs of chained launchers are merged into one call that runs both Linears
        # in one kernel when the batch has at most 128 rows (FusedMLPLauncher).  Off by default: at
        # the sizes measured (128 x 512 x 2048 x 512) the one kernel, a serial chain of two K loops
        # and two epilogues per CTA, is on a par with the two split-K launches at best (1-5 % slower)
        self.mlp_launchers: list = []
        self.fuse_mlp = bool(fuse_mlp)
        self.declined: list[tuple[str, str]] = []
        self._options = dict(dag_epilogue=dag_epilogue, multi_reduction=multi_reduction,
                             global_reductions=global_reductions, bare_trigger=bare_trigger, backward_ops=True)
        self._generator = Sm100KernelGenerator()
        self._cache = KernelCache()
        # Measured launch plans on disk (codegen/plan_cache.py).  `plan_cache` is a PlanCache, a
        # path, or None: then the file named by FUSEML_PLAN_CACHE (or the default under ~/.cache)
        # is used when that variable is set or autotuning is on.  `autotune` (default: the
        # FUSEML_AUTOTUNE environment variable) times candidate plans on the first call of every
        # new shape and stores the winner there.
        from .codegen import plan_cache as _pc

        self.autotune = _pc.autotune_requested() if autotune is None else bool(autotune)
        if isinstance(plan_cache, _pc.PlanCache):
            self.plan_cache = plan_cache
        elif plan_cache is not None:
            self.plan_cache = _pc.PlanCache(plan_cache)
        elif self.autotune or os.environ.get(_pc.ENV_PATH):
            self.plan_cache = _pc.PlanCache()
        else:
            self.plan_cache = None

    # ------------------------------------------------------------------ torch.compile entry
    def __call__(self, gm: torch.fx.GraphModule, example_inputs: list) -> Callable:
        def fw_compiler(aten_gm: torch.fx.GraphModule, aten_inputs: list) -> Callable:
            return make_boxed_func(self._compile_aten_graph(aten_gm, aten_inputs))

        def bw_compiler(aten_gm: torch.fx.GraphModule, aten_inputs: list) -> Callable:
            # Backward graphs go through the same discovery: dgrad GEMMs with their pointwise tails
            # (mm -> gelu_backward, mm -> add of the residual's gradient) and the wgrad GEMMs
            # dY^T @ X, whose transposed left operand the kernel reads in place.  A backward graph
            # with nothing to fuse, or any failure to lower it, leaves it to PyTorch.
            if self.fuse_backward:
                n_before = len(self.launchers)
                try:
                    fn = self._compile_aten_graph(aten_gm, aten_inputs)
                    self.backward_launchers.extend(self.launchers[n_before:])
                    return make_boxed_func(fn)
                except _NoFusionPossible as exc:
                    logger.info("backward graph left to PyTorch: %s", exc)
            return make_boxed_func(aten_gm.forward)

        try:
            return aot_module_simplified(gm, example_inputs, fw_compiler=fw_compiler, bw_compiler=bw_compiler,
                                         inference_compiler=fw_compiler)
        except _NoFusionPossible as exc:
            self.fusion_applied = False
            logger.info("Bypassing AOT decomposition — %s", exc)
            return gm.forward

    # ------------------------------------------------------------------ ATen-level compilation
    def _compile_aten_graph(self, gm: torch.fx.GraphModule, example_inputs: list) -> Callable:
        try:
            validate_graph_control_flow(gm)
        except ControlFlowError as exc:
            raise _NoFusionPossible(f"data-dependent control flow: {exc}") from exc

        triggers = [n for n in gm.graph.nodes if is_trigger(n)]
        self.fusion_candidates.extend(triggers)
        if not triggers:
            raise _NoFusionPossible("no addmm / mm in the graph")
        device = _graph_device(gm, example_inputs)
        if device is None or device.type != "cuda":
            raise _NoFusionPossible(f"tensors live on {device}; fused kernels exist for CUDA (sm_100a) only")

        fpass = FuseMLFusionPass(gm, self.registry, **self._options)
        fpass._tensor_meta_from_val()
        if not any("tensor_meta" in n.meta for n in gm.graph.nodes if n.op == "call_function"):
            from torch.fx.passes.shape_prop import ShapeProp

            ShapeProp(gm).propagate(*example_inputs)

        accepted: list[tuple[FusionGroup, KernelSpec]] = []
        for found in fpass._find_fusion_groups():
            candidates = [found]
            if not found.extra_outputs and found.store_output:
                candidates = [s.group for s in split_fusion_group(found) if s.kind == "fused" and s.group is not None]
            for group in candidates:
                try:
                    spec = self._generator.build_spec(group)
                    self._check_layouts(group, spec)
                except UnsupportedChainError as exc:
                    self.declined.append((repr(group), str(exc)))
                    logger.info("Leaving %s to eager: %s", group, exc)
                    continue
                accepted.append((group, spec))
        if not accepted:
            raise _NoFusionPossible("no chain can be lowered to the sm_100a kernel")

        # Build the launchers first (descriptors need the pre-surgery metadata), then cut the graph.
        launcher_of: dict[int, KernelLauncher] = {}
        for group, spec in accepted:
            launcher_of[id(group)] = self._build_launcher(group, spec)
        fpass._apply_surgery([g for g, _ in accepted])

        graph = gm.graph
        for node in list(graph.nodes):
            if node.op == "call_function" and node.target is fuseml_fused_kernel_placeholder:
                launcher = launcher_of[id(node.meta["fusion_group"])]
                with graph.inserting_after(node):
                    call = graph.call_function(launcher, args=node.args)
                call.meta.update({k: v for k, v in node.meta.items() if k in ("tensor_meta", "val", "fusion_group")})
                node.replace_all_uses_with(call)
                graph.erase_node(node)
        if self.fuse_mlp:
            self._merge_mlp_pairs(graph)
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
        self.fusion_applied = True
        self.fusion_strategy = "sm100"
        logger.info("FuseML: %d fused kernel(s) in graph (%d declined)", len(accepted), len(self.declined))
        return gm.forward

    def _merge_mlp_pairs(self, graph: torch.fx.Graph) -> None:
        """``second(..., first(...), ...)`` with the first launcher's output feeding only the second's
        left operand, plain stored outputs on both sides and at most 128 rows: one FusedMLPLauncher."""
        from .codegen.kernel_launcher import FusedMLPLauncher

        for node in list(graph.nodes):
            if node.op != "call_function" or not isinstance(node.target, KernelLauncher):
                continue
            second = node.target
            left = node.args[second._left_idx]
            if not (isinstance(left, torch.fx.Node) and left.op == "call_function" and isinstance(left.target, KernelLauncher)):
                continue
            first = left.target
            if len(left.users) != 1 or sum(1 for a in node.args if a is left) != 1:
                continue
            rows_shape = first._input_descriptors[first._left_idx].shape
            if len(rows_shape) != 2 or rows_shape[0] > 128 or not FusedMLPLauncher.mergeable(first, second):
                continue
            merged = FusedMLPLauncher(first, second)
            args = tuple(left.args) + tuple(a for i, a in enumerate(node.args) if i != second._left_idx)
            with graph.inserting_after(node):
                call = graph.call_function(merged, args=args)
            call.meta.update({k: v for k, v in node.meta.items() if k in ("tensor_meta", "val")})
            node.replace_all_uses_with(call)
            graph.erase_node(node)
            graph.erase_node(left)
            self.mlp_launchers.append(merged)
            logger.info("merged %s and %s into one small-M MLP launch", first, second)

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _check_layouts(group: FusionGroup, spec: KernelSpec) -> None:
        """Reject before surgery what the launch would reject: dtypes, ranks, TMA-addressable strides."""
        descs = [_node_to_descriptor(n) for n in group.inputs]
        if any(d is None for d in descs):
            raise UnsupportedChainError("missing shape metadata on a group input")
        left, right = descs[spec.left_index], descs[spec.right_index]
        if len(left.shape) < 2 or len(right.shape) != 2:
            raise UnsupportedChainError("GEMM operands: A needs at least two dimensions, B exactly two")
        if left.dtype != right.dtype or left.dtype not in _SUPPORTED_DTYPES:
            raise UnsupportedChainError(f"operand dtypes {left.dtype} / {right.dtype}")
        if 0 in left.shape or 0 in right.shape:
            raise UnsupportedChainError("empty GEMM operand")
        if len(left.shape) > 2:
            # [B, S, K] activations: the launcher flattens the leading dimensions (a view when
            # they collapse, a contiguous copy otherwise), so A is checked as row-major [M, K]
            rows = 1
            for v in left.shape[:-1]:
                rows *= v
            kdim = left.shape[-1]
            left = TensorDescriptor(left.name, (rows, kdim), (kdim, 1), left.dtype)
        if left.dtype != torch.float32:
            for d, role in ((left, "A"), (right, "B")):
                fp = TensorFingerprint(d.shape, d.stride, 0, True, str(d.dtype), tuple(s == 0 for s in d.stride))
                if role == "A" and d.stride[1] != 1:
                    continue  # the launcher makes a contiguous copy of a transposed activation
                if not fp.tma_legal:
                    raise UnsupportedChainError(f"{role} operand {d.name} stride {d.stride}: rows are not multiples of 16 bytes")
        M, Ncols = left.shape[0], right.shape[1]
        for st in spec.steps:
            if st.input_index >= 0:
                d = descs[st.input_index]
                if d.dtype not in _SUPPORTED_DTYPES:
                    raise UnsupportedChainError(f"epilogue operand {d.name}: dtype {d.dtype}")
                if classify_epilogue_operand(d.shape, M, Ncols) is None:
                    raise UnsupportedChainError(f"epilogue operand {d.name} of shape {d.shape} does not broadcast to "
                                                f"{M} rows x {Ncols} columns")
        out = group.output_metadata
        if spec.store_output and out.get("dtype") not in _SUPPORTED_DTYPES:
            src = group.output_node if not group.extra_outputs else group.output_node
            d = _node_to_descriptor(src)
            if d is None or d.dtype not in _SUPPORTED_DTYPES:
                raise UnsupportedChainError("output dtype not supported")

    def _build_launcher(self, group: FusionGroup, spec: KernelSpec) -> KernelLauncher:
        descs = []
        for n in group.inputs:
            d = _node_to_descriptor(n)
            if d is None:
                raise UnsupportedChainError(f"input {n.name} has no metadata")
            descs.append(d)
        matrix_node = group.output_node
        out_desc = _node_to_descriptor(matrix_node) or _descriptor_from_metadata("out", group.output_metadata)
        inter = [_node_to_descriptor(n) for n in group.intermediate_outputs]
        red_nodes = [n for n in group.all_nodes if n.op == "call_function" and n.target in _RED_KIND]
        red_dtypes = []
        red_shape = None
        for n in red_nodes[:len(spec.reductions)]:
            d = _node_to_descriptor(n)
            red_dtypes.append(d.dtype if d is not None else torch.float32)
            if d is not None and red_shape is None:
                red_shape = d.shape
        if len(red_dtypes) != len(spec.reductions):
            red_dtypes = [torch.float32] * len(spec.reductions)

        key = build_cache_key(group, {}, plan=(spec.signature(),))
        if key is not None:
            hit = self._cache.lookup(key)
            if hit is not None:
                self.launchers.append(hit)
                return hit
        launcher = KernelLauncher(
            spec, descs, out_desc, inter, descs[spec.left_index].name, descs[spec.right_index].name,
            is_autotuned=True, reduction_dtypes=red_dtypes, reduction_shape=red_shape,
            plan_cache=self.plan_cache, autotune=self.autotune)
        if key is not None:
            self._cache.store(key, launcher)
        self.launchers.append(launcher)
        return launcher

    # counters, as in the reference
    @property
    def kernel_cache(self) -> KernelCache:
        return self._cache
