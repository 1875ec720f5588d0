"""Discovery of fusible chains in an ATen-level FX graph, and the graph surgery that
replaces each chain with one call.

Default behaviour matches the reference pass (fuseml/passes/fusion_pass.py:98-347 discovery,
:644-887 surgery): starting at every ``addmm`` / ``mm`` the pass walks forward while the
current node has exactly one user, absorbing pointwise ops, shape-preserving views and
alias-safe in-place ops, and ending at a ``keepdim=False`` reduction, a barrier or an unknown
op; groups of a single node are dropped.  Surgery inserts a
``fuseml_fused_kernel_placeholder`` node whose args are the group's external inputs (the
kernel's argument order), rewires consumers (``getitem`` nodes for multi-output groups),
removes the dead originals and checks the graph is still acyclic.

What the sm_100a backend can express beyond that is opt-in (constructor keywords, all off
by default so that structural behaviour stays drop-in):

* ``dag_epilogue``      a value with two pointwise branches that re-join (``gelu(h) * sigmoid(h)``)
                        is absorbed as a diamond (evaluated with the epilogue's second register);
* ``multi_reduction``   several reductions of the same tensor become outputs of one kernel; the
                        matrix itself is only written if something else still reads it;
* ``global_reductions`` whole-tensor ``sum`` / ``amax`` / ``mean`` are accepted as reduction tails;
* ``bare_trigger``      an ``addmm`` / ``mm`` that absorbs nothing is still a group (the reference drops
                        it, fuseml/passes/fusion_pass.py:332-333, and the GEMM then runs in a library):
                        a bias is an epilogue, and a lone ``mm`` is the same kernel with an empty program;
* ``backward_ops``      pointwise ops of backward graphs (``aten.gelu_backward(grad, pre)``) are absorbed
                        when the chain value is their gradient argument: ``mm -> gelu_backward`` is the
                        data-gradient GEMM of a Linear -> GELU pair with ``gelu'(pre)`` as its epilogue.
"""
from __future__ import annotations

import operator as _operator
from typing import Any, Callable

import torch
from torch.fx.passes.shape_prop import ShapeProp

from .._logging import logger
from ..codegen.kernel_cache import _materialize_ints
from ..fusion_group import FusionGroup
from ..registry import SupportedOpsRegistry, build_default_registry
from .graph_cut import split_fusion_group, validate_fusion_group  # noqa: F401  (re-exported)
from .mutation_safety import is_safe_inplace
from .topology import (ABSORBABLE_OPS, BACKWARD_ABSORBABLE_OPS, BARRIER_OPS, GLOBAL_REDUCTION_OPS, INPLACE_OPS, REDUCTION_OPS,  # noqa: F401
                       TRANSPARENT_OPS, TRIGGER_OPS, NodeRole, classify_node, gemm_roofline,
                       RESHAPE_OPS, is_compute_bound_gemm, is_trigger, reduction_axis_code,
                       resolve_through_reshapes, resolve_to_defining_node, symint_safe_eq, symint_safe_len)

_aten = torch.ops.aten


def fuseml_fused_kernel_placeholder(*args):
    """Symbolic target of fused nodes between surgery and launcher substitution."""
    raise RuntimeError(
        "fuseml_fused_kernel_placeholder should never be called directly. "
        "It must be replaced by a compiled kernel launcher before execution.")


def _node_shape(n: Any):
    if not isinstance(n, torch.fx.Node):
        return None
    meta = n.meta.get("tensor_meta")
    if meta is not None and hasattr(meta, "shape"):
        return meta.shape
    val = n.meta.get("val")
    if val is not None and hasattr(val, "shape"):
        return val.shape
    return None


def _trigger_mnk(node: torch.fx.Node):
    """(M, N, K) of an addmm / mm trigger from metadata, or None."""
    args = node.args
    pair = args[1:3] if node.target is _aten.addmm.default and len(args) >= 3 else args[0:2]
    if len(pair) < 2:
        return None
    a, b = _node_shape(pair[0]), _node_shape(pair[1])
    if a is None or b is None or len(a) < 2 or len(b) < 2:
        return None
    try:
        return int(a[-2]), int(b[-1]), int(a[-1])
    except (TypeError, ValueError):
        return None


def _reduction_axis(node: torch.fx.Node):
    """'n' (per row), 'm' (per column), 'all', or None if the dims are not a reduction the kernel
    runs.  Rows are the flattened leading dimensions of the reduced tensor."""
    if node.target in GLOBAL_REDUCTION_OPS:
        return "all"
    shape = _node_shape(node.args[0]) if node.args else None
    rank = len(shape) if shape is not None else 2
    dims = node.args[1] if len(node.args) > 1 else []
    return reduction_axis_code(dims, rank)


def _reduction_keepdim(node: torch.fx.Node) -> bool:
    if node.target in GLOBAL_REDUCTION_OPS:
        return False
    return bool(node.args[2]) if len(node.args) > 2 else bool(node.kwargs.get("keepdim", False))


class FuseMLFusionPass:
    """Two phases: ``_find_fusion_groups`` (read-only) and ``_apply_surgery`` (rewrites the graph)."""

    _BARRIER_OPS: set[Callable] = BARRIER_OPS
    _ABSORBABLE_OPS: set[Callable] = ABSORBABLE_OPS
    _REDUCTION_OPS: set[Callable] = REDUCTION_OPS
    # The reference skipped chains whose output had fewer elements than this because a Triton
    # dispatch cost more than the saved round trip (fuseml/passes/fusion_pass.py:463-498).  Kept as
    # a queryable helper; the compiler no longer bypasses on it.
    _MIN_FUSION_OUTPUT_ELEMENTS: int = 500_000

    def __init__(self, graph_module: torch.fx.GraphModule, registry: SupportedOpsRegistry | None = None, *,
                 dag_epilogue: bool = False, multi_reduction: bool = False, global_reductions: bool = False,
                 bare_trigger: bool = False, backward_ops: bool = False) -> None:
        self.graph_module = graph_module
        self.registry = registry or build_default_registry()
        self.dag_epilogue = dag_epilogue
        self.multi_reduction = multi_reduction
        self.global_reductions = global_reductions
        self.bare_trigger = bare_trigger
        self.backward_ops = backward_ops

    # ------------------------------------------------------------------ discovery
    def _find_fusion_groups(self) -> list[FusionGroup]:
        groups: list[FusionGroup] = []
        claimed: set = set()
        for node in self.graph_module.graph.nodes:
            if not is_trigger(node) or node in claimed:
                continue
            group = self._grow_group(node, claimed)
            self._resolve_get_attr_bindings(group)
            if len(group) > 1 or self.bare_trigger:
                group.output_metadata = self._extract_tensor_metadata(group.output_node)
                group.original_inputs = list(group.inputs)
                for n in group.all_nodes:
                    group.node_args_snapshot[n.name] = tuple(n.args)
                logger.debug("Fusion group found: %s", group)
                groups.append(group)
        return groups

    def _grow_group(self, trigger: torch.fx.Node, claimed: set) -> FusionGroup:
        group = FusionGroup(base_node=trigger)
        members: set = {trigger}
        claimed.add(trigger)
        self._collect_external_inputs(trigger, members, group)

        def take(n: torch.fx.Node, is_output: bool = True) -> None:
            group.fused_nodes.append(n)
            if is_output:
                group.output_node = n
            members.add(n)
            claimed.add(n)
            self._collect_external_inputs(n, members, group)

        cur = trigger
        while True:
            users = list(cur.users)
            if len(users) != 1:
                if self.dag_epilogue and len(users) == 2:
                    diamond = self._match_diamond(cur, members)
                    if diamond is not None:
                        for n in diamond:
                            take(n)
                        cur = diamond[-1]
                        continue
                if self.multi_reduction and len(users) >= 2:
                    self._absorb_reduction_fanout(cur, users, group, take)
                break
            nxt = users[0]
            role = classify_node(nxt)
            if role is NodeRole.UNKNOWN and self.global_reductions and nxt.op == "call_function" \
                    and nxt.target in GLOBAL_REDUCTION_OPS:
                role = NodeRole.REDUCTION
            if role is NodeRole.UNKNOWN and self.backward_ops and nxt.op == "call_function" \
                    and nxt.target in BACKWARD_ABSORBABLE_OPS and nxt.args and nxt.args[0] is cur \
                    and all(a is not cur for a in nxt.args[1:]):
                role = NodeRole.ABSORBABLE
            if role in (NodeRole.UNKNOWN, NodeRole.BARRIER):
                break
            if role is NodeRole.REDUCTION:
                if not _reduction_keepdim(nxt) and _reduction_axis(nxt) is not None:
                    take(nxt)
                break
            if role is NodeRole.TRANSPARENT:
                if not (self._is_shape_preserving_2d(nxt) or self._is_row_preserving_view(nxt)):
                    break
                take(nxt, is_output=False)   # a view is never the "real" output
                cur = nxt
                continue
            if role is NodeRole.INPLACE:
                if not is_safe_inplace(nxt, members):
                    logger.debug("stop at in-place op %s: mutated tensor is aliased outside the group", nxt.name)
                    break
                take(nxt)
                cur = nxt
                continue
            if role is NodeRole.ABSORBABLE:
                take(nxt)
                cur = nxt
                continue
            break

        # views after the last real op stay in the graph as views of the fused output: absorbing
        # them would make the kernel store the same values twice (once per name)
        while group.fused_nodes and group.fused_nodes[-1] is not group.output_node \
                and classify_node(group.fused_nodes[-1]) is NodeRole.TRANSPARENT:
            tail = group.fused_nodes.pop()
            members.discard(tail)
            claimed.discard(tail)

        # escape nodes: interior values somebody outside still reads
        extra = set(group.extra_outputs)
        for n in group.all_nodes:
            if n is group.output_node or n in extra:
                continue
            if any(u not in members for u in n.users):
                group.intermediate_outputs.append(n)
        # nothing may escape after a reduction collapsed the tile
        seen_reduction = False
        for n in list(group.all_nodes):
            if n.target in REDUCTION_OPS or n.target in GLOBAL_REDUCTION_OPS:
                seen_reduction = True
            elif seen_reduction and n in group.intermediate_outputs:
                logger.warning("Escape node %s after reduction in group %s — removing (unsafe store).", n.name, group)
                group.intermediate_outputs.remove(n)
        return group

    # -- extensions ---------------------------------------------------------------------
    def _match_diamond(self, fork: torch.fx.Node, members: set):
        """``fork`` has two users.  Follow each as a single-user chain of unary pointwise ops (or
        binary ops with an outside operand) until both meet in one binary pointwise op.  Returns
        the nodes in evaluation order ``[branch A..., branch B..., join]`` or None."""
        order = {n: i for i, n in enumerate(self.graph_module.graph.nodes)}
        fork_pos = order[fork]

        def unary_like(n: torch.fx.Node, prev: torch.fx.Node) -> bool:
            """pointwise op of ``prev`` whose other tensor operands were produced before the fork
            (so they cannot belong to the sibling branch)"""
            if classify_node(n) is not NodeRole.ABSORBABLE:
                return False
            tensor_args = [a for a in n.args if isinstance(a, torch.fx.Node)]
            inside = [a for a in tensor_args if a is prev]
            return len(inside) == 1 and all(a is prev or (a not in members and order[a] < fork_pos)
                                            for a in tensor_args)

        def walk(start: torch.fx.Node):
            chain, prev, n = [], fork, start
            while True:
                chain.append(n)
                if len(n.users) != 1:
                    return chain
                nxt = next(iter(n.users))
                if not unary_like(nxt, n):
                    return chain
                prev, n = n, nxt

        u0, u1 = list(fork.users)
        # direct join: fork feeds the join itself on one side (h * sigmoid(h))
        for a, b in ((u0, u1), (u1, u0)):
            if classify_node(a) is NodeRole.ABSORBABLE and a.target in (_aten.add.Tensor, _aten.mul.Tensor) \
                    and fork in a.args:
                other = [x for x in a.args if isinstance(x, torch.fx.Node) and x is not fork]
                if len(other) == 1 and unary_like(b, fork):
                    chain_b = walk(b)
                    if chain_b[-1] is other[0] and len(chain_b[-1].users) == 1:
                        return [*chain_b, a]
        if not (unary_like(u0, fork) and unary_like(u1, fork)):
            return None
        ca, cb = walk(u0), walk(u1)
        ta, tb = ca[-1], cb[-1]
        if len(ta.users) != 1 or len(tb.users) != 1:
            return None
        join = next(iter(ta.users))
        if join is not next(iter(tb.users)) or join.target not in (_aten.add.Tensor, _aten.mul.Tensor):
            return None
        tensor_args = [x for x in join.args if isinstance(x, torch.fx.Node)]
        if len(tensor_args) != 2 or {id(tensor_args[0]), id(tensor_args[1])} != {id(ta), id(tb)}:
            return None
        return [*ca, *cb, join]

    def _absorb_reduction_fanout(self, cur, users, group, take) -> None:
        """``cur`` feeds several reductions (and possibly other readers): make the reductions
        outputs of this kernel.  All must share one axis and be keepdim=False."""
        def is_red(n):
            return n.op == "call_function" and (n.target in REDUCTION_OPS or
                                                (self.global_reductions and n.target in GLOBAL_REDUCTION_OPS))
        reds = [u for u in users if is_red(u) and not _reduction_keepdim(u)]
        if not reds:
            return
        axes = {_reduction_axis(r) for r in reds}
        if len(axes) != 1 or None in axes:
            return
        others = [u for u in users if u not in reds]
        group.store_output = bool(others)
        primary_is_matrix = bool(others)
        for i, r in enumerate(reds):
            take(r, is_output=(not primary_is_matrix and i == 0))
        group.extra_outputs = reds if primary_is_matrix else reds[1:]
        if primary_is_matrix:
            group.output_node = cur

    # -- helpers shared with the compiler ---------------------------------------------------
    @staticmethod
    def _extract_tensor_metadata(node: torch.fx.Node) -> dict:
        meta = node.meta.get("tensor_meta")
        if meta is not None and not hasattr(meta, "shape"):
            meta = meta[0] if isinstance(meta, (tuple, list)) and len(meta) > 0 else None
        if meta is None or not hasattr(meta, "shape"):
            return {}
        return {"shape": _materialize_ints(meta.shape), "stride": _materialize_ints(meta.stride),
                "dtype": meta.dtype}

    @staticmethod
    def _is_compute_bound_trigger(node: torch.fx.Node, *, min_penalty: float = 0.0) -> bool:
        """Is the tensor roof the bound of this trigger's GEMM?  False when shapes are unknown."""
        mnk = _trigger_mnk(node)
        if mnk is None:
            return False
        meta = node.meta.get("tensor_meta")
        dtype = meta.dtype if meta is not None and hasattr(meta, "dtype") else torch.float32
        n_epi, cur = 0, node
        while len(cur.users) == 1:
            nxt = next(iter(cur.users))
            role = classify_node(nxt)
            if role in (NodeRole.ABSORBABLE, NodeRole.INPLACE):
                n_epi += 1
                cur = nxt
                continue
            if role is NodeRole.REDUCTION:
                n_epi += 1
            break
        return is_compute_bound_gemm(*mnk, dtype, n_epi, min_penalty=min_penalty)

    @staticmethod
    def _is_tiny_output(node: torch.fx.Node) -> bool:
        mnk = _trigger_mnk(node)
        if mnk is None or node.target is not _aten.addmm.default:
            return False
        return mnk[0] * mnk[1] < FuseMLFusionPass._MIN_FUSION_OUTPUT_ELEMENTS

    @staticmethod
    def _collect_external_inputs(node: torch.fx.Node, group_node_set: set, group: FusionGroup) -> None:
        """Append ``node``'s outside producers to ``group.inputs`` (order of first use), looking
        through pure reshapes to the tensor they regroup (``view(x, [B*S, D])`` -> ``x``: the
        launcher flattens it again).  The reference walks back through every view op
        (fuseml/passes/fusion_pass.py:321-331 there); behind a permute, slice or expand the
        defining tensor holds other elements per position, so here those views stay the input."""
        for arg in node.args:
            if not isinstance(arg, torch.fx.Node) or arg in group_node_set:
                continue
            resolved = resolve_through_reshapes(arg)
            src = resolved if resolved not in group_node_set else arg
            if src not in group.inputs:
                group.inputs.append(src)

    @staticmethod
    def _is_shape_preserving_2d(node: torch.fx.Node) -> bool:
        meta = node.meta.get("tensor_meta")
        if meta is None or not hasattr(meta, "shape"):
            return False
        if not node.args or not isinstance(node.args[0], torch.fx.Node):
            return False
        pmeta = node.args[0].meta.get("tensor_meta")
        if pmeta is None or not hasattr(pmeta, "shape"):
            return False
        if symint_safe_len(meta.shape) != 2 or symint_safe_len(pmeta.shape) != 2:
            return False
        return symint_safe_eq(meta.shape[0], pmeta.shape[0]) and symint_safe_eq(meta.shape[1], pmeta.shape[1])

    @staticmethod
    def _is_row_preserving_view(node: torch.fx.Node) -> bool:
        """A reshape that only regroups the leading dimensions, ``[M, N] <-> [B, S, N]``: the chain
        value keeps its rows and columns, so the kernel (which works on the flattened ``[M, N]``)
        does not see it.  This is what ``nn.Linear`` puts around ``addmm`` for 3-D activations; the
        reference stops the chain there (fuseml/passes/fusion_pass.py:244-257, 537-579)."""
        if node.target not in RESHAPE_OPS or not node.args or not isinstance(node.args[0], torch.fx.Node):
            return False
        shape, pshape = _node_shape(node), _node_shape(node.args[0])
        if shape is None or pshape is None:
            return False
        if (symint_safe_len(shape) or 0) < 2 or (symint_safe_len(pshape) or 0) < 2:
            return False
        return symint_safe_eq(shape[-1], pshape[-1])

    @staticmethod
    def _fetch_attr(gm: torch.fx.GraphModule, target: str):
        obj: Any = gm
        for atom in target.split("."):
            obj = getattr(obj, atom)
        return obj

    def _resolve_get_attr_bindings(self, group: FusionGroup) -> None:
        """``group.param_bindings[target] = live tensor`` for get_attr inputs (also one hop
        behind an input, e.g. ``get_attr -> t -> addmm``)."""
        def bind(n: Any) -> None:
            if getattr(n, "op", None) == "get_attr" and n.target not in group.param_bindings:
                try:
                    group.param_bindings[n.target] = self._fetch_attr(self.graph_module, n.target)
                except AttributeError:
                    logger.warning("Could not resolve get_attr target %r on graph module.", n.target)

        for inp in group.inputs:
            bind(inp)
        for inp in group.inputs:
            for arg in getattr(inp, "args", ()) or ():
                if isinstance(arg, torch.fx.Node):
                    bind(arg)

    # ------------------------------------------------------------------ surgery
    def _apply_surgery(self, groups: list[FusionGroup]) -> None:
        graph = self.graph_module.graph
        order = {n: i for i, n in enumerate(graph.nodes)}
        for group in groups:
            self._validate_insertion_topology(group, order)
            with graph.inserting_after(group.output_node):
                fused = graph.call_function(fuseml_fused_kernel_placeholder, args=tuple(group.inputs))
            if "tensor_meta" in group.output_node.meta:
                fused.meta["tensor_meta"] = group.output_node.meta["tensor_meta"]
            if "val" in group.output_node.meta:
                fused.meta["val"] = group.output_node.meta["val"]
            fused.meta["fusion_group"] = group
            fused.meta["fused_op_names"] = [n.name for n in group.all_nodes]
            fused.meta["param_bindings"] = group.param_bindings
            logger.debug("Inserted fused placeholder %s for group %s", fused.name, group)

            replaced = self._rewire_consumers(graph, group, fused)

            # later groups may list a node we just replaced among their inputs
            for other in groups:
                if other is not group:
                    other.inputs[:] = [replaced.get(i, i) for i in other.inputs]
            # the graph's output node must not keep pointing at a dead original
            out = next((n for n in graph.nodes if n.op == "output"), None)
            if out is not None:
                def patch(a):
                    if isinstance(a, torch.fx.Node):
                        return replaced.get(a, a)
                    if isinstance(a, (tuple, list)):
                        return type(a)(patch(x) for x in a)
                    return a
                new_args = tuple(patch(a) for a in out.args)
                if new_args != out.args:
                    out.args = new_args

        # sweep orphans (weight get_attrs, aten.t views, the absorbed nodes), keep the placeholders
        for n in reversed(list(graph.nodes)):
            if not n.users and n.op in ("get_attr", "call_function") \
                    and not (n.op == "call_function" and n.target is fuseml_fused_kernel_placeholder):
                graph.erase_node(n)
        graph.eliminate_dead_code()
        self._validate_acyclicity(graph)
        graph.lint()
        self.graph_module.recompile()
        logger.info("Graph surgery complete — %d group(s) replaced with placeholder kernels.", len(groups))

    def _rewire_consumers(self, graph: torch.fx.Graph, group: FusionGroup, fused: torch.fx.Node) -> dict:
        """Point every outside reader at the fused node (or at ``getitem(fused, i)`` when the
        kernel has several outputs: primary, escape stores, extra reductions — in that order).
        Returns {original node: replacement}."""
        extras = list(group.intermediate_outputs) + list(group.extra_outputs)
        if not extras:
            group.output_node.replace_all_uses_with(fused, propagate_meta=False)
            return {group.output_node: fused}

        members = set(group.all_nodes)
        replaced: dict = {}
        anchor = fused
        for idx, original in enumerate([group.output_node, *extras]):
            with graph.inserting_after(anchor):
                item = graph.call_function(_operator.getitem, args=(fused, idx))
            for key in ("tensor_meta", "val"):
                if key in original.meta:
                    item.meta[key] = original.meta[key]
            replaced[original] = item
            anchor = item
        for original, item in replaced.items():
            for user in list(original.users):
                if user not in members and user is not item:
                    user.replace_input_with(original, item)
        fused.meta["num_outputs"] = 1 + len(extras)
        fused.meta["intermediate_output_names"] = [n.name for n in group.intermediate_outputs]
        fused.meta["extra_output_names"] = [n.name for n in group.extra_outputs]
        return replaced

    @staticmethod
    def _validate_insertion_topology(group: FusionGroup, topo_index: dict | None = None) -> None:
        """Every input must be defined before the insertion point (right after ``output_node``)."""
        if topo_index is None:
            topo_index = {n: i for i, n in enumerate(group.base_node.graph.nodes)}
        at = topo_index.get(group.output_node)
        if at is None:
            return
        for inp in group.inputs:
            pos = topo_index.get(inp)
            if pos is not None and pos > at:
                raise RuntimeError(
                    f"SSA violation: input '{inp.name}' (topo position {pos}) appears after output_node "
                    f"'{group.output_node.name}' (topo position {at}); inserting the fused call there would "
                    f"create a cyclic dependency.")

    @staticmethod
    def _validate_acyclicity(graph: torch.fx.Graph) -> None:
        """Iterative three-colour DFS over def->use edges; a grey successor is a back edge."""
        WHITE, GREY, BLACK = 0, 1, 2
        colour = {n: WHITE for n in graph.nodes}
        for root in graph.nodes:
            if colour[root] != WHITE:
                continue
            stack = [(root, iter(root.users))]
            colour[root] = GREY
            while stack:
                node, it = stack[-1]
                advanced = False
                for user in it:
                    c = colour.get(user, WHITE)
                    if c == GREY:
                        raise RuntimeError(f"Cycle detected after graph surgery: '{node.name}' → '{user.name}' "
                                           f"forms a back edge.")
                    if c == WHITE:
                        colour[user] = GREY
                        stack.append((user, iter(user.users)))
                        advanced = True
                        break
                if not advanced:
                    colour[node] = BLACK
                    stack.pop()

    # ------------------------------------------------------------------ entry point
    def run(self, example_inputs: tuple | None = None) -> torch.fx.GraphModule:
        """Shape propagation (unless FakeTensor metadata is already there), discovery, the
        graph-cut safeguard, surgery.  Returns the same, modified, graph module."""
        if example_inputs is not None:
            have_fake = any(n.meta.get("val") is not None for n in self.graph_module.graph.nodes
                            if n.op == "call_function")
            if have_fake:
                self._tensor_meta_from_val()
            else:
                ShapeProp(self.graph_module).propagate(*example_inputs)
        groups: list[FusionGroup] = []
        for group in self._find_fusion_groups():
            if group.extra_outputs or not group.store_output:
                groups.append(group)        # extension groups are built from supported ops only
                continue
            for seg in split_fusion_group(group):
                if seg.kind == "fused" and seg.group is not None:
                    groups.append(seg.group)
                else:
                    logger.info("Native fallback for %d node(s): %s", len(seg.nodes), [n.name for n in seg.nodes])
        if groups:
            logger.info("Found %d fusion group(s) — applying graph surgery.", len(groups))
            self._apply_surgery(groups)
        else:
            logger.info("No fusible sequences detected — graph unchanged.")
        return self.graph_module

    def _tensor_meta_from_val(self) -> None:
        """Dynamo / AOT graphs carry FakeTensors in ``meta['val']``; derive ``tensor_meta`` from
        them so that the rest of the pass reads one kind of metadata."""
        from torch.fx.passes.shape_prop import _extract_tensor_metadata as extract

        for n in self.graph_module.graph.nodes:
            val = n.meta.get("val")
            if "tensor_meta" not in n.meta and isinstance(val, torch.Tensor):
                try:
                    n.meta["tensor_meta"] = extract(val)
                except Exception:  # symbolic shapes etc.: leave it absent
                    pass
