"""Front end on CPU: discovery against the reference's own groups (tests/golden/structure.json),
the opt-in extensions, lowering to kernel specifications, cache / launcher host logic, and —
when the reference checkout is present — the reference's own pass-level tests run against
this package through the ``fuseml`` alias."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch
from torch.fx.experimental.proxy_tensor import make_fx
from torch.fx.passes.shape_prop import ShapeProp

import fuseml_b200 as F
from fuseml_b200 import _native as N
from fuseml_b200.codegen.kernel_generator import Sm100KernelGenerator, UnsupportedChainError
from oracle import configs

ROOT = Path(__file__).resolve().parent.parent
# FUSEML_REFERENCE_DIR names a checkout of the reference; its own pass-level tests are then run
# against this package (skipped when the variable is unset)
REFERENCE = Path(os.environ["FUSEML_REFERENCE_DIR"]) if os.environ.get("FUSEML_REFERENCE_DIR") else None
CFGS = list(configs.MAKERS)


def _trace(case):
    with torch.no_grad():
        gm = make_fx(lambda *a: case.module(*a))(*case.args)
    ShapeProp(gm).propagate(*case.args)
    return gm


def _specs(gm):
    gen = Sm100KernelGenerator()
    out = []
    for n in gm.graph.nodes:
        g = n.meta.get("fusion_group")
        if g is not None:
            out.append((g, gen.build_spec(g)))
    return out


@pytest.mark.parametrize("name", CFGS)
def test_default_discovery_equals_reference(golden_dir, name):
    golden = json.loads((golden_dir / "structure.json").read_text())[name]
    case = configs.make(name, small=(name != "cfg1"))
    groups = F.FuseMLFusionPass(_trace(case))._find_fusion_groups()
    assert [list(g.op_signature) for g in groups] == [g["op_signature"] for g in golden]
    assert [len(g.inputs) for g in groups] == [g["n_inputs"] for g in golden]
    assert [list(g.output_metadata.get("shape", ())) for g in groups] == [g["output_shape"] for g in golden]
    assert [len(g.intermediate_outputs) for g in groups] == [g["intermediate_outputs"] for g in golden]
    for g, ref in zip(groups, golden):
        assert [n.op for n in g.inputs] == ref["input_kinds"]


def test_extensions_fuse_what_the_reference_cannot():
    opts = dict(dag_epilogue=True, multi_reduction=True, global_reductions=True)
    # cfg2: addmm has two users -> one diamond group, evaluated with the second register
    gm = _trace(configs.make("cfg2", small=True))
    F.FuseMLFusionPass(gm, **opts).run()
    (g, spec), = _specs(gm)
    assert list(g.op_signature) == ["aten.addmm.default", "aten.gelu.default", "aten.sigmoid.default",
                                    "aten.mul.Tensor", "aten.add.Tensor"]
    assert [N.OP_NAMES[s.opcode] for s in spec.steps] == ["add_t", "save", "gelu_erf", "swap", "sigmoid",
                                                          "mul_saved", "add_t"]
    assert spec.uses_second_register and spec.store_output and not spec.reductions
    # cfg3: both reductions in one kernel, the matrix is never stored
    gm = _trace(configs.make("cfg3", small=True))
    F.FuseMLFusionPass(gm, **opts).run()
    (g, spec), = _specs(gm)
    assert [(r.op, r.axis) for r in spec.reductions] == [("max", 1), ("mean", 1)]
    assert not spec.store_output and len(g.extra_outputs) == 1
    # cfg5: last block stores its output and also yields the global sum and amax
    gm = _trace(configs.make("cfg5", small=True))
    F.FuseMLFusionPass(gm, **opts).run()
    specs = _specs(gm)
    assert len(specs) == 8
    last = specs[-1][1]
    assert last.store_output and [(r.op, r.axis) for r in last.reductions] == [("sum", 2), ("max", 2)]
    # the graph now returns getitem(fused, 0..2)
    out = next(n for n in gm.graph.nodes if n.op == "output")
    assert all(a.target.__name__ == "getitem" for a in out.args[0])


def test_lowering_of_addmm_scaling_and_scalars():
    def f(bias, x, w, r):
        h = torch.addmm(bias, x, w, beta=0.5, alpha=2.0)
        h = torch.relu(h) * 3.0
        h = h + 1.5
        return torch.add(h, r, alpha=2.0)
    args = (torch.randn(8), torch.randn(4, 16), torch.randn(16, 8), torch.randn(4, 8))
    gm = make_fx(f)(*args)
    ShapeProp(gm).propagate(*args)
    F.FuseMLFusionPass(gm).run()
    (_, spec), = _specs(gm)
    names = [(N.OP_NAMES[s.opcode], round(s.imm, 6)) for s in spec.steps]
    assert names == [("mul_imm", 4.0), ("add_t", 0.0), ("mul_imm", 0.5), ("relu", 0.0), ("mul_imm", 3.0),
                     ("add_imm", 1.5), ("mul_imm", 0.5), ("add_t", 0.0), ("mul_imm", 2.0)]
    assert (spec.left_index, spec.right_index) == (1, 2)


def test_lowering_rejects_what_the_vm_cannot_express():
    def f(a, b):
        return torch.mm(a, b).amax(-1, keepdim=True)
    args = (torch.randn(4, 8), torch.randn(8, 4))
    gm = make_fx(f)(*args)
    ShapeProp(gm).propagate(*args)
    assert F.FuseMLFusionPass(gm)._find_fusion_groups() == []      # keepdim=True is never absorbed
    # gelu(approximate='tanh') lowers to its own opcode instead of silently using erf
    def g(a, b):
        return torch.nn.functional.gelu(torch.mm(a, b), approximate="tanh")
    gm = make_fx(g)(*args)
    ShapeProp(gm).propagate(*args)
    F.FuseMLFusionPass(gm).run()
    (_, spec), = _specs(gm)
    assert [N.OP_NAMES[s.opcode] for s in spec.steps] == ["gelu_tanh"]


def test_compiler_on_cpu_hands_back_eager_like_the_reference(golden_dir):
    """On CPU tensors nothing is lowered (no CPU implementation of the fused path exists)."""
    import numpy as np

    case = configs.make("cfg1")
    comp = F.FuseMLCompiler()
    out = torch.compile(case.module, backend=comp)(*case.args)
    assert comp.fusion_applied is False and comp.fusion_strategy == "none" and comp.launchers == []
    np.testing.assert_allclose(out.detach().numpy(), np.load(golden_dir / "numeric_cfg1.npz")["y"], rtol=1e-5, atol=1e-5)
    torch._dynamo.reset()


def test_launcher_host_contract():
    from fuseml_b200.codegen.kernel_generator import KernelSpec, TensorDescriptor

    spec = KernelSpec(left_index=1, right_index=2, n_inputs=3)
    d = [TensorDescriptor("bias", (8,), (1,), torch.bfloat16), TensorDescriptor("x", (4, 16), (16, 1), torch.bfloat16),
         TensorDescriptor("w", (16, 8), (1, 16), torch.bfloat16)]
    out = TensorDescriptor("out", (4, 8), (8, 1), torch.bfloat16)
    L = F.KernelLauncher(spec, d, out, [], "x", "w")
    assert L.__name__ == "fuseml_fused_kernel"
    with pytest.raises(ValueError, match="Expected 3 input"):
        L(torch.zeros(1))
    with pytest.raises(ValueError, match="left_name"):
        F.KernelLauncher(spec, d, out, [], "nope", "w")
    with pytest.raises(ValueError, match="disagree"):
        F.KernelLauncher(spec, d, out, [], "w", "x")
    with pytest.raises(RuntimeError):      # CPU tensors: no fallback, a loud error
        L(torch.zeros(8, dtype=torch.bfloat16), torch.zeros(4, 16, dtype=torch.bfloat16),
          torch.zeros(8, 16, dtype=torch.bfloat16).t())


def test_launch_params_and_tile_chooser():
    lp = F.compute_launch_params(8192, 16384, 4096, torch.bfloat16)
    assert (lp.block_m, lp.block_n, lp.block_k, lp.num_stages) == (128, 256, 64, 6)
    assert F.compute_sram_bytes(128, 256, 64, 2, 4) == 4 * (16384 + 32768)
    tuner = F.SRAMAutotuner()
    cfg = tuner.get_best_config(8192, 16384, 4096, torch.bfloat16)
    assert cfg.block_m == 128 and cfg.block_n == 256 and cfg.sram_bytes <= tuner.sram_budget and cfg.tmem_cols == 512
    assert tuner.get_best_config(8192, 16384, 4096, torch.bfloat16) is cfg and tuner.cache_size == 1
    small = F.SRAMAutotuner(sram_budget=100 * 1024)
    assert small.get_best_config(8192, 16384, 4096).sram_bytes <= 100 * 1024
    assert all(c.sram_bytes <= 64 * 1024 for c in F.generate_sram_safe_configs(torch.bfloat16, 64 * 1024))


def test_library_epilogue_patterns_are_programs_now():
    gm = _trace(configs.make("cfg4", small=True))
    triggers = [n for n in gm.graph.nodes if F.is_trigger(n)]
    pats = [F.match_cublas_epilogue(t) for t in triggers]
    assert [p.epilogue_type for p in pats] == ["GELU_BIAS", "BIAS_RESIDUAL"]
    assert pats[0].program() == ("add_t", "gelu_erf") and pats[1].program() == ("add_t", "add_t")
    assert F.cublas_epilogue_available() is False


def test_fuseml_alias_package():
    import fuseml
    from fuseml.passes.fusion_pass import FuseMLFusionPass as P1
    from fuseml.codegen.kernel_cache import KernelCache as C1

    assert P1 is F.FuseMLFusionPass and C1 is F.KernelCache and fuseml.FuseMLCompiler is F.FuseMLCompiler


REF_TESTS = ["test_registry", "test_fusion_group", "test_pattern_matching", "test_graph_surgery",
             "test_get_attr_resolution", "test_shape_propagation", "test_aot_topology", "test_graph_cut",
             "test_mutation_safety", "test_control_flow_validation", "test_end_to_end", "test_kernel_cache"]


@pytest.mark.skipif(REFERENCE is None or not (REFERENCE / "tests").is_dir(),
                    reason="FUSEML_REFERENCE_DIR does not name a reference checkout")
def test_reference_pass_level_suite_passes_against_this_package(tmp_path):
    """Run the reference's own structural tests, unmodified and in place, with ``fuseml``
    resolving to this package."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), PYTHONDONTWRITEBYTECODE="1")
    files = [str(REFERENCE / "tests" / f"{t}.py") for t in REF_TESTS]
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", f"--rootdir={tmp_path}", *files],
                          cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
    tail = proc.stdout.strip().splitlines()[-1] if proc.stdout.strip() else proc.stderr[-500:]
    assert proc.returncode == 0, proc.stdout[-3000:]
    assert "passed" in tail and "failed" not in tail


def test_batched_activations_fuse_through_the_flatten_views():
    """[B, S, D] activations: nn.Linear wraps addmm in view(x, [B*S, D]) ... view(out, [B, S, N]).
    The chain continues through those row-regrouping views (the reference stops there:
    fuseml/passes/fusion_pass.py:244-257), the 3-D residual lines up with the flattened tile,
    and a reduction over the last dimension is a per-row reduction."""
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = torch.nn.Linear(16, 32)
            self.fc2 = torch.nn.Linear(32, 16)

        def forward(self, x):
            y = self.fc2(torch.nn.functional.gelu(self.fc1(x))) + x
            return y, y.amax(-1)

    from torch._functorch.aot_autograd import aot_module_simplified
    from functorch.compile import make_boxed_func
    seen = {}

    def grab(gm, inputs):
        seen["gm"] = gm
        return make_boxed_func(gm.forward)

    block, x = Block().eval(), torch.randn(2, 3, 16)
    with torch.no_grad():
        aot_module_simplified(block, (x,), fw_compiler=grab, inference_compiler=grab)(x)
    gm = seen["gm"]
    fpass = F.FuseMLFusionPass(gm, dag_epilogue=True, multi_reduction=True, global_reductions=True)
    fpass._tensor_meta_from_val()
    groups = fpass._find_fusion_groups()
    sigs = [[s for s in g.op_signature if "view" not in s] for g in groups]
    assert sigs == [["aten.addmm.default", "aten.gelu.default"],
                    ["aten.addmm.default", "aten.add.Tensor", "aten.amax.default"]]
    gen = Sm100KernelGenerator()
    specs = [gen.build_spec(g) for g in groups]
    assert [[N.OP_NAMES[s.opcode] for s in sp.steps] for sp in specs] == [["add_t", "gelu_erf"], ["add_t", "add_t"]]
    assert [(r.axis, r.op) for r in specs[1].reductions] == [(1, "max")] and specs[1].store_output
    # A of the first group is x itself (3-D): the launcher flattens it; the residual of the second is x again
    from fuseml_b200.passes.fusion_pass import _node_shape
    shapes = [[tuple(_node_shape(n)) for n in g.inputs] for g in groups]
    assert (2, 3, 16) in shapes[0] and (2, 3, 16) in shapes[1]
    # a reduction over the sequence dimension is not one the kernel runs: it stays outside the group
    def f(x, w):
        return torch.mm(x.view(6, 16), w).view(2, 3, 8).relu().sum(1)
    args = (torch.randn(2, 3, 16), torch.randn(16, 8))
    gm2 = make_fx(f)(*args)
    ShapeProp(gm2).propagate(*args)
    (g2,) = F.FuseMLFusionPass(gm2)._find_fusion_groups()
    assert [s for s in g2.op_signature if "view" not in s] == ["aten.mm.default", "aten.relu.default"]


def test_row_grouping_helpers():
    """How reduction dims and outside operands line up with the flattened [rows, N] tile."""
    from fuseml_b200.passes.topology import classify_epilogue_operand as c, reduction_axis_code as r

    assert [r([-1], 3), r([2], 3), r(-1, 2), r([1], 2)] == ["n"] * 4
    assert r([0], 2) == "m" and r([0], 3) is None and r([1], 3) is None
    assert [r([], 3), r(None, 2), r([0, 1], 2), r([0, 1, 2], 3)] == ["all"] * 4
    rows, n = 4 * 512, 256
    assert c((4, 512, 256), rows, n) == "full" and c((2048, 256), rows, n) == "full"
    assert c((256,), rows, n) == "row" and c((1, 1, 256), rows, n) == "row" and c((1, 256), rows, n) == "row"
    assert c((4, 512, 1), rows, n) == "col" and c((2048, 1), rows, n) == "col" and c((2048,), rows, n) == "col"
    assert c((), rows, n) == "scalar" and c((1, 1), rows, n) == "scalar"
    assert c((512, 256), rows, n) is None            # broadcast over the batch only: not a [rows, N] pattern
    assert c((4, 1, 256), rows, n) is None
    assert c((256,), 256, 256) == "row"              # the reference's 1-D rule: length N runs along N first


def test_plan_cache_round_trip_and_candidates(tmp_path):
    """Measured plans persist as JSON: written atomically, merged on write, malformed entries
    ignored; the candidate list holds the router's plan first and only neighbours that differ."""
    from fuseml_b200.codegen import plan_cache as pc

    path = tmp_path / "sub" / "plans.json"
    cache = pc.PlanCache(path)
    assert len(cache) == 0 and cache.get("missing") is None and cache.misses == 1
    plan = N.Plan()
    plan.tile_m, plan.tile_n, plan.cluster, plan.grid, plan.group_m, plan.split_k = 128, 224, 2, 148, 4, 1
    key = pc.plan_key("NVIDIA B200", "abc123", 1024, 16384, 4096, N.BF16, N.BF16, "k", "sig")
    cache.put(key, pc.entry_of(plan, 61.25, 5))
    other = pc.PlanCache(path)                       # a second process
    other.put("other-key", pc.entry_of(plan, 1.0, 1))
    again = pc.PlanCache(path)
    assert len(again) == 2 and again.get(key)["tile_n"] == 224 and again.get(key)["us"] == 61.25
    fresh = N.Plan()
    assert pc.apply_entry(fresh, again.get(key)) and (fresh.tile_n, fresh.cluster, fresh.grid) == (224, 2, 148)
    for bad in ({}, {"tile_n": 48, "cluster": 2, "grid": 1, "group_m": 1, "split_k": 1},
                {"tile_n": 256, "cluster": 3, "grid": 1, "group_m": 1, "split_k": 1}):
        untouched = N.Plan()
        assert not pc.apply_entry(untouched, bad) and untouched.tile_n == 0
    path.write_text("not json")
    assert len(pc.PlanCache(path)) == 0              # unreadable file: ignored, not fatal
    base = N.Plan()
    base.tile_m, base.tile_n, base.cluster, base.grid, base.group_m, base.split_k = 128, 256, 2, 148, 4, 1
    # 1024 rows x 16384 columns: 256 tiles are 3.46 waves of 74 pairs; 224-wide tiles fill four waves
    shard = pc.candidate_plans(base, 1024, 16384)
    assert shard[0].tile_n == 256 and 224 in [c.tile_n for c in shard]
    # its last wave holds 34 tiles (at most half of the pairs): the K-split last wave is tried too,
    # and the choice survives the file (the per-call expansion bit does not)
    toggled = [c for c in shard if c.flags & N.PLAN_STREAM_K]
    assert len(toggled) == 1 and toggled[0].tile_n == 256
    toggled[0].flags |= N.PLAN_B_EXPANSION_VALID
    entry = pc.entry_of(toggled[0], 1.0, 1)
    restored = N.Plan()
    assert entry["stream_k"] == 1 and pc.apply_entry(restored, entry) and restored.flags == N.PLAN_STREAM_K
    entry.pop("stream_k")
    assert pc.apply_entry(restored, entry) and restored.flags == N.PLAN_STREAM_K      # older entry: flag untouched
    # 8192 rows: 27.7 waves, nothing to gain from narrower tiles; the group size varies, and the
    # ragged last wave (50 tiles) may be shared by K ranges
    full = pc.candidate_plans(base, 8192, 16384)
    assert {c.tile_n for c in full} == {256} and len(full) == 5
    assert sum(1 for c in full if c.flags & N.PLAN_GROUP_N) == 1          # the walk the other way round is tried too
    assert [c.grid for c in full if c.flags & N.PLAN_STREAM_K] == [148]


def test_backward_graph_lowers_to_four_fused_gemms():
    """The backward graph AOT autograd builds for ``l2(gelu(l1(x))) + x`` (written out with ATen ops):
    with the backward extensions on, the data-gradient GEMM absorbs ``gelu_backward`` (the saved
    pre-activation becomes an epilogue operand), the other one absorbs the residual's gradient, and
    the two weight-gradient GEMMs (transposed-view left operand) are bare triggers."""
    aten = torch.ops.aten

    def bw(x, t, addmm, gelu, t_1, tang):
        mm = aten.mm(tang, aten.t(t_1))
        mm_1 = aten.mm(aten.t(tang), gelu)
        gb = aten.gelu_backward(mm, addmm)
        mm_2 = aten.mm(gb, aten.t(t))
        mm_3 = aten.mm(aten.t(gb), x)
        return aten.t(mm_3), aten.sum.dim_IntList(gb, [0], True), aten.add.Tensor(tang, mm_2), aten.t(mm_1)

    M, D, I = 32, 64, 256
    args = (torch.randn(M, D), torch.randn(I, D).t(), torch.randn(M, I), torch.randn(M, I), torch.randn(D, I).t(),
            torch.randn(M, D))
    gm = make_fx(bw)(*args)
    ShapeProp(gm).propagate(*args)
    assert F.FuseMLFusionPass(gm)._find_fusion_groups()[0].op_signature == ("aten.mm.default", "aten.add.Tensor")
    F.FuseMLFusionPass(gm, bare_trigger=True, backward_ops=True).run()
    lowered = sorted(([N.OP_NAMES[s.opcode] for s in spec.steps], len(g.inputs)) for g, spec in _specs(gm))
    assert lowered == [([], 2), ([], 2), (["add_t"], 3), (["gelu_erf_bwd_t"], 3)]
    # gelu_backward of the tanh form has no epilogue op: the chain is declined, not mis-lowered
    def bw_tanh(tang, w, pre):
        return aten.gelu_backward(aten.mm(tang, w), pre, approximate="tanh")
    args = (torch.randn(8, 16), torch.randn(16, 8), torch.randn(8, 8))
    gm = make_fx(bw_tanh)(*args)
    ShapeProp(gm).propagate(*args)
    F.FuseMLFusionPass(gm, backward_ops=True).run()
    g = next(n.meta["fusion_group"] for n in gm.graph.nodes if n.meta.get("fusion_group") is not None)
    with pytest.raises(UnsupportedChainError):
        Sm100KernelGenerator().build_spec(g)
