"""End to end on a GPU: ``torch.compile(module, backend=FuseMLCompiler())`` — the call a user of
the reference makes — on the five configurations, against the reference's own outputs
(tests/golden) and the stage oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import configs

pytestmark = pytest.mark.gpu

BF16_TOL = dict(rtol=1.6e-2, atol=1e-2)
F32_TOL = dict(rtol=1e-3, atol=1e-3)
EXPECTED_KERNELS = {"cfg1": 2, "cfg2": 1, "cfg3": 1, "cfg4": 2, "cfg5": 8}


def _cuda_case(name):
    case = configs.make(name, small=(name != "cfg1"))
    td = {"bf16": torch.bfloat16, "f32": torch.float32}[case.dtype]
    module = case.module.to(device="cuda", dtype=td)
    args = tuple(a.to(device="cuda", dtype=td) for a in case.args)
    return case, module, args


@pytest.mark.parametrize("name", list(configs.MAKERS))
def test_compiled_module_matches_reference_fixture(native_lib, golden_dir, name):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch._dynamo.reset()
    case, module, args = _cuda_case(name)
    comp = F.FuseMLCompiler()
    compiled = torch.compile(module, backend=comp)
    with torch.no_grad():
        out = compiled(*args)
        out2 = compiled(*args)          # second call: prepared-launch fast path
    torch.cuda.synchronize()
    assert F.device_status() == 0
    assert comp.fusion_applied and comp.fusion_strategy == "sm100", comp.declined
    assert sum(L.launch_count for L in set(comp.launchers)) == 2 * EXPECTED_KERNELS[name]
    if not isinstance(out, (tuple, list)):
        out, out2 = (out,), (out2,)
    golden = np.load(golden_dir / f"numeric_{name}.npz")
    oracle = configs.run_stages_oracle(case)
    for k, got, again in zip(case.outputs, out, out2):
        g = got.float().cpu().numpy()
        assert np.array_equal(g, again.float().cpu().numpy()), "launches are deterministic"
        ref = golden[k]
        if ref.ndim <= 1:
            # reductions leave the graph in the dtype the graph asked for (bf16 here): compare
            # with the tolerance of that dtype against the reference, and tightly against the oracle
            tol = BF16_TOL if case.dtype == "bf16" else F32_TOL
            np.testing.assert_allclose(g, ref, err_msg=f"{name}:{k}", **tol)
            np.testing.assert_allclose(g, oracle[k], err_msg=f"{name}:{k} vs oracle", **tol)
        else:
            np.testing.assert_allclose(g, ref, err_msg=f"{name}:{k}", **(F32_TOL if case.dtype == "f32" else BF16_TOL))
    torch._dynamo.reset()


def test_unfusable_layout_is_left_to_eager_not_failed(native_lib):
    """A chain whose rows are not multiples of 16 bytes was never matched: it runs as ATen ops."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch._dynamo.reset()
    lin = torch.nn.Linear(100, 36).to("cuda", torch.bfloat16)      # K = 100 -> 200-byte rows
    x = torch.randn(16, 100, device="cuda", dtype=torch.bfloat16)
    comp = F.FuseMLCompiler()
    f = torch.compile(lambda t: torch.relu(lin(t)), backend=comp)
    with torch.no_grad():
        y = f(x)
        ref = torch.relu(lin(x))
    assert not comp.fusion_applied and comp.declined and "16 bytes" in comp.declined[0][1]
    assert torch.equal(y, ref)
    torch._dynamo.reset()


def test_fp32_reductions_keep_fp32(native_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch._dynamo.reset()
    a = torch.randn(300, 128, device="cuda")
    b = torch.randn(128, 520, device="cuda") / 11

    def f(a, b):
        c = torch.sigmoid(a @ b)
        return c.sum(dim=0), c.amax(dim=0)
    comp = F.FuseMLCompiler()
    with torch.no_grad():
        s, m = torch.compile(f, backend=comp)(a, b)
        rs, rm = f(a.double(), b.double())
    assert comp.fusion_applied and s.dtype == torch.float32 and s.shape == (520,)
    assert ((s.double() - rs).abs().max() / rs.abs().max()).item() < 1e-3
    assert ((m.double() - rm).abs().max()).item() < 1e-3
    torch._dynamo.reset()


def test_host_streamed_runtime_matches_direct_call(native_lib):
    """Row chunks through three CUDA streams give the same bytes as one direct call."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F
    from fuseml_b200.runtime import HostStreamedModule

    torch._dynamo.reset()
    case, module, args = _cuda_case("cfg4")
    rows, d = 1024, case.sizes["D"]
    compiled = torch.compile(module, backend=F.FuseMLCompiler())
    g = torch.Generator().manual_seed(7)
    x_host = torch.randn(rows, d, generator=g).to(torch.bfloat16).pin_memory()
    y_host = torch.zeros(rows, d, dtype=torch.bfloat16).pin_memory()
    runner = HostStreamedModule(compiled, rows_per_chunk=256)
    for _ in range(3):                       # batches pipeline into each other
        runner.submit(x_host, y_host)
    runner.synchronize()
    with torch.no_grad():
        ref = compiled(x_host.cuda()).cpu()
    assert torch.equal(y_host, ref)
    assert runner.h2d_bytes == 3 * rows * d * 2 and runner.d2h_bytes == 3 * rows * d * 2
    with pytest.raises(ValueError):
        runner.submit(torch.zeros(4, d, dtype=torch.bfloat16), y_host)     # not pinned
    # a per-batch metric next to the row output: copied whole when the batch is one chunk,
    # refused when the batch is cut (it would be the metric of the last chunk only)
    def with_metric(x):
        y = compiled(x)
        return y, y.float().sum().reshape(1)
    s_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    whole = HostStreamedModule(with_metric, rows_per_chunk=rows)
    whole.submit(x_host, (y_host, s_host))
    whole.synchronize()
    assert torch.equal(y_host, ref)
    np.testing.assert_allclose(float(s_host), float(ref.float().sum()), rtol=1e-5)
    with pytest.raises(ValueError):
        HostStreamedModule(with_metric, rows_per_chunk=256).submit(x_host, (y_host, s_host))
    torch.cuda.synchronize()
    torch._dynamo.reset()


def test_batched_activations_run_fused_and_match_the_flattened_block(native_lib):
    """The residual MLP block on [B, S, D] activations (what an unmodified Transformer layer
    feeds it): two fused kernels, 3-D outputs, same numbers as the block on the flattened
    [B*S, D] input (which the 2-D parity tests pin against the reference) and within the bf16
    tolerance of the fp32 oracle chain; the row maximum comes back as [B, S]."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F
    from oracle import chain

    class Block(torch.nn.Module):
        def __init__(self, d, i):
            super().__init__()
            self.fc1 = torch.nn.Linear(d, i)
            self.fc2 = torch.nn.Linear(i, d)

        def forward(self, x):
            y = self.fc2(torch.nn.functional.gelu(self.fc1(x))) + x
            return y, y.amax(-1)

    torch._dynamo.reset()
    torch.manual_seed(0)
    B, S, D, I = 3, 200, 256, 512           # 600 rows: ragged against the 128/256-row tiles
    block = Block(D, I).to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randn(B, S, D, device="cuda", dtype=torch.bfloat16)
    comp = F.FuseMLCompiler()
    compiled = torch.compile(block, backend=comp)
    with torch.no_grad():
        y, ymax = compiled(x)
        y2, _ = compiled(x.view(B * S, D).clone().view(B, S, D))
    torch.cuda.synchronize()
    assert F.device_status() == 0
    assert comp.fusion_applied and len(set(comp.launchers)) == 2, comp.declined
    assert sum(L.launch_count for L in set(comp.launchers)) == 4
    assert y.shape == (B, S, D) and ymax.shape == (B, S)
    assert torch.equal(y, y2)
    # oracle: the same chain on the flattened rows, fp32 arithmetic on the bf16-rounded values
    f = lambda t: t.detach().float().cpu().numpy()
    xs = f(x).reshape(B * S, D)
    h = chain.fused_chain(xs, f(block.fc1.weight).T, [("add", f(block.fc1.bias)), ("gelu",)], "bf16")["d"]
    want = chain.fused_chain(h, f(block.fc2.weight).T, [("add", f(block.fc2.bias)), ("add", xs)], "bf16")["d"]
    np.testing.assert_allclose(f(y).reshape(B * S, D), want, **BF16_TOL)
    np.testing.assert_allclose(f(ymax).reshape(-1), want.max(axis=1), **BF16_TOL)
    torch._dynamo.reset()


def test_misaligned_views_run_fused_on_an_aligned_copy(native_lib):
    """A column slice that starts in the middle of a 16-byte word cannot be read by TMA in place.
    The compile-time layout check sees shapes and strides only, so the launcher meets such a
    tensor at run time: it copies the operand into an aligned buffer and launches the fused
    kernel on the copy instead of raising out of the compiled graph."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch._dynamo.reset()
    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 384).to("cuda", torch.bfloat16)
    big = torch.randn(200, 264, device="cuda", dtype=torch.bfloat16)
    aligned, shifted = big[:, 8:264], big[:, 4:260]          # same shape and strides; 16- and 8-byte offsets
    comp = F.FuseMLCompiler()
    f = torch.compile(lambda t: torch.nn.functional.gelu(lin(t)), backend=comp)
    with torch.no_grad():
        y0 = f(aligned)
        y1 = f(shifted)
        ref0 = torch.nn.functional.gelu(lin(aligned).float())
        ref1 = torch.nn.functional.gelu(lin(shifted).float())
    torch.cuda.synchronize()
    assert F.device_status() == 0
    assert comp.fusion_applied and sum(L.launch_count for L in set(comp.launchers)) == 2
    np.testing.assert_allclose(y0.float().cpu().numpy(), ref0.cpu().numpy(), **BF16_TOL)
    np.testing.assert_allclose(y1.float().cpu().numpy(), ref1.cpu().numpy(), **BF16_TOL)
    torch._dynamo.reset()


def test_fp32_weight_expansion_is_reused_until_the_weight_changes(native_lib):
    """fp32 operands are expanded into the launcher's workspace before the MMA; the expansion of
    an unchanged weight is reused by the next launch, and redone after an in-place update."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch._dynamo.reset()
    torch.manual_seed(5)
    lin = torch.nn.Linear(96, 160).to("cuda")
    x = torch.randn(64, 96, device="cuda")
    comp = F.FuseMLCompiler()
    f = torch.compile(lambda t: torch.relu(lin(t)), backend=comp)
    with torch.no_grad():
        y0 = f(x)
        y1 = f(x)                                  # second launch: B's expansion reused
        assert torch.equal(y0, y1)
        lin.weight.mul_(-1.0)                      # in-place update bumps the version counter
        y2 = f(x)
        ref = torch.relu(lin(x))
    torch.cuda.synchronize()
    assert F.device_status() == 0
    np.testing.assert_allclose(y2.cpu().numpy(), ref.cpu().numpy(), **F32_TOL)
    assert not torch.equal(y2, y0)
    torch._dynamo.reset()


def test_autotuned_plan_is_persisted_and_reused(native_lib, tmp_path):
    """With autotuning on, the first call of a shape times the router's plan and its neighbours
    and writes the winner to the plan cache; a second compiler (a later process) pointed at the
    same file starts from that plan without measuring, and computes the same matrix."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch.manual_seed(7)
    lin = torch.nn.Linear(512, 2048).to("cuda", torch.bfloat16)
    x = torch.randn(1024, 512, device="cuda", dtype=torch.bfloat16)
    path = tmp_path / "plans.json"
    outs = []
    for autotune in (True, False):
        torch._dynamo.reset()
        comp = F.FuseMLCompiler(plan_cache=path, autotune=autotune)
        f = torch.compile(lambda t: torch.nn.functional.gelu(lin(t)), backend=comp)
        with torch.no_grad():
            outs.append(f(x))
        torch.cuda.synchronize()
        assert F.device_status() == 0
        (launcher,) = set(comp.launchers)
        if autotune:
            assert launcher.tuned_signatures == 1 and path.exists() and len(comp.plan_cache) == 1
        else:
            assert launcher.tuned_signatures == 0 and comp.plan_cache.hits == 1
    with torch.no_grad():
        ref = torch.nn.functional.gelu(lin(x).float())
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)
    assert torch.equal(outs[0], outs[1])
    torch._dynamo.reset()


def test_compiled_forward_replays_from_a_cuda_graph(native_lib):
    """The launch path allocates through torch only and never synchronises the host, so a compiled
    forward can be captured once and replayed (the reference's launcher was built towards the same
    use, fuseml/codegen/kernel_launcher.py:640-670): new input values written into the static
    input tensor show up in the replayed output."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F
    from fuseml_b200.runtime import GraphedCallable

    torch._dynamo.reset()
    case, module, args = _cuda_case("cfg4")
    comp = F.FuseMLCompiler()
    compiled = torch.compile(module, backend=comp)
    static_x = args[0].clone()
    graphed = GraphedCallable(compiled, static_x)
    before = sum(L.launch_count for L in set(comp.launchers))
    y0 = graphed().clone()
    new_x = torch.randn_like(static_x)
    static_x.copy_(new_x)
    y1 = graphed().clone()
    torch.cuda.synchronize()
    assert F.device_status() == 0
    assert sum(L.launch_count for L in set(comp.launchers)) == before, "replays do not pass through Python"
    with torch.no_grad():
        ref0, ref1 = compiled(args[0]), compiled(new_x)
    assert torch.equal(y0, ref0) and torch.equal(y1, ref1) and not torch.equal(y0, y1)
    torch._dynamo.reset()


def test_k_split_last_wave_through_the_compiler_and_a_cuda_graph(native_lib):
    """A Linear whose tile count leaves a third of a wave (2560 x 2560 outputs = 100 pair tiles on
    74 pairs, 128 K blocks): the router marks the plan FUSEML_PLAN_STREAM_K, the launcher sizes the
    workspace for the partial tiles and flags, and the launch (a memset of the flags + the
    kernel) is captured and replayed like any other."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F
    from fuseml_b200 import _native as N
    from fuseml_b200.runtime import GraphedCallable

    torch._dynamo.reset()
    torch.manual_seed(3)
    lin = torch.nn.Linear(8192, 2560).to(device="cuda", dtype=torch.bfloat16)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = lin

        def forward(self, x):
            return torch.nn.functional.gelu(self.lin(x))

    comp = F.FuseMLCompiler()
    compiled = torch.compile(Block(), backend=comp)
    x = torch.randn(2560, 8192, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        y = compiled(x)
        plans = [p.plan for L in set(comp.launchers) for p in L._prepared.values()]
        assert plans and all(p.flags & N.PLAN_STREAM_K and p.cluster == 2 and p.grid == 148 for p in plans)
        ref = torch.nn.functional.gelu(x.float() @ lin.weight.float().t() + lin.bias.float())
        np.testing.assert_allclose(y.float().cpu().numpy(), ref.cpu().numpy(), rtol=1.6e-2, atol=1e-2)
        static_x = x.clone()
        graphed = GraphedCallable(compiled, static_x)
        y0 = graphed().clone()
        static_x.copy_(-x)
        y1 = graphed().clone()
        torch.cuda.synchronize()
        assert F.device_status() == 0
        assert torch.equal(y0, y) and torch.equal(y1, compiled(-x)) and not torch.equal(y0, y1)
    torch._dynamo.reset()


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_training_step_runs_fused_forward_and_backward(native_lib, dtype):
    """Forward and backward of the residual MLP block through the compiler.  The forward graph of a
    training step keeps the pre-activation for the backward pass (an escape store of the first
    kernel); the backward graph becomes four fused launches: the data-gradient GEMM with
    gelu'(pre) as its epilogue, the data-gradient GEMM with the residual's gradient added, and
    the two weight-gradient GEMMs dY^T @ X, whose transposed left operand is read in place.
    Gradients are compared with fp32 autograd on the same (rounded) parameters."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    td = {"bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    torch._dynamo.reset()
    case = configs.make("cfg4", small=True)                   # 136 tokens, 128 -> 520 -> 128
    model = case.module.to(device="cuda", dtype=td)
    ref_model = configs.make("cfg4", small=True).module.to(device="cuda", dtype=torch.float32)
    with torch.no_grad():
        for p_ref, p in zip(ref_model.parameters(), model.parameters()):
            p_ref.copy_(p.float())
    x = case.args[0].to(device="cuda", dtype=td).requires_grad_(True)
    x_ref = x.detach().float().requires_grad_(True)
    w = torch.randn(x.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))

    comp = F.FuseMLCompiler()
    y = torch.compile(model, backend=comp)(x)
    (y.float() * w).sum().backward()
    y_ref = ref_model(x_ref)
    (y_ref * w).sum().backward()
    torch.cuda.synchronize()
    assert F.device_status() == 0
    assert comp.fusion_applied and len(comp.launchers) == 6 and len(comp.backward_launchers) == 4, comp.declined
    assert all(L.launch_count == 1 for L in comp.launchers)
    tol = dict(rtol=3e-2, atol=3e-2) if dtype == "bf16" else dict(rtol=2e-3, atol=2e-3)

    def close(got, ref, what):
        scale = float(ref.abs().max())
        np.testing.assert_allclose(got.float().cpu().numpy() / scale, ref.cpu().numpy() / scale, err_msg=what, **tol)

    close(y.detach(), y_ref.detach(), "y")
    close(x.grad, x_ref.grad, "dx")
    for (name, p), p_ref in zip(model.named_parameters(), ref_model.parameters()):
        close(p.grad, p_ref.grad, f"d{name}")
    torch._dynamo.reset()


def test_small_batch_mlp_runs_as_one_kernel_and_larger_batches_as_two(native_lib):
    """With ``fuse_mlp=True`` two chained Linears compiled at 64 rows are merged into one launcher
    that runs both in one kernel (h in shared memory); the same module compiled at 200 rows keeps
    its two fused launches.  Same values either way, against eager."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import fuseml_b200 as F

    torch.manual_seed(11)
    block = torch.nn.Sequential(torch.nn.Linear(256, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 256)).to("cuda", torch.bfloat16)
    for rows, merged in ((64, True), (200, False)):
        torch._dynamo.reset()
        x = torch.randn(rows, 256, device="cuda", dtype=torch.bfloat16)
        comp = F.FuseMLCompiler(fuse_mlp=True)
        with torch.no_grad():
            y = torch.compile(block, backend=comp)(x)
            ref = block.float()(x.float())
            block.to(torch.bfloat16)
        torch.cuda.synchronize()
        assert F.device_status() == 0
        assert len(comp.launchers) == 2 and (len(comp.mlp_launchers) == 1) == merged
        if merged:
            assert comp.mlp_launchers[0].fused_count == 1
        else:
            assert sum(L.launch_count for L in comp.launchers) == 2
        np.testing.assert_allclose(y.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)
    torch._dynamo.reset()
