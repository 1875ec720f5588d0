"""GPU parity: the sm_100a kernels (through the C ABI) against the CPU oracle.

Tolerances, from the benchmark definition: bf16 outputs within rtol 1.6e-2 / atol 1e-2
of the fp32 result, fp32 outputs within 1e-3 / 1e-3, reductions within 1e-3 relative.
Every test checks the device status word afterwards: a bounded wait that ran out
would make the launch "succeed" with garbage, and must fail the test instead.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import chain, configs

pytestmark = pytest.mark.gpu

BF16_TOL = dict(rtol=1.6e-2, atol=1e-2)
F32_TOL = dict(rtol=1e-3, atol=1e-3)


@pytest.fixture(scope="module")
def K(native_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuseml_b200 import kernels

    return kernels


def _to_dev(t: torch.Tensor, dtype: str) -> torch.Tensor:
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    return t.to(td).cuda()


def _status_ok(K):
    assert K.device_status() == 0, "a bounded device-side wait ran out"


def _program(K, ops, env):
    """oracle op tuples -> EpilogueProgram with device tensors."""
    prog = K.EpilogueProgram()
    for op in ops:
        k = op[0]
        if k == "gelu_bwd":
            prog.gelu_backward(env[op[1]])
        elif k in ("bias", "add"):
            prog.add_tensor(env[op[1]])
        elif k == "mul":
            prog.mul_tensor(env[op[1]])
        elif k == "sub":
            prog.sub_tensor(env[op[1]])
        elif k == "rsub":
            prog.rsub_tensor(env[op[1]])
        elif k == "add_scalar":
            prog.add_scalar(op[1])
        elif k == "mul_scalar":
            prog.mul_scalar(op[1])
        elif k == "gelu":
            prog.gelu()
        elif k == "gelu_tanh":
            prog.gelu("tanh")
        elif k == "store_aux":
            prog.store_aux(env[op[1]])
        else:
            getattr(prog, k)()
    return prog


def run_stages_gpu(K, case) -> dict:
    """Mirror of oracle.configs.run_stages_oracle on the GPU kernels."""
    env = {k: _to_dev(v, case.dtype) for k, v in case.tensors.items()}
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[case.dtype]
    for st in case.stages:
        a = env[st.a]
        b = env[st.b].t() if st.b_view == "t" else env[st.b]
        prog = _program(K, st.ops, env)
        res = K.fused_gemm(a, b, prog, out_dtype=td, store=st.out is not None, reduce=st.reduce, axis=st.axis)
        if st.reduce:
            out, reds = res
            for k, nm in st.red_names.items():
                env[nm] = reds[k]
        else:
            out = res
        if st.out is not None:
            env[st.out] = out
    torch.cuda.synchronize()
    return {k: env[k].float().cpu().numpy() for k in case.outputs}


def _assert_close(got, ref, dtype, what):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, what
    if ref.ndim <= 1:
        scale = max(np.abs(ref).max(), 1e-30)
        assert np.abs(got - ref).max() <= 1e-3 * scale + 1e-6, what
    else:
        np.testing.assert_allclose(got, ref, err_msg=what, **(F32_TOL if dtype == "f32" else BF16_TOL))


# ---- the five configurations, scaled down, against oracle and golden fixtures ----

@pytest.mark.parametrize("name", list(configs.MAKERS))
def test_config_small_matches_oracle_and_reference_fixture(K, golden_dir, name):
    case = configs.make(name, small=(name != "cfg1"))
    got = run_stages_gpu(K, case)
    _status_ok(K)
    oracle = configs.run_stages_oracle(case)
    golden = np.load(golden_dir / f"numeric_{name}.npz")
    for k in case.outputs:
        # against the stage oracle (same bf16 storage points): tight
        if np.asarray(oracle[k]).ndim <= 1:
            _assert_close(got[k], oracle[k], case.dtype, f"{name}:{k} vs oracle")
        else:
            tol = F32_TOL if case.dtype == "f32" else dict(rtol=1.6e-2, atol=1e-2)
            np.testing.assert_allclose(got[k], oracle[k], err_msg=f"{name}:{k} vs oracle", **tol)
        # against the reference's own output (fp32 eager on the same inputs)
        if name == "cfg5" and k == "amax":
            np.testing.assert_allclose(got[k], golden[k], **BF16_TOL)
        else:
            _assert_close(got[k], golden[k], case.dtype, f"{name}:{k} vs reference fixture")


# ---- shape / layout sweep -------------------------------------------------------

SHAPES = [
    (1, 8, 8), (7, 24, 40), (128, 64, 256), (128, 512, 256), (129, 72, 264), (200, 136, 304),
    (384, 256, 640), (512, 512, 1024), (1000, 1000, 1000), (2048, 1024, 4096), (300, 4104, 520),
]


@pytest.mark.parametrize("b_view", ["t", "n"])
@pytest.mark.parametrize("M,Kd,Nn", SHAPES)
def test_plain_gemm_bf16(K, M, Kd, Nn, b_view):
    g = torch.Generator().manual_seed(M * 7 + Kd * 3 + Nn)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    b = (torch.randn(Kd, Nn, generator=g) / Kd ** 0.5).to(torch.bfloat16)
    ref = chain.fused_chain(a.float().numpy(), b.float().numpy(), (), out_dtype="bf16")["d"]
    bd = b.cuda() if b_view == "n" else b.t().contiguous().cuda().t()
    out = K.fused_gemm(a.cuda(), bd)
    torch.cuda.synchronize()
    _status_ok(K)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, **BF16_TOL)


@pytest.mark.parametrize("dtype,tol", [("f16", dict(rtol=2e-3, atol=2e-3)), ("f32", dict(rtol=1e-4, atol=1e-4))])
@pytest.mark.parametrize("b_view", ["t", "n"])
def test_other_operand_dtypes(K, dtype, tol, b_view):
    td = {"f16": torch.float16, "f32": torch.float32}[dtype]
    g = torch.Generator().manual_seed(5)
    a = torch.randn(200, 136, generator=g).to(td)
    b = (torch.randn(136, 304, generator=g) / 12).to(td)
    ref = chain.fused_chain(a.float().numpy(), b.float().numpy(), (), out_dtype=dtype)["d"]
    bd = b.cuda() if b_view == "n" else b.t().contiguous().cuda().t()
    out = K.fused_gemm(a.cuda(), bd)
    torch.cuda.synchronize()
    _status_ok(K)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, **tol)


def test_fp32_is_close_to_true_fp32_not_tf32(K):
    """fp32 operands run as three TF32 products (hi*hi + lo*hi + hi*lo).  What remains is
    the tensor core's own fp32 accumulation error (about K * 2^-24 of the running sum), so
    the result is several times closer to true fp32 than a single TF32 pass (~5e-4 here)
    and an order of magnitude inside the 1e-3 gate of the fp32 configuration."""
    g = torch.Generator().manual_seed(11)
    a = torch.randn(128, 2048, generator=g)
    b = torch.randn(2048, 512, generator=g) / 45
    ref = a.double() @ b.double()
    out = K.fused_gemm(a.cuda(), b.cuda()).cpu().double()
    _status_ok(K)
    err = (out - ref).abs().max().item()
    assert err < 2.5e-4, err


@pytest.mark.parametrize("b_view", ["t", "n"])
def test_tile_widths_and_cta_pairs(K, b_view):
    """Every tile width the router may pick (multiples of 32; CTA pairs above 128 columns,
    a single CTA at 128 and below) gives the same matrix."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(3)
    a = torch.randn(600, 256, generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn(256, 1000, generator=g) / 16).to(torch.bfloat16)
    b = b.cuda() if b_view == "n" else b.t().contiguous().cuda().t()
    ref = (a.float() @ b.float()).cpu().numpy()
    for tile_n, cluster in ((32, 1), (64, 1), (96, 1), (128, 1), (256, 1), (160, 2), (192, 2), (224, 2), (256, 2)):
        out = torch.full((600, 1000), float("nan"), dtype=torch.bfloat16, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, b, None, out, torch.bfloat16)
        plan = K.plan_for(desc, K.device_props())
        plan.tile_n, plan.cluster, plan.grid = tile_n, cluster, 6
        K.fused_gemm(a, b, None, out=out, plan=plan)
        torch.cuda.synchronize()
        _status_ok(K)
        np.testing.assert_allclose(out.float().cpu().numpy(), ref, err_msg=f"tile_n={tile_n} cluster={cluster}", **BF16_TOL)


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("M,Kd,Nn", [(256, 512, 384), (200, 136, 304), (1000, 4096, 520), (72, 8192, 256)])
def test_transposed_left_operand_is_read_in_place(K, M, Kd, Nn, dtype):
    """A stored [K, M] (the dY^T of a weight gradient, dW = dY^T @ X, where K is the token
    dimension) with B row-major [K, N]: both operands MN-major, no copy of either."""
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    g = torch.Generator().manual_seed(M + Kd + Nn)
    a_t = torch.randn(Kd, M, generator=g).to(td)                 # dY: [tokens, out_features]
    b = (torch.randn(Kd, Nn, generator=g) / Kd ** 0.5).to(td)     # X:  [tokens, in_features]
    ref = chain.fused_chain(a_t.float().numpy().T, b.float().numpy(), (), out_dtype=dtype)["d"]
    a_dev = a_t.cuda().t()
    assert K.addressable_left(a_dev, b.cuda()) is a_dev, "the view is passed as it is"
    out = K.fused_gemm(a_dev, b.cuda())
    torch.cuda.synchronize()
    _status_ok(K)
    tol = {"bf16": BF16_TOL, "f16": dict(rtol=2e-3, atol=2e-3), "f32": dict(rtol=1e-4, atol=1e-4)}[dtype]
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, **tol)


def test_strided_views_without_copies(K):
    """Row-strided A, row-strided output and a column-sliced weight are addressed in place."""
    g = torch.Generator().manual_seed(4)
    big_a = torch.randn(256, 512, generator=g).to(torch.bfloat16).cuda()
    a = big_a[:, :256]                      # lda = 512
    w = (torch.randn(384, 512, generator=g) / 16).to(torch.bfloat16).cuda()
    b = w[:, 128:384].t()                   # [256, 384] view, K-major with ld 512, offset 256 bytes
    big_out = torch.zeros(256, 1024, dtype=torch.bfloat16, device="cuda")
    out = big_out[:, 512:896]               # ldd = 1024
    K.fused_gemm(a, b, None, out=out)
    torch.cuda.synchronize()
    _status_ok(K)
    ref = a.float() @ b.float()
    np.testing.assert_allclose(out.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)
    assert float(big_out[:, :512].abs().max()) == 0.0 and float(big_out[:, 896:].abs().max()) == 0.0


def test_unsupported_layout_raises(K):
    a = torch.zeros(64, 100, dtype=torch.bfloat16, device="cuda")   # 200-byte rows
    b = torch.zeros(100, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="layout"):
        K.fused_gemm(a, b)


# ---- epilogue programs ----------------------------------------------------------------

def _epi_case(K, ops_fn, M=200, Kd=136, Nn=304, dtype="bf16", seed=0, **kw):
    g = torch.Generator().manual_seed(seed)
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    a = torch.randn(M, Kd, generator=g).to(td)
    b = (torch.randn(Kd, Nn, generator=g) / Kd ** 0.5).to(td)
    T = {
        "row": torch.randn(Nn, generator=g).to(td), "col": torch.randn(M, 1, generator=g).to(td),
        "full": torch.randn(M, Nn, generator=g).to(td), "full32": torch.randn(M, Nn, generator=g),
        "row2d": torch.randn(1, Nn, generator=g).to(td), "vecm": torch.randn(M, generator=g).to(td),
    }
    ops = ops_fn()
    np_ops = [tuple(T[o].float().numpy() if isinstance(o, str) and i > 0 else o for i, o in enumerate(op)) for op in ops]
    ref = chain.fused_chain(a.float().numpy(), b.float().numpy(), np_ops, out_dtype=dtype, **kw)
    env = {k: v.cuda() for k, v in T.items()}
    prog = _program(K, ops, env)
    res = K.fused_gemm(a.cuda(), b.cuda(), prog, **{("reduce" if k == "reduce" else k): v for k, v in kw.items()})
    torch.cuda.synchronize()
    _status_ok(K)
    return res, ref


EPILOGUES = {
    "relu": lambda: [("relu",)],
    "bias_gelu": lambda: [("bias", "row"), ("gelu",)],
    "bias_gelu_tanh": lambda: [("bias", "row"), ("gelu_tanh",)],
    "bias_sigmoid": lambda: [("bias", "row"), ("sigmoid",)],
    "bias_residual": lambda: [("bias", "row"), ("add", "full")],
    "residual_fp32_operand": lambda: [("add", "full32")],
    "scalars": lambda: [("mul_scalar", 0.5), ("add_scalar", 0.125)],
    "col_vector": lambda: [("mul", "col")],
    "row_2d": lambda: [("add", "row2d")],
    "sub_rsub": lambda: [("sub", "row"), ("rsub", "full")],
    "dag_gelu_mul_sigmoid_add": lambda: [("bias", "row"), ("save",), ("gelu",), ("swap",), ("sigmoid",),
                                         ("mul_saved",), ("add", "full")],
    "dag_sigmoid_first": lambda: [("bias", "row"), ("save",), ("sigmoid",), ("swap",), ("gelu",), ("mul_saved",)],
    "dag_saved_read_again": lambda: [("save",), ("gelu",), ("swap",), ("sigmoid",), ("mul_saved",), ("add_saved",)],
    "gelu_times_sigmoid_op": lambda: [("bias", "row"), ("gelu_times_sigmoid",), ("add", "full")],
    "dag_add_saved": lambda: [("save",), ("relu",), ("add_saved",)],
    "gelu_backward": lambda: [("gelu_bwd", "full")],
    "gelu_backward_fp32_operand_then_residual": lambda: [("gelu_bwd", "full32"), ("add", "full")],
    "long_chain": lambda: [("bias", "row"), ("relu",), ("mul_scalar", 2.0), ("add", "full"), ("sigmoid",),
                           ("mul", "col"), ("add_scalar", -0.25), ("gelu",)],
}


@pytest.mark.parametrize("name", list(EPILOGUES))
def test_epilogue_program(K, name):
    out, ref = _epi_case(K, EPILOGUES[name])
    np.testing.assert_allclose(out.float().cpu().numpy(), ref["d"], **BF16_TOL)


def test_one_d_operand_of_length_m_runs_along_rows(K):
    # square-ish case where the 1-D length equals M but not N
    out, ref = _epi_case(K, lambda: [("add", "vecm")], M=200, Nn=304)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref["d"], **BF16_TOL)


def test_epilogue_fp32_and_fp16_outputs(K):
    out, ref = _epi_case(K, EPILOGUES["bias_gelu"], dtype="f32")
    np.testing.assert_allclose(out.cpu().numpy(), ref["d"], **F32_TOL)
    out, ref = _epi_case(K, lambda: [("mul_scalar", 1e5)], dtype="f16")   # saturates at 65504
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all() and np.abs(got).max() == 65504.0
    np.testing.assert_allclose(got, ref["d"], rtol=2e-3, atol=1.0)


def test_escape_store_of_an_intermediate(K):
    g = torch.Generator().manual_seed(9)
    a = torch.randn(200, 136, generator=g).to(torch.bfloat16)
    b = (torch.randn(136, 304, generator=g) / 12).to(torch.bfloat16)
    aux = torch.zeros(200, 304, dtype=torch.bfloat16, device="cuda")
    prog = K.EpilogueProgram().relu().store_aux(aux).mul_scalar(3.0)
    out = K.fused_gemm(a.cuda(), b.cuda(), prog)
    torch.cuda.synchronize()
    _status_ok(K)
    ref = chain.fused_chain(a.float().numpy(), b.float().numpy(), [("relu",), ("store_aux",), ("mul_scalar", 3.0)])
    np.testing.assert_allclose(aux.float().cpu().numpy(), ref["aux"][0], **BF16_TOL)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref["d"], **BF16_TOL)


# ---- reductions ----------------------------------------------------------------------------

@pytest.mark.parametrize("axis", [-1, 0, None])
@pytest.mark.parametrize("store", [False, True])
def test_fused_reductions(K, axis, store):
    (out, reds), ref = _epi_case(K, EPILOGUES["bias_gelu"], M=520, Kd=256, Nn=1000, store=store,
                                 reduce=("sum", "max", "mean"), axis=axis)
    if store:
        np.testing.assert_allclose(out.float().cpu().numpy(), ref["d"], **BF16_TOL)
    else:
        assert out is None
    for k in ("sum", "max", "mean"):
        _assert_close(reds[k].cpu().numpy(), ref[k], "bf16", f"{k} axis={axis}")


def test_reduction_of_negative_values_and_ragged_edges(K):
    """max must not be polluted by the zero padding of edge tiles."""
    (out, reds), ref = _epi_case(K, lambda: [("add_scalar", -50.0)], M=130, Kd=72, Nn=264, store=False,
                                 reduce=("max", "sum"), axis=-1)
    assert (reds["max"].cpu().numpy() < -30).all()
    _assert_close(reds["max"].cpu().numpy(), ref["max"], "bf16", "max")
    _assert_close(reds["sum"].cpu().numpy(), ref["sum"], "bf16", "sum")


@pytest.mark.parametrize("axis", [-1, 0, None])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_standalone_reduce_tail(K, axis, dtype):
    g = torch.Generator().manual_seed(2)
    td = {"bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    x = torch.randn(1000, 3001 if dtype == "f32" else 3000, generator=g).to(td)
    r = K.reduce_tail(x.cuda(), ("sum", "max", "mean"), axis=axis)
    torch.cuda.synchronize()
    ref = chain.reduce_tail(x.float().numpy(), ("sum", "max", "mean"), axis)
    for k in ("sum", "max", "mean"):
        got = r[k].cpu().numpy()
        scale = max(np.abs(ref[k]).max(), 1.0)
        assert np.abs(got.astype(np.float64) - ref[k]).max() <= 1e-3 * scale, (k, axis)


# ---- full-size properties (no CPU oracle at these sizes) --------------------------------

def test_full_size_linearity_and_checksum(K):
    """At the benchmark's GEMM size: the kernel is linear in A (exactly, for power-of-two
    scaling) and a column checksum agrees with a GEMV computed independently."""
    g = torch.Generator(device="cuda").manual_seed(0)
    M, Kd, Nn = 8192, 4096, 4096
    a = torch.randn(M, Kd, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(Nn, Kd, generator=g, device="cuda") / 64).to(torch.bfloat16)
    out1 = K.fused_gemm(a, w.t(), out_dtype=torch.float32)
    out2 = K.fused_gemm(a * 2, w.t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _status_ok(K)
    assert torch.equal(out2, out1 * 2)
    # checksum of checksums: (1^T A) W^T == 1^T (A W^T)
    col = (a.double().sum(0) @ w.double().t())
    got = out1.double().sum(0)
    rel = ((got - col).abs().max() / col.abs().max()).item()
    assert rel < 1e-4, rel


def test_full_size_cfg3_reductions_match_unfused_path(K):
    """relu(A@B) -> amax/mean fused (C never stored) equals storing C in fp32 and reducing it."""
    case = configs.make("cfg3")
    A = case.tensors["A"].to(torch.bfloat16).cuda()
    B = case.tensors["B"].to(torch.bfloat16).cuda()
    prog = K.EpilogueProgram().relu()
    _, reds = K.fused_gemm(A, B, prog, store=False, reduce=("max", "mean"), axis=-1)
    c = K.fused_gemm(A, B, K.EpilogueProgram().relu(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _status_ok(K)
    assert torch.equal(reds["max"], c.amax(-1))
    ref_mean = c.double().mean(-1)
    assert ((reds["mean"].double() - ref_mean).abs().max() / ref_mean.abs().max()).item() < 1e-5
    # and against the fp32 eager path of the oracle on a slice of rows (CPU time bounded)
    rows = slice(0, 256)
    e = torch.relu(case.tensors["A"][rows] @ case.tensors["B"])
    _assert_close(reds["max"][rows].cpu().numpy(), e.amax(-1).numpy(), "bf16", "amax vs eager")
    _assert_close(reds["mean"][rows].cpu().numpy(), e.double().mean(-1).float().numpy(), "bf16", "mean vs eager")


@pytest.mark.parametrize("out_dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,Kd,Nn,pitch_pad", [(300, 256, 1000, 0), (256, 512, 2048, 0), (520, 192, 776, 8), (260, 128, 264, 3)])
def test_lone_tile_path_is_bit_identical_to_the_persistent_path(K, M, Kd, Nn, pitch_pad, out_dtype):
    """A launch whose CTA pairs get one tile each runs the sixteen-warp epilogue and moves the
    residual and the output through shared memory by TMA; forcing two CTA pairs to walk all
    tiles runs the eight-warp persistent path with direct loads and stores.  Same arithmetic in
    the same order: the outputs must be equal bit for bit, ragged edges included.  A residual
    whose row pitch is not a multiple of 16 bytes (pitch_pad = 3) cannot have a tensor map and
    keeps the direct path in both."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(11)
    td = {"bf16": torch.bfloat16, "f16": torch.float16}[out_dtype]
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(Nn, Kd, generator=g) / 8).to(torch.bfloat16).cuda()
    bias = torch.randn(Nn, generator=g).to(torch.bfloat16).cuda()
    r_full = torch.randn(M, Nn + pitch_pad, generator=g).to(torch.bfloat16).cuda()
    resid = r_full[:, :Nn]
    outs = []
    for grid in (None, 4):
        prog = K.EpilogueProgram().bias(bias).save().gelu().swap().sigmoid().mul_saved().add_tensor(resid)
        out = torch.full((M, Nn), float("nan"), dtype=td, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), prog, out, td)
        plan = K.plan_for(desc, K.device_props())
        assert plan.cluster == 2 and plan.tile_n == 256
        if grid is not None:
            plan.grid = grid
        K.fused_gemm(a, w.t(), prog, out_dtype=td, out=out, plan=plan)
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    h = a.float() @ w.float().t() + bias.float()
    ref = torch.nn.functional.gelu(h) * torch.sigmoid(h) + resid.float()
    tol = BF16_TOL if out_dtype == "bf16" else dict(rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), ref.cpu().numpy(), **tol)


@pytest.mark.parametrize("dtype,M,Kd,Nn", [("bf16", 128, 4096, 1024), ("bf16", 37, 2048, 520), ("f16", 64, 8192, 264),
                                            ("f32", 128, 512, 2048), ("bf16", 16, 16384, 4096)])
def test_split_k_matches_the_single_pass_launch(K, dtype, M, Kd, Nn):
    """Small-M problems with a long K loop are planned as split-K: several CTAs share one tile's
    K loop, store fp32 partial tiles, and a second kernel folds them and runs the epilogue
    (here a diamond with a residual and a row vector).  The same descriptor run with
    split_k = 1 walks the whole K loop per tile: same result up to the fp32 summation order."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(5)
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    a = torch.randn(M, Kd, generator=g).to(td).cuda()
    w = (torch.randn(Nn, Kd, generator=g) / Kd ** 0.5).to(td).cuda()
    bias = torch.randn(Nn, generator=g).to(td).cuda()
    resid = torch.randn(M, Nn, generator=g).to(td).cuda()
    outs = []
    for split in (None, 1):
        prog = K.EpilogueProgram().bias(bias).save().gelu().swap().sigmoid().mul_saved().add_tensor(resid)
        out = torch.full((M, Nn), float("nan"), dtype=td, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), prog, out, td)
        plan = K.plan_for(desc, K.device_props())
        if split is None:
            assert plan.split_k > 1 and plan.cluster == 1, plan.as_dict()
        else:
            plan.split_k = 1
            plan.grid = (Nn + plan.tile_n - 1) // plan.tile_n
        K.fused_gemm(a, w.t(), prog, out_dtype=td, out=out, plan=plan)
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(out.float().cpu().numpy())
    h = a.double() @ w.double().t() + bias.double()
    ref = (torch.nn.functional.gelu(h) * torch.sigmoid(h) + resid.double()).cpu().numpy()
    tol = {"bf16": BF16_TOL, "f16": dict(rtol=2e-3, atol=2e-3), "f32": dict(rtol=1e-3, atol=1e-3)}[dtype]
    np.testing.assert_allclose(outs[0], ref, **tol)
    np.testing.assert_allclose(outs[1], ref, **tol)
    np.testing.assert_allclose(outs[0], outs[1], **tol)


@pytest.mark.parametrize("M,Kd,Nn,tile_n", [(100, 256, 1000, 128), (128, 320, 1288, 256), (37, 128, 520, 64)])
def test_single_cta_lone_tile_path_is_bit_identical_to_the_persistent_path(K, M, Kd, Nn, tile_n):
    """The same comparison for one row of tiles (M <= 128, single-CTA kernels): one tile per CTA
    runs the sixteen-warp instance with the residual and output tiles moved by TMA, two CTAs
    walking all tiles run the eight-warp persistent path."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(13)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(Nn, Kd, generator=g) / 8).to(torch.bfloat16).cuda()
    bias = torch.randn(Nn, generator=g).to(torch.bfloat16).cuda()
    resid = torch.randn(M, Nn, generator=g).to(torch.bfloat16).cuda()
    tiles = (Nn + tile_n - 1) // tile_n
    outs = []
    for grid in (tiles, 2):
        prog = K.EpilogueProgram().bias(bias).gelu().mul_tensor(resid).add_scalar(0.25)
        out = torch.full((M, Nn), float("nan"), dtype=torch.bfloat16, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), prog, out, torch.bfloat16)
        plan = K.plan_for(desc, K.device_props())
        assert plan.cluster == 1
        plan.tile_n, plan.split_k, plan.grid = tile_n, 1, grid
        K.fused_gemm(a, w.t(), prog, out=out, plan=plan)
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    h = a.float() @ w.float().t() + bias.float()
    ref = torch.nn.functional.gelu(h) * resid.float() + 0.25
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)


# ---- the benchmark configurations at their full sizes, against the oracle on sampled rows ----
#
# Every op of these chains is independent per row of the activations, so the CPU oracle
# (seconds per few hundred rows at full width) is run on a sample of rows and compared with the
# same rows of the full-size GPU result: first and last rows, rows on both sides of every kind
# of tile boundary (128-row CTA blocks, 256-row pair tiles) and of the boundary between the waves
# of the persistent schedule, and an even spread in between.

def _sample_rows(M, n_even=160):
    picks = [np.arange(0, min(M, 4)), np.arange(max(0, M - 4), M)]
    for edge in (128, 256, 512, 1024, M // 2, M - 256, M - 128):
        if 0 < edge < M:
            picks.append(np.arange(max(0, edge - 3), min(M, edge + 3)))
    # 74 pair tiles of 256 rows form one wave of the persistent schedule
    for wave_edge in range(74 * 256, M, 74 * 256):
        picks.append(np.arange(wave_edge - 2, min(M, wave_edge + 2)))
    picks.append(np.linspace(0, M - 1, n_even).astype(np.int64))
    return np.unique(np.concatenate(picks))


def _row_subcase(case, rows, row_tensors):
    """The same case restricted to `rows` of its activations (weights and vectors unchanged);
    global reductions are dropped (they are checked separately), per-row ones kept."""
    import copy

    sub = copy.copy(case)
    sub.tensors = dict(case.tensors)
    for k in row_tensors:
        sub.tensors[k] = case.tensors[k][torch.as_tensor(rows)]
    sub.stages = []
    for st in case.stages:
        st2 = copy.copy(st)
        if st.reduce and st.axis is None:
            st2.reduce, st2.red_names = (), {}
        sub.stages.append(st2)
    sub.outputs = tuple(k for k in case.outputs if k not in ("sum",) and not (k == "amax" and case.name == "cfg5"))
    return sub


def test_full_size_cfg2_matches_oracle_on_every_row(K):
    """cfg2 at 256 x 16384 x 4096: 64 lone tiles on 64 CTA pairs, the sixteen-warp epilogue with
    TMA tile I/O, row-major [K,N] weight, the diamond gelu(h) * sigmoid(h) + r."""
    case = configs.make("cfg2")
    got = run_stages_gpu(K, case)
    _status_ok(K)
    ref = configs.run_stages_oracle(case)
    np.testing.assert_allclose(got["out"], ref["out"], **BF16_TOL)
    # the K-major view of the same weight (what nn.Linear holds) gives the same matrix
    env = {k: _to_dev(v, "bf16") for k, v in case.tensors.items()}
    wt = env["W"].t().contiguous().t()
    prog = _program(K, case.stages[0].ops, env)
    out = K.fused_gemm(env["x"], wt, prog)
    torch.cuda.synchronize()
    _status_ok(K)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref["out"], **BF16_TOL)


def test_full_size_cfg4_matches_oracle_on_sampled_rows(K):
    """cfg4 at M = 8192, D = 4096, I = 16384: seven waves of the persistent pair schedule in the
    first GEMM, the 256-block K loop (K = 16384) in the second."""
    case = configs.make("cfg4")
    got = run_stages_gpu(K, case)
    _status_ok(K)
    rows = _sample_rows(case.sizes["M"])
    ref = configs.run_stages_oracle(_row_subcase(case, rows, ("x",)))
    np.testing.assert_allclose(got["y"][rows], ref["y"], **BF16_TOL)


def test_full_size_cfg4_row_shards_equal_the_unsharded_result(K):
    """Rows sharded 8 ways (1024 rows per shard, the shape each GPU of a box gets) give the rows of
    the unsharded launch.  The shard launches deal the K loops of their ragged last wave out over
    all CTA pairs (stream-K), so a few tiles sum their K blocks in two or three parts instead of
    one run: equal up to the last bit of bf16 there, bit for bit everywhere else."""
    case = configs.make("cfg4")
    full = run_stages_gpu(K, case)["y"]
    M = case.sizes["M"]
    for shard in (0, 5, 7):
        rows = np.arange(shard * (M // 8), (shard + 1) * (M // 8))
        part = run_stages_gpu(K, _row_subcase(case, rows, ("x",)))["y"]
        np.testing.assert_allclose(part, full[rows], rtol=2.0 ** -7, atol=2.0 ** -7)
        assert (part == full[rows]).mean() > 0.9, shard
    _status_ok(K)


def test_full_size_cfg5_matches_oracle_on_sampled_rows_and_its_own_fold(K):
    """cfg5 at M = 32768: four residual blocks (eight fused GEMMs), the last one also producing the
    global sum and amax.  Sampled rows against the oracle; the two scalars against the float64
    fold of the kernel's own bf16 output."""
    case = configs.make("cfg5")
    nb = case.sizes["blocks"]
    got = run_stages_gpu(K, case)
    _status_ok(K)
    y = got[f"x{nb}"]
    rows = _sample_rows(case.sizes["M"], n_even=96)
    ref = configs.run_stages_oracle(_row_subcase(case, rows, ("x0",)))
    np.testing.assert_allclose(y[rows], ref[f"x{nb}"], **BF16_TOL)
    y64 = y.astype(np.float64)
    fold_sum = y64.sum()
    # the kernel sums the fp32 values it then rounds to bf16 for the store; the fold sees the
    # rounded ones: allow four standard deviations of that rounding (independent errors of
    # about 2^-9 relative per element) on top of the 1e-3 relative gate of a reduction
    rounding = 4.0 * np.sqrt(y64.size) * 2.0 ** -9 * np.sqrt((y64 ** 2).mean())
    assert abs(float(got["sum"]) - fold_sum) <= 1e-3 * abs(fold_sum) + rounding, (float(got["sum"]), fold_sum, rounding)
    top = float(y.max())
    assert abs(float(got["amax"]) - top) <= 2.0 ** -8 * abs(top), (float(got["amax"]), top)


# ---- the time-out path ----------------------------------------------------------------------

@pytest.mark.parametrize("cluster", [1, 2])
def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_correct(K, cluster):
    """Every device-side wait is bounded.  The failure is injected on the host: with the
    diagnostic switch on, each producer issues no TMA load for the last K block of its last tile,
    so the MMA thread waits (20 ms here instead of 2 s) on a barrier that nothing completes, with
    no copy in flight.  The kernel records where it gave up, frees its TMEM and returns; the host
    reads FUSEML_E_TIMEOUT / WHERE_MMA_FULL, and the same launch without the switch is correct."""
    import ctypes as C

    from fuseml_b200 import _native as N

    lib = N.load()
    g = torch.Generator().manual_seed(21)
    M = 128 if cluster == 1 else 256
    a = torch.randn(M, 256, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(512, 256, generator=g) / 16).to(torch.bfloat16).cuda()

    def launch():
        out = torch.empty(M, 512, dtype=torch.bfloat16, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), None, out, torch.bfloat16)
        plan = K.plan_for(desc, K.device_props())
        # two 256-column tiles walked by one CTA (or one CTA pair): the persistent eight-warp instance
        plan.tile_n, plan.cluster, plan.split_k, plan.grid = 256, cluster, 1, cluster
        return K.fused_gemm(a, w.t(), None, out=out, plan=plan)

    good = launch()
    torch.cuda.synchronize()
    _status_ok(K)
    K.set_diagnostics(wait_limit_us=20000, drop_last_load=True)
    try:
        launch()
        status = C.c_int32(0)
        rc = lib.fuseml_sm100_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(status))
    finally:
        K.set_diagnostics()
    assert rc == N.E_TIMEOUT and status.value == N.WHERE_MMA_FULL, (rc, hex(status.value))
    again = launch()
    torch.cuda.synchronize()
    _status_ok(K)
    assert torch.equal(again, good)
    np.testing.assert_allclose(good.float().cpu().numpy(), (a.float() @ w.float().t()).cpu().numpy(), **BF16_TOL)


# ---- both Linears of a small-M block in one kernel -------------------------------------------

MLP_CASES = [
    ("f32", 128, 512, 2048, 512),       # the fp32 parity configuration (cfg1)
    ("bf16", 128, 512, 2048, 512),
    ("bf16", 37, 256, 1024, 300),       # ragged rows, an output width that is not a multiple of 256
    ("f16", 64, 128, 576, 128),         # 576 = 9 slices of 64: more slices than 128-wide candidates allow
    ("f32", 100, 96, 160, 264),         # 160 = 5 slices of 32
    ("bf16", 128, 1024, 8192, 512),     # several slices per CTA (64 slices on 32 CTAs per output chunk)
]


@pytest.mark.parametrize("dtype,M,D,I,Dout", MLP_CASES)
def test_small_mlp_block_in_one_kernel_matches_two_stage_oracle(K, dtype, M, D, I, Dout):
    """y = (gelu(x W1^T + b1)) W2^T + b2 + r with h handed over in shared memory, against the oracle
    run as two fused stages (h rounded to the storage dtype between them, as the kernel does)."""
    td = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    g = torch.Generator().manual_seed(M + D + I + Dout)
    x = torch.randn(M, D, generator=g).to(td)
    w1 = (torch.randn(I, D, generator=g) / D ** 0.5).to(td)
    b1 = (torch.randn(I, generator=g) * 0.1).to(td)
    w2 = (torch.randn(Dout, I, generator=g) / I ** 0.5).to(td)
    b2 = (torch.randn(Dout, generator=g) * 0.1).to(td)
    r = torch.randn(M, Dout, generator=g).to(td)
    f = lambda t: t.float().numpy()
    h = chain.fused_chain(f(x), f(w1).T, [("bias", f(b1)), ("gelu",)], out_dtype=dtype)["d"]
    ref = chain.fused_chain(h, f(w2).T, [("bias", f(b2)), ("add", f(r))], out_dtype=dtype)["d"]
    dev = [t.cuda() for t in (x, w1, b1, w2, b2, r)]
    xd, w1d, b1d, w2d, b2d, rd = dev
    outs = []
    for _ in range(2):                         # twice: the second call finds the barriers' memory used
        y = K.fused_mlp(xd, w1d, w2d, K.EpilogueProgram().bias(b1d).gelu(), K.EpilogueProgram().bias(b2d).add_tensor(rd))
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(y)
    assert torch.equal(outs[0], outs[1]), "deterministic"
    tol = {"bf16": BF16_TOL, "f16": dict(rtol=4e-3, atol=4e-3), "f32": F32_TOL}[dtype]
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), ref, **tol)
    # and the same block as two separate fused launches
    h2 = K.fused_gemm(xd, w1d.t(), K.EpilogueProgram().bias(b1d).gelu())
    y2 = K.fused_gemm(h2, w2d.t(), K.EpilogueProgram().bias(b2d).add_tensor(rd))
    torch.cuda.synchronize()
    np.testing.assert_allclose(outs[0].float().cpu().numpy(), y2.float().cpu().numpy(), **tol)


def test_small_mlp_block_declines_what_it_cannot_run(K):
    x = torch.zeros(200, 64, dtype=torch.bfloat16, device="cuda")      # more than 128 rows
    w1 = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    w2 = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="one kernel"):
        K.fused_mlp(x, w1, w2)
    with pytest.raises(RuntimeError, match="one kernel"):               # an output wider than two 256-column chunks
        K.fused_mlp(x[:64], torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda"),
                    torch.zeros(1024, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="one kernel"):               # 104 columns of I: no slice width divides it
        K.fused_mlp(x[:64], torch.zeros(104, 64, dtype=torch.bfloat16, device="cuda"),
                    torch.zeros(64, 104, dtype=torch.bfloat16, device="cuda"))


# ---- K-split last wave ---------------------------------------------------------

@pytest.mark.parametrize("M,Kd,Nn,group,red", [
    (1500, 512, 2300, 3, ()),              # 6 x 9 pair tiles, bands of 3 columns, ragged edges
    (1500, 512, 2300, 4, ("sum", "max")),  # a last band of one column; row reductions
    (700, 1024, 1300, 8, ()),              # a band wider than the matrix: one band
    (2048, 8192, 4096, 2, ()),             # 8 x 16 tiles in eight bands: several tiles per pair
])
def test_column_band_rasterisation_matches_row_groups(K, M, Kd, Nn, group, red):
    """FUSEML_PLAN_GROUP_N only changes the order in which tiles are visited: every tile is still
    computed exactly once, so outputs (and reductions, up to the order of their partial sums) equal
    those of the row-group walk bit for bit."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(M + Nn + group)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(Nn, Kd, generator=g) / Kd ** 0.5).to(torch.bfloat16).cuda()
    bias = torch.randn(Nn, generator=g).to(torch.bfloat16).cuda()
    outs = []
    for band in (True, False):
        out = torch.full((M, Nn), float("nan"), dtype=torch.bfloat16, device="cuda")
        prog = K.EpilogueProgram().bias(bias).gelu()
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), prog, out, torch.bfloat16)
        plan = K.plan_for(desc, K.device_props())
        plan.group_m = group
        plan.flags = (plan.flags | N.PLAN_GROUP_N) if band else (plan.flags & ~N.PLAN_GROUP_N)
        res = K.fused_gemm(a, w.t(), K.EpilogueProgram().bias(bias).gelu(), out=out, plan=plan, reduce=red,
                           axis=-1 if red else None)
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(res)
    if red:
        (y_band, r_band), (y_rows, r_rows) = outs
        for k in red:
            assert torch.equal(r_band[k], r_rows[k]), k      # per-row partials are indexed by tile column, not by visit order
    else:
        y_band, y_rows = outs
    assert not torch.isnan(y_band.float()).any() and torch.equal(y_band, y_rows)
    ref = torch.nn.functional.gelu(a.double() @ w.double().t() + bias.double())
    np.testing.assert_allclose(y_band.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)


def test_k_split_launches_on_two_streams_do_not_wait_for_each_other(K):
    """In a K-split launch CTA pairs wait for other pairs of the same launch, so the whole grid has
    to be resident at once; such a kernel is launched cooperatively, which keeps two of them on two
    streams from each holding SMs the other needs.  Ten rounds of two concurrent launches finish
    with a clean status word and the right values."""
    from fuseml_b200 import _native as N

    M, Nn, Kd = 2560, 2560, 8192              # 100 pair tiles on 74 pairs: 26 left, two K slices each
    g = torch.Generator().manual_seed(11)
    sets = []
    for _ in range(2):
        a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(Nn, Kd, generator=g) / Kd ** 0.5).to(torch.bfloat16).cuda()
        r = torch.randn(M, Nn, generator=g).to(torch.bfloat16).cuda()
        sets.append((a, w, r, torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")))
    desc = N.GemmDesc()
    K.fill_desc(desc, sets[0][0], sets[0][1].t(), K.EpilogueProgram().add_tensor(sets[0][2]), sets[0][3], torch.bfloat16)
    plan = K.plan_for(desc, K.device_props())
    assert plan.flags & N.PLAN_STREAM_K and plan.grid == 148
    K.set_diagnostics(wait_limit_us=200_000)   # a wait that ran out would show within 0.2 s, as a status code
    try:
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        torch.cuda.synchronize()
        for _ in range(10):
            for st, (a, w, r, out) in zip(streams, sets):
                with torch.cuda.stream(st):
                    K.fused_gemm(a, w.t(), K.EpilogueProgram().add_tensor(r), out=out, plan=plan)
        torch.cuda.synchronize()
        _status_ok(K)
    finally:
        K.set_diagnostics()
    for a, w, r, out in sets:
        ref = a.double() @ w.double().t() + r.double()
        np.testing.assert_allclose(out.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)


STREAM_K_CASES = [
    # M, K, N, grid (CTAs; None = the router's), epilogue, reductions
    (1024, 4096, 16384, None, "gelu", ()),          # 256 tiles on 74 pairs: 3 whole waves + 34 tiles in two K slices each
    (4096, 16384, 4096, None, "res", ()),           # the same tile count with a 256-block K loop
    (600, 4096, 1000, 10, "res", ()),               # 12 tiles on 5 pairs: 2 tiles left, two slices each; ragged edges
    (520, 2048, 1100, 14, "gelu", ("sum", "max")),  # 15 tiles on 7 pairs: 1 tile left in seven slices; row reductions
    (2048, 1024, 2048, 18, "relu", ("mean",)),      # 64 tiles on 9 pairs: 1 tile left, 16 K blocks in 8 slices, one pair idle
    # more than half of the pairs hold a tile of the last wave: the others take the K tails
    (1024, 16384, 4096, None, "res", ()),           # 64 tiles, no whole wave: 10 helpers, seven short parts each
    (2048, 16384, 4096, None, "res", ()),           # 128 tiles: a whole wave, then 54 owners and 20 helpers
    (1280, 448, 256, 16, "gelu", ("sum", "max")),   # 5 tiles on 8 pairs, 7 K blocks: two helpers, one pair idle; reductions
    (200, 2560, 2200, 20, "res", ()),               # 9 tiles on 10 pairs: one helper adds 4 K blocks to every tile; ragged
    (600, 4096, 1000, 10, "saved", ()),             # a second value register: the flag is ignored, whole tiles
]


@pytest.mark.parametrize("M,Kd,Nn,grid,epi,red", STREAM_K_CASES)
def test_stream_k_matches_whole_tile_waves(K, M, Kd, Nn, grid, epi, red):
    """The same launch with and without FUSEML_PLAN_STREAM_K: each tile of the last wave is computed
    in equal K slices by several CTA pairs, the later slices pass through the workspace and are
    added in slice order.  Same values up to the order of the fp32 additions; both against fp64."""
    from fuseml_b200 import _native as N

    g = torch.Generator().manual_seed(M + Nn)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(Nn, Kd, generator=g) / Kd ** 0.5).to(torch.bfloat16).cuda()
    bias = torch.randn(Nn, generator=g).to(torch.bfloat16).cuda()
    r = torch.randn(M, Nn, generator=g).to(torch.bfloat16).cuda()

    def program():
        prog = K.EpilogueProgram().bias(bias)
        return {"gelu": prog.gelu, "relu": prog.relu, "res": lambda: prog.add_tensor(r),
                "saved": lambda: prog.save().relu().add_saved()}[epi]()

    outs = []
    for on in (True, False):
        out = torch.full((M, Nn), float("nan"), dtype=torch.bfloat16, device="cuda")
        desc = N.GemmDesc()
        K.fill_desc(desc, a, w.t(), program(), out, torch.bfloat16)
        plan = K.plan_for(desc, K.device_props())
        assert plan.cluster == 2
        if grid is not None:
            plan.grid = grid
        plan.flags = (plan.flags | N.PLAN_STREAM_K) if on else (plan.flags & ~N.PLAN_STREAM_K)
        res = K.fused_gemm(a, w.t(), program(), out=out, plan=plan, reduce=red, axis=-1 if red else None)
        torch.cuda.synchronize()
        _status_ok(K)
        outs.append(res)
    on, off = outs
    if red:
        (y_on, red_on), (y_off, red_off) = on, off
        for k in red:
            kk = {"max": "max"}.get(k, k)
            _assert_close(red_on[kk].cpu().numpy(), red_off[kk].cpu().numpy(), "bf16", k)
    else:
        y_on, y_off = on, off
    h = a.double() @ w.double().t() + bias.double()
    ref = {"gelu": torch.nn.functional.gelu, "relu": torch.relu, "res": lambda t: t + r.double(),
           "saved": lambda t: torch.relu(t) + t}[epi](h)
    np.testing.assert_allclose(y_on.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)
    np.testing.assert_allclose(y_off.float().cpu().numpy(), ref.cpu().numpy(), **BF16_TOL)
    assert not torch.isnan(y_on.float()).any()
    assert (y_on == y_off).float().mean() > 0.9
