"""The five benchmark configurations: seeded inputs, the eager fp32 module, and the
list of fused stages each one lowers to.  TEST INFRASTRUCTURE.

Inputs are synthetic and fully specified (no dataset): ``torch.manual_seed(seed)``
before the model is built, ``nn.Linear`` default init (Kaiming-uniform weights,
uniform bias), then the activations drawn in the listed order from N(0,1)
(the reference's benchmark does the same: ``x = torch.randn(M, d_model)``,
benchmarks/bench_mlp_block.py:968; models ``:160-220``).  For bf16 configurations
every tensor is drawn in fp32 and rounded to bf16 once; the oracle then works on
those rounded values in fp32, which is what "the reference's fp32 eager result on
the same inputs" means here.

The eager module is also the reference's own CPU path: on a CPU its compiler
cannot launch fused kernels and returns the un-lowered ``gm.forward``
(fuseml/compiler.py:213-228), i.e. exactly these modules.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import chain

# Full sizes named by the benchmark definition.
FULL = {
    "cfg1": dict(M=128, D=512, I=2048, dtype="f32"),
    "cfg2": dict(M=256, K=4096, N=16384, dtype="bf16"),
    "cfg3": dict(M=8192, K=4096, N=4096, dtype="bf16"),
    "cfg4": dict(M=8192, D=4096, I=16384, dtype="bf16"),
    "cfg5": dict(M=32768, D=4096, I=16384, blocks=4, dtype="bf16"),
}

# Scaled-down shapes the oracle finishes in well under a second; deliberately not
# multiples of the 128 x 256 tile so that edge tiles are exercised.
SMALL = {
    "cfg1": dict(M=128, D=512, I=2048, dtype="f32"),
    "cfg2": dict(M=72, K=200, N=328, dtype="bf16"),
    "cfg3": dict(M=200, K=136, N=304, dtype="bf16"),
    "cfg4": dict(M=136, D=128, I=520, dtype="bf16"),
    "cfg5": dict(M=264, D=128, I=512, blocks=4, dtype="bf16"),
}


def _q(t: torch.Tensor, dtype: str) -> torch.Tensor:
    """Round to the storage dtype once, keep as fp32."""
    if dtype == "bf16":
        return t.to(torch.bfloat16).float()
    if dtype == "f16":
        return t.to(torch.float16).float()
    return t.float()


@dataclass
class Stage:
    """One fused kernel: ``out = epilogue(A @ B)`` and/or reductions of it.

    ``a`` / ``b`` / operand entries name tensors in ``Case.tensors``; ``b_view`` is
    ``"t"`` when B is the transposed view of a stored ``[N,K]`` weight (nn.Linear)
    and ``"n"`` when B is stored row-major ``[K,N]``.
    """

    a: str
    b: str
    b_view: str
    ops: list                      # chain.run_epilogue op tuples with tensor *names* as operands
    out: str | None
    reduce: tuple = ()
    axis: object = None
    red_names: dict = field(default_factory=dict)


@dataclass
class Case:
    name: str
    dtype: str
    sizes: dict
    tensors: dict                  # name -> fp32 torch tensor (values exact in `dtype`)
    stages: list
    module: nn.Module              # the eager fp32 module (what the reference runs on a CPU)
    args: tuple                    # its positional inputs
    outputs: tuple                 # names of the module's outputs, in order
    tokens: int
    flops: float
    algo_bytes: float

    def eager(self) -> dict:
        """fp32 eager outputs by name."""
        with torch.no_grad():
            out = self.module(*self.args)
        if not isinstance(out, (tuple, list)):
            out = (out,)
        return {k: v for k, v in zip(self.outputs, out)}


class _MLP(nn.Module):
    def __init__(self, d, i, residual: bool):
        super().__init__()
        self.linear1 = nn.Linear(d, i)
        self.linear2 = nn.Linear(i, d)
        self.residual = residual

    def forward(self, x):
        y = self.linear2(F.gelu(self.linear1(x)))
        return y + x if self.residual else y


class _ActHeavy(nn.Module):
    def __init__(self, W, b):
        super().__init__()
        self.W = nn.Parameter(W, requires_grad=False)
        self.b = nn.Parameter(b, requires_grad=False)

    def forward(self, x, r):
        h = torch.addmm(self.b, x, self.W)
        return F.gelu(h) * torch.sigmoid(h) + r


class _GemmReduce(nn.Module):
    def forward(self, a, b):
        c = torch.relu(a @ b)
        return c.amax(-1), c.mean(-1)


class _Stack(nn.Module):
    def __init__(self, blocks):
        super().__init__()
        self.blocks = nn.ModuleList(blocks)

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        return x, x.sum(), x.amax()


def _quantize_module(m: nn.Module, dtype: str) -> None:
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(_q(p, dtype))


def make_cfg1(sizes=None, seed=0) -> Case:
    """fp32 MLP block: ``l2(gelu(l1(x)))``."""
    s = dict(FULL["cfg1"] if sizes is None else sizes)
    torch.manual_seed(seed)
    m = _MLP(s["D"], s["I"], residual=False).eval()
    x = torch.randn(s["M"], s["D"])
    T = {"x": x, "w1": m.linear1.weight.detach(), "b1": m.linear1.bias.detach(),
         "w2": m.linear2.weight.detach(), "b2": m.linear2.bias.detach()}
    stages = [
        Stage("x", "w1", "t", [("bias", "b1"), ("gelu",)], "h"),
        Stage("h", "w2", "t", [("bias", "b2")], "y"),
    ]

    M, D, I = s["M"], s["D"], s["I"]
    return Case("cfg1", "f32", s, T, stages, m, (x,), ("y",), M, 4.0 * M * D * I,
                4.0 * (M * D + D * I + I + I * D + D + M * D) + 8.0 * M * I)


def make_cfg2(sizes=None, seed=0) -> Case:
    """bf16 ``h = x@W + b; out = gelu(h) * sigmoid(h) + r`` with W stored row-major [K,N]."""
    s = dict(FULL["cfg2"] if sizes is None else sizes)
    dt = s["dtype"]
    torch.manual_seed(seed)
    lin = nn.Linear(s["K"], s["N"])
    W = _q(lin.weight.detach().t().contiguous(), dt)
    b = _q(lin.bias.detach(), dt)
    x = _q(torch.randn(s["M"], s["K"]), dt)
    r = _q(torch.randn(s["M"], s["N"]), dt)
    T = {"x": x, "W": W, "b": b, "r": r}
    stages = [Stage("x", "W", "n", [("bias", "b"), ("save",), ("gelu",), ("swap",), ("sigmoid",),
                                    ("mul_saved",), ("add", "r")], "out")]

    M, K, N = s["M"], s["K"], s["N"]
    return Case("cfg2", dt, s, T, stages, _ActHeavy(W, b).eval(), (x, r), ("out",), M, 2.0 * M * K * N,
                2.0 * (M * K + K * N + N + 2 * M * N))


def make_cfg3(sizes=None, seed=0) -> Case:
    """bf16 ``c = relu(A@B)``; ``amax(c,-1)``, ``mean(c,-1)``; C is never stored."""
    s = dict(FULL["cfg3"] if sizes is None else sizes)
    dt = s["dtype"]
    torch.manual_seed(seed)
    A = _q(torch.randn(s["M"], s["K"]), dt)
    B = _q(torch.randn(s["K"], s["N"]) / float(np.sqrt(s["K"])), dt)
    T = {"A": A, "B": B}
    stages = [Stage("A", "B", "n", [("relu",)], None, reduce=("max", "mean"), axis=-1,
                    red_names={"max": "amax", "mean": "mean"})]

    M, K, N = s["M"], s["K"], s["N"]
    return Case("cfg3", dt, s, T, stages, _GemmReduce().eval(), (A, B), ("amax", "mean"), M, 2.0 * M * K * N,
                2.0 * (M * K + K * N) + 8.0 * M)


def _mlp_stages(prefix, x_name, out_name):
    return [
        Stage(x_name, prefix + "w1", "t", [("bias", prefix + "b1"), ("gelu",)], prefix + "h"),
        Stage(prefix + "h", prefix + "w2", "t", [("bias", prefix + "b2"), ("add", x_name)], out_name),
    ]


def _mlp_bytes(M, D, I):
    # x read twice + out written (3 * M*D), both weights, h written and read back, biases; bf16
    return 2.0 * (3 * M * D + 2 * D * I + 2 * M * I + I + D)


def make_cfg4(sizes=None, seed=0) -> Case:
    """bf16 residual MLP block: ``l2(gelu(l1(x))) + x``."""
    s = dict(FULL["cfg4"] if sizes is None else sizes)
    dt = s["dtype"]
    torch.manual_seed(seed)
    m = _MLP(s["D"], s["I"], residual=True).eval()
    _quantize_module(m, dt)
    x = _q(torch.randn(s["M"], s["D"]), dt)
    T = {"x": x, "w1": m.linear1.weight.detach(), "b1": m.linear1.bias.detach(),
         "w2": m.linear2.weight.detach(), "b2": m.linear2.bias.detach()}
    stages = _mlp_stages("", "x", "y")

    M, D, I = s["M"], s["D"], s["I"]
    return Case("cfg4", dt, s, T, stages, m, (x,), ("y",), M, 4.0 * M * D * I, _mlp_bytes(M, D, I))


def make_cfg5(sizes=None, seed=0) -> Case:
    """bf16 stack of residual MLP blocks, then global ``sum`` and ``amax`` of the output."""
    s = dict(FULL["cfg5"] if sizes is None else sizes)
    dt = s["dtype"]
    nb = s.get("blocks", 4)
    torch.manual_seed(seed)
    blocks = [_MLP(s["D"], s["I"], residual=True).eval() for _ in range(nb)]
    for m in blocks:
        _quantize_module(m, dt)
    x = _q(torch.randn(s["M"], s["D"]), dt)
    T = {"x0": x}
    stages = []
    for i, m in enumerate(blocks):
        p = f"blk{i}_"
        T.update({p + "w1": m.linear1.weight.detach(), p + "b1": m.linear1.bias.detach(),
                  p + "w2": m.linear2.weight.detach(), p + "b2": m.linear2.bias.detach()})
        stages += _mlp_stages(p, f"x{i}", f"x{i + 1}")
    last = stages[-1]
    last.reduce, last.axis, last.red_names = ("sum", "max"), None, {"sum": "sum", "max": "amax"}

    M, D, I = s["M"], s["D"], s["I"]
    return Case("cfg5", dt, s, T, stages, _Stack(blocks).eval(), (x,), (f"x{nb}", "sum", "amax"), M, nb * 4.0 * M * D * I,
                nb * _mlp_bytes(M, D, I) + 8.0)


MAKERS = {"cfg1": make_cfg1, "cfg2": make_cfg2, "cfg3": make_cfg3, "cfg4": make_cfg4, "cfg5": make_cfg5}


def make(name: str, small: bool = False, seed: int = 0, sizes=None) -> Case:
    if sizes is None and small:
        sizes = SMALL[name]
    return MAKERS[name](sizes, seed)


def run_stages_oracle(case: Case) -> dict:
    """Run the stage list through :mod:`oracle.chain` (numpy), stage outputs rounded to the
    storage dtype exactly where the fused kernels write them to HBM."""
    env = {k: v.numpy() for k, v in case.tensors.items()}
    for st in case.stages:
        a = env[st.a]
        b = env[st.b].T if st.b_view == "t" else env[st.b]
        ops = [tuple(env[o] if isinstance(o, str) and i > 0 else o for i, o in enumerate(op)) for op in st.ops]
        res = chain.fused_chain(a, b, ops, out_dtype=case.dtype, reduce=st.reduce, axis=st.axis,
                                store=st.out is not None)
        if st.out is not None:
            env[st.out] = res["d"]
        for k, nm in st.red_names.items():
            env[nm] = res[k]
    return {k: env[k] for k in case.outputs}
