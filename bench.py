#!/usr/bin/env python
"""Benchmark of the fused GEMM + epilogue path on B200.

``python bench.py --gpus N --steps K --warmup W`` runs the residual Transformer-MLP block
(d_model 4096, d_intermediate 16384, 8192 tokens, bf16; synthetic N(0,1) activations,
nn.Linear-initialised weights), its rows sharded over the N GPUs (strong scaling, weights
replicated, no collective), and prints ONE JSON line with

* ``value``      tokens/s over all GPUs, inputs resident in HBM, K steps timed with CUDA events;
* ``e2e``        the same metric through the public call with pinned HOST buffers (host->device
                 copy of the tokens and device->host read of the result inside the timed region),
                 next to the copy-only ceiling of the same buffers on the same streams;
* ``roofline``   the dominant kernel's achieved TFLOP/s (or GB/s) over the K timed steps against
                 the measured peak of the matching regime (burst for a region well under a
                 second), and ``roofline_sustained``: the same step repeated for at least a
                 second, against the sustained peak, clocks sampled inside that region only;
* ``workloads``  the other benchmark configurations (cfg1 small fp32 MLP, cfg2 weight-streaming
                 GEMM, cfg3 GEMM + row reductions, cfg5 stacked MLP with global reductions and,
                 on several GPUs, its all-reduce), each timed for at least a second;
* ``cpu_baseline`` the CPU oracle (fp32 eager, what the reference executes on a CPU) timed on this
                 machine's host cores on a bounded sample.

``--impl reference`` times that CPU path alone (rank 0 only).  ``--workload`` makes another
configuration the headline; ``--no-extras`` skips the ``workloads`` sub-records.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
import torch.nn as nn  # noqa: E402
import torch.nn.functional as F  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum),
# from the ncu captures summarised under profiles/gemm_epilogue_kernel_v2_*.md.  cfg4 is the
# mean of its two launches (first GEMM 0.669 GB, second GEMM 1.337 GB: with K = 16384 the operand
# slabs of one wave of tiles do not survive in L2 until the next wave; algorithmic bytes are
# 0.47 GB per launch).  cfg5 was not captured (the same two kernels as cfg4, four times).
NCU_TRAFFIC_BYTES = {"cfg1": None, "cfg4": 1.0033e9, "cfg2": 1.483e8, "cfg3": 1.065e8, "cfg5": None,
                     "cfg4_training_step": None}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------------------
# workloads (same shapes and seeded synthetic inputs as the benchmark definition)
# --------------------------------------------------------------------------------------

class TransformerMLP(nn.Module):
    """Linear -> GELU -> Linear -> + residual (the reference's benchmark block,
    benchmarks/bench_mlp_block.py:160-182)."""

    def __init__(self, d_model, d_intermediate):
        super().__init__()
        self.linear1 = nn.Linear(d_model, d_intermediate)
        self.linear2 = nn.Linear(d_intermediate, d_model)

    def forward(self, x):
        return self.linear2(F.gelu(self.linear1(x))) + x


class StackedMLP(nn.Module):
    """``blocks`` residual MLP blocks; with ``reductions`` also the global sum and amax of the output."""

    def __init__(self, d_model, d_intermediate, blocks, reductions):
        super().__init__()
        self.blocks = nn.ModuleList([TransformerMLP(d_model, d_intermediate) for _ in range(blocks)])
        self.reductions = reductions

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        if self.reductions:
            return x, x.sum(), x.amax()
        return x


class ActHeavy(nn.Module):
    def __init__(self, W, b):
        super().__init__()
        self.W = nn.Parameter(W, requires_grad=False)
        self.b = nn.Parameter(b, requires_grad=False)

    def forward(self, x, r):
        h = torch.addmm(self.b, x, self.W)
        return F.gelu(h) * torch.sigmoid(h) + r


class GemmReduce(nn.Module):
    def __init__(self, B):
        super().__init__()
        self.B = nn.Parameter(B, requires_grad=False)

    def forward(self, a):
        c = torch.relu(a @ self.B)
        return c.amax(-1), c.mean(-1)


class Workload:
    """Resident tensors + ``step()`` (one pass of the hot path over one batch) + ``e2e_step()``
    (the same pass fed from pinned host memory, result read back).  Every pass goes through the
    public entry point, ``torch.compile(module, backend=FuseMLCompiler())``."""

    name = ""
    dtype = "bf16"
    bound = "tensor"
    expected_kernels = 1

    def _compile(self, module):
        import fuseml_b200 as FM

        self.compiler = FM.FuseMLCompiler()
        self.module = module.eval()
        self.compiled = torch.compile(self.module, backend=self.compiler)

    def check_compiled(self):
        c = self.compiler
        if not c.fusion_applied or len(c.launchers) != self.expected_kernels:
            raise SystemExit(f"{self.name}: expected {self.expected_kernels} fused kernels, compiler built "
                             f"{len(c.launchers)} (declined: {c.declined})")

    def fused_launches(self):
        return sum(L.launch_count for L in set(self.compiler.launchers))

    def e2e_finish(self):
        """Called once after the last e2e step, before the closing event is recorded."""

    #: steps one call of ``step()`` runs (a captured graph may hold several consecutive steps)
    steps_per_call = 1

    def use_graphs(self, steps_hint=1):
        """Capture the resident step in CUDA graphs where that pays (launch-bound steps)."""
        return False


def graph_steps(steps_hint, limit=60):
    """How many consecutive steps one captured graph holds: the timed step count itself when it is
    small, else its largest divisor up to `limit` (so that K timed steps are whole replays)."""
    k = max(1, int(steps_hint))
    for g in range(min(k, limit), 0, -1):
        if k % g == 0:
            return g
    return 1


class MLPBlock(Workload):
    """cfg4 (blocks=1) and cfg5 (blocks=4 + global sum/amax [+ allreduce])."""

    def __init__(self, rows, d_model=4096, d_inter=16384, blocks=1, reductions=False, world=1, seed=0):
        self.rows, self.D, self.I, self.blocks, self.reductions, self.world = rows, d_model, d_inter, blocks, reductions, world
        self.name = "cfg5_stacked_mlp_x4" if blocks > 1 else "cfg4_mlp_block"
        torch.manual_seed(seed)
        self._compile(StackedMLP(d_model, d_inter, blocks, reductions).to(device="cuda", dtype=torch.bfloat16))
        self.expected_kernels = 2 * blocks
        g = torch.Generator().manual_seed(seed + 1 + int(os.environ.get("RANK", "0")))
        self.x_host = torch.randn(rows, d_model, generator=g).to(torch.bfloat16).pin_memory()
        self.y_host = torch.empty(rows, d_model, dtype=torch.bfloat16).pin_memory()
        self.x = self.x_host.cuda()
        self.x_in = torch.empty_like(self.x)
        self.tokens = rows
        self.flops_per_launch = 2.0 * rows * d_model * d_inter
        self.launches_per_step = 2 * blocks + (1 if reductions else 0)
        self.gemm_launches_per_step = 2 * blocks
        self.flops = self.flops_per_launch * 2 * blocks
        # bf16: x read twice + out written, both weights, h written and read back, biases
        self.algo_bytes = blocks * 2.0 * (3 * rows * d_model + 2 * d_model * d_inter + 2 * rows * d_inter + d_inter + d_model)
        self.h2d_bytes = rows * d_model * 2
        self.d2h_bytes = rows * d_model * 2 + (8 if reductions else 0)
        self.scalars = None
        self.runner = None

    def _forward(self, x):
        with torch.no_grad():
            out = self.compiled(x)
        if not self.reductions:
            return out
        y, s, m = out
        if self.world > 1:
            from fuseml_b200.sharding import allreduce_scalars

            s, m = allreduce_scalars(total=s, maximum=m)     # NCCL all-reduce: SUM and MAX of one scalar each
        self.scalars = (s, m)
        return y

    def step(self):
        return self._forward(self.x)

    def _forward_all(self, x):
        """(y, sum, amax): what a caller of the stacked block gets back, scalars as 1-element tensors."""
        y = self._forward(x)
        s, m = self.scalars
        return y, s.reshape(1), m.reshape(1)

    def e2e_step(self):
        # rows are independent: copy-in / kernels / copy-out run on three CUDA streams
        # (fuseml_b200.runtime), successive batches pipelining into each other; the metrics of the
        # stacked workload travel back with the output, 4 bytes each, into pinned host memory
        if self.runner is None:
            from fuseml_b200.runtime import HostStreamedModule

            # one chunk per batch measured best here: successive batches still pipeline into each other
            self.runner = HostStreamedModule(self._forward_all if self.reductions else self.compiled,
                                             rows_per_chunk=self.rows)
            if self.reductions:
                _, s, m = self._forward_all(self.x)
                self.s_host = torch.empty(1, dtype=s.dtype).pin_memory()
                self.m_host = torch.empty(1, dtype=m.dtype).pin_memory()
                self.d2h_bytes = self.rows * self.D * 2 + s.element_size() + m.element_size()
        if self.reductions:
            self.runner.submit(self.x_host, (self.y_host, self.s_host, self.m_host))
        else:
            self.runner.submit(self.x_host, self.y_host)
        return None

    def e2e_finish(self):
        if self.runner is not None:
            self.runner.wait_on()


class ActHeavyGemm(Workload):
    """cfg2: out = gelu(h) * sigmoid(h) + r with h = x @ W + b, W row-major [K,N]."""

    name = "cfg2_act_heavy_gemm"
    bound = "hbm"

    def __init__(self, rows=256, Kd=4096, Nn=16384, seed=0, copies=3):
        torch.manual_seed(seed)
        lin = nn.Linear(Kd, Nn)
        W = lin.weight.detach().t().contiguous().to(torch.bfloat16).cuda()
        b = lin.bias.detach().to(torch.bfloat16).cuda()
        self._compile(ActHeavy(W, b))
        # rotate several copies of the 128 MB weight so that no launch finds it in the 126 MB L2
        self.Ws = [W] + [W.clone() for _ in range(copies - 1)]
        self.x_host = torch.randn(rows, Kd).to(torch.bfloat16).pin_memory()
        self.r_host = torch.randn(rows, Nn).to(torch.bfloat16).pin_memory()
        self.y_host = torch.empty(rows, Nn, dtype=torch.bfloat16).pin_memory()
        self.x, self.r = self.x_host.cuda(), self.r_host.cuda()
        self.x_in, self.r_in = torch.empty_like(self.x), torch.empty_like(self.r)
        self.i = 0
        self.graphs = None
        self.tokens = rows
        self.flops_per_launch = self.flops = 2.0 * rows * Kd * Nn
        self.algo_bytes = 2.0 * (rows * Kd + Kd * Nn + Nn + 2 * rows * Nn)
        self.launches_per_step = self.gemm_launches_per_step = 1
        self.h2d_bytes = rows * Kd * 2 + rows * Nn * 2
        self.d2h_bytes = rows * Nn * 2

    def _forward(self, x, r):
        self.module.W.data = self.Ws[self.i % len(self.Ws)]   # same shape / stride: no recompilation
        self.i += 1
        with torch.no_grad():
            return self.compiled(x, r)

    def step(self):
        if self.graphs is not None:
            return self.graphs()
        return self._forward(self.x, self.r)

    def use_graphs(self, steps_hint=1):
        """One captured graph of several consecutive steps, each on the next copy of the weight (the
        step is a single kernel of about 35 us: launched one by one, the host's launch path and the
        gap between two graph launches are part of the measurement; inside a graph the launches
        keep their programmatic dependency, so a step's set-up overlaps its predecessor's tail)."""
        from fuseml_b200.runtime import GraphedCallable

        g = graph_steps(steps_hint)

        def several(x, r):
            return [self._forward(x, r) for _ in range(g)]

        self.graphs = GraphedCallable(several, self.x, self.r)
        self.steps_per_call = g
        return True

    def e2e_step(self):
        self.x_in.copy_(self.x_host, non_blocking=True)
        self.r_in.copy_(self.r_host, non_blocking=True)
        y = self._forward(self.x_in, self.r_in)
        self.y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class GemmRowReduce(Workload):
    """cfg3: relu(A @ B) -> amax and mean over the last dim; C is never written."""

    name = "cfg3_gemm_row_reductions"

    def __init__(self, rows=8192, Kd=4096, Nn=4096, seed=0):
        torch.manual_seed(seed)
        self.a_host = torch.randn(rows, Kd).to(torch.bfloat16).pin_memory()
        self.A = self.a_host.cuda()
        self.A_in = torch.empty_like(self.A)
        self._compile(GemmReduce((torch.randn(Kd, Nn) / Kd ** 0.5).to(torch.bfloat16).cuda()))
        self.out_host = torch.empty(2, rows, dtype=torch.bfloat16).pin_memory()
        self.tokens = rows
        self.flops_per_launch = self.flops = 2.0 * rows * Kd * Nn
        self.algo_bytes = 2.0 * (rows * Kd + Kd * Nn) + 8.0 * rows
        self.launches_per_step = 2
        self.gemm_launches_per_step = 1
        self.h2d_bytes = rows * Kd * 2
        self.d2h_bytes = rows * 4

    def _forward(self, A):
        with torch.no_grad():
            return self.compiled(A)

    def step(self):
        return self._forward(self.A)

    def e2e_step(self):
        self.A_in.copy_(self.a_host, non_blocking=True)
        mx, mean = self._forward(self.A_in)
        self.out_host[0].copy_(mx, non_blocking=True)
        self.out_host[1].copy_(mean, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class SmallFp32MLP(Workload):
    """cfg1: fp32 ``linear2(gelu(linear1(x)))`` at M = 128 (a latency-bound parity configuration:
    both Linears run the fused kernel on 3xTF32 operands, the first with bias + GELU, the second
    with its bias alone as the epilogue; no library GEMM is left in the step)."""

    name = "cfg1_fp32_mlp_small"
    dtype = "f32"
    bound = "hbm"

    def __init__(self, rows=128, d_model=512, d_inter=2048, seed=0):
        torch.manual_seed(seed)

        class Block(nn.Module):
            def __init__(self):
                super().__init__()
                self.linear1 = nn.Linear(d_model, d_inter)
                self.linear2 = nn.Linear(d_inter, d_model)

            def forward(self, x):
                return self.linear2(F.gelu(self.linear1(x)))

        self._compile(Block().to(device="cuda"))
        self.x_host = torch.randn(rows, d_model).pin_memory()
        self.y_host = torch.empty(rows, d_model).pin_memory()
        self.x = self.x_host.cuda()
        self.x_in = torch.empty_like(self.x)
        self.graph = None
        self.tokens = rows
        self.flops_per_launch = 2.0 * rows * d_model * d_inter
        self.flops = 2 * self.flops_per_launch
        # two kernels, h makes an fp32 round trip: x, W1, b1, h out | h in, W2, b2, y out
        self.algo_bytes = 4.0 * (rows * d_model + 2 * d_model * d_inter + d_inter + d_model + rows * d_model) \
            + 8.0 * rows * d_inter
        self.expected_kernels = 2
        # per Linear: the operand expansion, the split-K GEMM and its finish pass
        self.launches_per_step = 6
        self.gemm_launches_per_step = 2
        self.h2d_bytes = rows * d_model * 4
        self.d2h_bytes = rows * d_model * 4

    def _forward(self, x):
        with torch.no_grad():
            return self.compiled(x)

    def step(self):
        return self.graph() if self.graph is not None else self._forward(self.x)

    def use_graphs(self, steps_hint=1):
        from fuseml_b200.runtime import GraphedCallable

        g = graph_steps(steps_hint)

        def several(x):
            return [self._forward(x) for _ in range(g)]

        self.graph = GraphedCallable(several, self.x)
        self.steps_per_call = g
        return True

    def e2e_step(self):
        self.x_in.copy_(self.x_host, non_blocking=True)
        y = self._forward(self.x_in)
        self.y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class TrainingStep(Workload):
    """Forward and backward of the cfg4 block through the compiler: two fused forward kernels (the
    first also stores the pre-activation for the backward pass) and four fused backward GEMMs
    (data gradients with gelu'(pre) / the residual's gradient as epilogues, weight gradients with
    the transposed operand read in place).  Six GEMMs of 2*M*D*I FLOP each per step."""

    name = "cfg4_training_step"
    bound = "tensor"
    expected_kernels = 6

    def __init__(self, rows=8192, d_model=4096, d_inter=16384, seed=0):
        torch.manual_seed(seed)
        self._compile(TransformerMLP(d_model, d_inter).to(device="cuda", dtype=torch.bfloat16))
        self.module.train()
        self.x = torch.randn(rows, d_model, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        self.dy = torch.randn(rows, d_model, device="cuda", dtype=torch.bfloat16)
        self.tokens = rows
        self.flops_per_launch = 2.0 * rows * d_model * d_inter
        self.flops = 6 * self.flops_per_launch
        self.launches_per_step = self.gemm_launches_per_step = 6

    def step(self):
        for p in self.module.parameters():
            p.grad = None
        self.x.grad = None
        self.compiled(self.x).backward(self.dy)


def make_workload(name, world, scaling):
    if name == "cfg1":
        return SmallFp32MLP()
    if name == "cfg4":
        return MLPBlock(8192 if scaling == "weak" else 8192 // world, world=world)
    if name == "cfg5":
        return MLPBlock(32768 if scaling == "weak" else 32768 // world, blocks=4, reductions=True, world=world)
    if name == "cfg2":
        return ActHeavyGemm()
    if name == "cfg3":
        return GemmRowReduce()
    raise SystemExit(f"unknown workload {name}")


# config.workload of each --workload choice (the same string in both arms)
WORKLOAD_NAMES = {"cfg1": "cfg1_fp32_mlp_small", "cfg2": "cfg2_act_heavy_gemm", "cfg3": "cfg3_gemm_row_reductions",
                  "cfg4": "cfg4_mlp_block", "cfg5": "cfg5_stacked_mlp_x4"}
GLOBAL_ROWS = {"cfg1": 128, "cfg2": 256, "cfg3": 8192, "cfg4": 8192, "cfg5": 32768}
SHARDED = ("cfg4", "cfg5")


def workload_config(name, world, scaling):
    """The ``config`` object of the JSON line: the same in both arms."""
    sharded = name in SHARDED and world > 1
    per_gpu = GLOBAL_ROWS[name] if (scaling == "weak" or not sharded) else GLOBAL_ROWS[name] // world
    return {
        "workload": WORKLOAD_NAMES[name], "rows_per_gpu": per_gpu,
        "global_rows": per_gpu * world if name in SHARDED else per_gpu,
        "l2": ("9 MB working set, resident in L2: a latency-bound parity configuration, not a roofline claim"
               if name == "cfg1" else
               "inputs larger than L2 (weights + activations per step exceed 126 MB"
               + ("; weight copies rotated)" if name == "cfg2" else ")")),
        "parallelism": (f"rows sharded over {world} GPU(s), weights replicated" if name in SHARDED
                        else "one GPU per replica"),
    }


# --------------------------------------------------------------------------------------
# CPU baseline: the oracle's eager fp32 module on the host cores
# --------------------------------------------------------------------------------------

CPU_SAMPLE_ROWS = {"cfg1": 128, "cfg4": 512, "cfg5": 128, "cfg3": 512, "cfg2": 64}


def cpu_baseline(workload_name, budget_s=20.0, steps=None, warmup=1):
    """Times the CPU oracle (fp32 eager module = what the reference runs on a CPU) on a
    bounded sample of the workload.  Returns (tokens_per_s, description, cores, ms_per_step, steps)."""
    from oracle import configs

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    full = dict(configs.FULL[workload_name])
    rows = CPU_SAMPLE_ROWS[workload_name]
    full["M"] = rows
    case = configs.make(workload_name, sizes=full)
    with torch.no_grad():
        for _ in range(max(1, warmup)):
            case.module(*case.args)
        times = []
        t_start = time.perf_counter()
        n = 0
        while True:
            t0 = time.perf_counter()
            case.module(*case.args)
            times.append(time.perf_counter() - t0)
            n += 1
            if steps is not None:
                if n >= steps:
                    break
            elif time.perf_counter() - t_start > budget_s or n >= 50:
                break
    mean = sum(times) / len(times)
    desc = (f"{workload_name} at full width, {rows} of the rows per step, fp32 eager PyTorch on "
            f"{cores} threads, mean of {n} steps after {max(1, warmup)} warm-up")
    return rows / mean, desc, cores, mean * 1e3, n


# --------------------------------------------------------------------------------------
# clocks: NVML polled from a thread, only while a timed region runs
# --------------------------------------------------------------------------------------

class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, polled through NVML every few
    milliseconds between ``start()`` and ``stop()``.  The host thread that launches the timed
    steps spends the region inside ``cudaDeviceSynchronize`` (GIL released), so the poller runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, cuda_index):
        self.handle = None
        self.nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(cuda_index)
            bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
            self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None
        self._stop = threading.Event()
        self._thread = None
        self.samples = []

    def _poll(self):
        nv, h = self.nvml, self.handle
        while not self._stop.is_set():
            try:
                clk = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                self.samples.append((clk, watts, mask))
            except Exception:
                pass
            self._stop.wait(0.004)

    def start(self):
        self.samples = []
        self._stop.clear()
        if self.handle is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None
        out = {"sm_mhz": None, "sm_max_mhz": getattr(self, "max_mhz", None), "reasons": [], "samples": len(self.samples),
               "window": "inside the timed region only"}
        if self.samples:
            clks = sorted(c for c, _, _ in self.samples)
            mask = 0
            for _, _, m in self.samples:
                mask |= m
            out.update(sm_mhz=clks[len(clks) // 2], sm_mhz_min=clks[0], sm_mhz_max=clks[-1],
                       reasons=sorted(n for b, n in self.REASONS.items() if mask & b),
                       power_w_max=max(w for _, w, _ in self.samples))
        return out


# --------------------------------------------------------------------------------------

def run_reference(args):
    """The reference arm: its CPU path for this workload on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    steps, warm = max(1, args.steps), max(1, args.warmup)
    # the sample is sized so that `steps` + `warmup` passes end within a few minutes
    val, desc, cores, ms, n = cpu_baseline(args.workload, steps=min(steps, 100), warmup=min(warm, 10))
    line = {
        "impl": "reference", "metric": "mlp_block_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": n, "warmup": min(warm, 10), "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, world, args.scaling),
        "note": "CPU path of the reference = eager fp32 module (its compiler returns gm.forward on a CPU); "
                "each step is a bounded row sample of the workload at full width",
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


class Harness:
    """Timing on one rank of the job: barriers, CUDA events, max over ranks, clocks inside the region."""

    def __init__(self, dist, sampler):
        self.dist = dist
        self.sampler = sampler

    def barrier(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def allmax(self, v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, n, finish=None, clocks=True):
        """ms for n calls of fn (max over ranks) and the clock record of exactly that region."""
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if clocks and self.sampler is not None:
            self.sampler.start()
        e0.record()
        for _ in range(n):
            fn()
        if finish is not None:
            finish()          # make the timing stream wait for work enqueued on other streams
        e1.record()
        torch.cuda.synchronize()
        rec = self.sampler.stop() if clocks and self.sampler is not None else {}
        ms = self.allmax(e0.elapsed_time(e1))
        self.barrier()
        return ms, rec

    def timed_for(self, fn, seconds, per_step_ms, finish=None):
        """Repeat fn for at least `seconds`; the count comes from an all-reduced estimate, so every
        rank runs the same number of steps (and collectives)."""
        n = max(3, min(200000, int(math.ceil(seconds * 1e3 / max(per_step_ms, 1e-3)))))
        ms, rec = self.timed(fn, n, finish=finish)
        return ms, n, rec


def roofline_of(wl, name, launch_ms, region_s, peaks, peak_src):
    """Achieved rate of the dominant kernel over a timed region against the measured peak of the
    regime the region ran in: a region well under a second is a burst (the GPU has not settled at
    the power cap yet), a region of a second or more is sustained."""
    if wl.bound == "tensor":
        achieved = wl.flops_per_launch / (launch_ms * 1e-3) / 1e12
        kind = "bf16_tflops" if region_s < 0.5 else "bf16_tflops_sustained"
        peak = peaks[kind]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_kind": f"{kind}, {peak_src}", "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"]}
    else:
        achieved = wl.algo_bytes / (launch_ms * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": f"hbm_gbs, {peak_src}"}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(name)
    roof["kernel"] = "gemm_epilogue_kernel_v2"
    roof["launch_us"] = launch_ms * 1e3
    roof["region_s"] = region_s
    return roof


def prepare(wl, W, use_graph, steps):
    for _ in range(W):
        wl.step()
    wl.check_compiled()
    graphed = False
    if use_graph:
        try:
            graphed = wl.use_graphs(steps)
        except Exception as exc:          # capture is an optimisation, never a requirement
            print(f"[bench] CUDA graph capture failed, stepping eagerly: {exc!r}", file=sys.stderr)
            wl.graphs = wl.graph = None
            wl.steps_per_call = 1
        for _ in range(3):
            wl.step()
    torch.cuda.synchronize()
    return graphed


def check_status():
    from fuseml_b200 import kernels as K

    status = K.device_status()
    if status != 0:
        raise SystemExit(f"device status {status:#x}: a bounded wait ran out; numbers would be meaningless")


def link_ceiling(h, wl, steps):
    """Copy-only ceiling of the end-to-end path: the same pinned buffers, one host->device and one
    device->host copy per step on two streams, no kernel; every rank at once.  ms per step."""
    ins = [t for t in (getattr(wl, n, None) for n in ("x_host", "r_host", "a_host")) if t is not None]
    outs = [t for t in (getattr(wl, n, None) for n in ("y_host", "out_host")) if t is not None]
    dev_in = [torch.empty_like(t, device="cuda") for t in ins]
    dev_out = [torch.empty_like(t, device="cuda") for t in outs]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copy_step():
        with torch.cuda.stream(s_in):
            for d, t in zip(dev_in, ins):
                d.copy_(t, non_blocking=True)
        with torch.cuda.stream(s_out):
            for d, t in zip(dev_out, outs):
                t.copy_(d, non_blocking=True)

    def finish():
        cur = torch.cuda.current_stream()
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    for _ in range(2):
        copy_step()
    finish()
    ms, _ = h.timed(copy_step, steps, finish=finish, clocks=False)
    return ms / steps


def measure(h, wl, name, W, steps, use_graph, peaks, peak_src, world, sustained_s=1.0):
    """K timed steps (the headline numbers) and the same step repeated for `sustained_s` seconds."""
    graphed = prepare(wl, W, use_graph, steps)
    spc = wl.steps_per_call            # a captured graph may hold several consecutive steps
    steps = max(1, steps // spc) * spc
    before = wl.fused_launches()
    total_ms, clocks = h.timed(wl.step, steps // spc)
    launches = wl.gemm_launches_per_step * steps if graphed else wl.fused_launches() - before
    launches += steps * (wl.launches_per_step - wl.gemm_launches_per_step)
    check_status()
    ms_per_step = total_ms / steps
    out = {
        "ms_per_step": ms_per_step, "steps": steps, "tokens_per_s": wl.tokens * world / (ms_per_step * 1e-3),
        "tflops": wl.flops * world / (ms_per_step * 1e-3) / 1e12,
        "roofline": roofline_of(wl, name, ms_per_step / wl.gemm_launches_per_step, total_ms * 1e-3, peaks, peak_src),
        "clocks": clocks, "gpu_launches": launches, "cuda_graph": bool(graphed), "steps_per_graph": spc if graphed else None,
    }
    if sustained_s:
        s_ms, calls, s_clocks = h.timed_for(wl.step, sustained_s, ms_per_step * spc)
        n = calls * spc
        check_status()
        out["sustained"] = {
            "ms_per_step": s_ms / n, "steps": n, "tokens_per_s": wl.tokens * world / (s_ms / n * 1e-3),
            "roofline": roofline_of(wl, name, s_ms / n / wl.gemm_launches_per_step, s_ms * 1e-3, peaks, peak_src),
            "clocks": s_clocks,
        }
    return out


def measure_e2e(h, wl, steps, world):
    ceiling_ms = link_ceiling(h, wl, steps)
    # warm-up: the three-stream pipeline keeps several steps' outputs alive at once; the caching
    # allocator must have grown to that depth before the timed region (a cudaMalloc inside it
    # synchronises the device and stalls the pipeline)
    for _ in range(8):
        wl.e2e_step()
    wl.e2e_finish()
    torch.cuda.synchronize()
    e2e_ms, _ = h.timed(wl.e2e_step, steps, finish=wl.e2e_finish, clocks=False)
    per = e2e_ms / steps
    moved = (wl.h2d_bytes + wl.d2h_bytes) * world
    return {"value": wl.tokens * world / (per * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": wl.h2d_bytes * world, "d2h_bytes_per_step": wl.d2h_bytes * world,
            "ms_per_step": per,
            # both directions run at once: bytes moved per second over all ranks, copies alone against the full step
            "link_ceiling_ms_per_step": ceiling_ms, "link_ceiling_gbs": moved / (ceiling_ms * 1e-3) / 1e9,
            "link_achieved_gbs": moved / (per * 1e-3) / 1e9}


def release():
    """Free the previous workload's device memory and compiled graphs (the caller drops its reference first)."""
    import gc

    gc.collect()
    torch._dynamo.reset()
    torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong: the configuration's rows are split over the GPUs; weak: every GPU gets all of them")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no `workloads` sub-records)")
    ap.add_argument("--no-graph", action="store_true", help="do not capture launch-bound steps in CUDA graphs")
    ap.add_argument("--profile", action="store_true",
                    help="for runs under a profiler: the K timed steps of the headline workload only (no sustained "
                         "leg, no end-to-end leg, no other workloads, no CPU baseline, no CUDA graph)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    dist = None
    numa_cores = None
    if world > 1:
        import torch.distributed as dist
        from fuseml_b200.sharding import bind_to_device_numa

        # one process per GPU, each streaming its own batch through pinned memory: keep the
        # buffers on the GPU's own socket (N = 1 keeps every core for the CPU baseline leg)
        numa_cores = bind_to_device_numa(local_rank)

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from fuseml_b200 import _native, build as _build

    _build.build()
    _native.load()
    W = max(3, args.warmup)
    steps = max(1, args.steps)
    h = Harness(dist, ClockSampler(local_rank))
    peaks, peak_src = load_peaks()
    use_graph = not args.no_graph
    name = args.workload
    scaling = args.scaling if name in SHARDED else "weak"

    wl = make_workload(name, world, scaling)
    if args.profile:
        head = measure(h, wl, name, W, steps, False, peaks, peak_src, world, sustained_s=0)
        if rank == 0:
            print(json.dumps({"profile_run": True, "config": workload_config(name, world, scaling),
                              "ms_per_step": head["ms_per_step"], "gpu_launches": head["gpu_launches"]}))
        if dist is not None:
            dist.destroy_process_group()
        return
    head = measure(h, wl, name, W, steps, use_graph, peaks, peak_src, world)
    e2e = measure_e2e(h, wl, steps, world)
    wl = None
    release()

    extras = {}
    if not args.no_extras:
        if world > 1 and name == "cfg4" and scaling == "strong":
            # the replica case beside the sharded one: every GPU runs the whole 8192-token block
            wl = make_workload("cfg4", world, "weak")
            m = measure(h, wl, "cfg4", 3, steps, use_graph, peaks, peak_src, world, sustained_s=0)
            extras["cfg4_replicas"] = {"scaling": "weak", "rows_per_gpu": wl.tokens, "ms_per_step": m["ms_per_step"],
                                       "tokens_per_s": m["tokens_per_s"], "roofline": m["roofline"]}
            wl = None
            release()
        others = [n for n in ("cfg5", "cfg3", "cfg2", "cfg1") if n != name and (world == 1 or n in SHARDED)]
        for other in others:
            sc = "strong" if other in SHARDED else "weak"
            wl = make_workload(other, world, sc)
            m = measure(h, wl, other, 3, 5, use_graph, peaks, peak_src, world)
            rec = {"config": workload_config(other, world, sc), "dtype": wl.dtype, "cuda_graph": m["cuda_graph"],
                   "burst": {k: m[k] for k in ("ms_per_step", "steps", "tokens_per_s", "roofline")},
                   **m["sustained"]}
            if other == "cfg5" and world > 1:
                from fuseml_b200.sharding import allreduce_scalars

                s, mx = wl.scalars
                ar_ms, _ = h.timed(lambda: allreduce_scalars(total=s, maximum=mx), 200, clocks=False)
                rec["allreduce"] = {"ms_per_call": ar_ms / 200, "calls_per_step": 1, "inside_timed_region": True,
                                    "what": "NCCL all-reduce of the global sum (SUM) and amax (MAX), 4 bytes each"}
            extras[other] = rec
            wl = None
            release()
        if world == 1 and name == "cfg4":
            wl = TrainingStep()
            m = measure(h, wl, "cfg4_training_step", 3, 5, False, peaks, peak_src, world)
            extras["cfg4_training_step"] = {"what": "forward + backward of the cfg4 block, six fused GEMMs, bf16",
                                            "burst": {k: m[k] for k in ("ms_per_step", "steps", "tokens_per_s", "roofline")},
                                            **m["sustained"]}
            wl = None
            release()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cfg = workload_config(name, world, scaling)
    line = {
        "metric": "mlp_block_tokens_per_s", "value": head["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": W, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": {"cfg1": "f32"}.get(name, "bf16"), "data": "synthetic", "config": cfg,
        "runtime": {"cuda_graph": head["cuda_graph"],
                    "host_affinity": (f"rank 0 bound to the {len(numa_cores)} cores NVML reports local to its GPU"
                                      if numa_cores else "unchanged")},
        "e2e": e2e, "gpu_launches": head["gpu_launches"], "roofline": head["roofline"], "clocks": head["clocks"],
        "roofline_sustained": {**head["sustained"]["roofline"], "ms_per_step": head["sustained"]["ms_per_step"],
                               "steps": head["sustained"]["steps"], "clocks": head["sustained"]["clocks"]},
        "tflops": head["tflops"],
    }
    if extras:
        line["workloads"] = extras
    if not args.no_cpu_baseline and world == 1:
        try:
            v, desc, cores, ms, n = cpu_baseline(name, budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}
        except Exception as exc:  # the GPU numbers stand on their own
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {exc!r}"}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
