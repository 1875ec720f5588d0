#!/usr/bin/env python
"""Benchmark of the fused GEMM + epilogue path on B200.

``python bench.py --gpus N --steps K --warmup W`` runs the residual Transformer-MLP
block (d_model 4096, d_intermediate 16384, 8192 tokens per GPU, bf16; synthetic
N(0,1) activations, nn.Linear-initialised weights) and prints ONE JSON line with

* ``value``      tokens/s over all GPUs, inputs resident in HBM, CUDA-event timed;
* ``e2e``        the same metric through the public call with pinned HOST buffers
                 (host->device copy of the tokens and device->host read of the result
                 inside the timed region);
* ``roofline``   the dominant kernel's achieved TFLOP/s (or GB/s) against the measured peak;
* ``cpu_baseline`` the CPU oracle (fp32 eager, what the reference executes on a CPU)
                 timed on this machine's host cores on a bounded sample.

``--impl reference`` times that CPU path alone (rank 0 only).  ``--workload`` selects
the other benchmark configurations (cfg1 small fp32 MLP, cfg2 weight-streaming GEMM,
cfg3 GEMM + row reductions, cfg5 stacked MLP with global reductions).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
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
# mean of its two launches (GEMM1 0.670 GB, GEMM2 1.751 GB: with K = 16384 the operand slabs of one
# wave of tiles do not survive in L2 until the next wave; algorithmic bytes are 0.47 GB per launch).
# cfg5 was not captured (same kernel as cfg4 at half the rows).
NCU_TRAFFIC_BYTES = {"cfg1": None, "cfg4": 1.2108e9, "cfg2": 1.501e8, "cfg3": 1.508e8, "cfg5": None}


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

    def use_graphs(self):
        """Capture the resident step in CUDA graphs where that pays (launch-bound steps)."""
        return False


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
            g = self.graphs[self.i % len(self.graphs)]
            self.i += 1
            return g()
        return self._forward(self.x, self.r)

    def use_graphs(self):
        """One captured graph per weight copy (the step is a single ~50 us kernel: without a
        graph the host's launch path is part of the measurement)."""
        from fuseml_b200.runtime import GraphedCallable

        graphs = []
        for W in self.Ws:
            self.module.W.data = W
            graphs.append(GraphedCallable(self.compiled, self.x, self.r))
        self.graphs = graphs
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
    the first Linear + GELU is one fused kernel on 3xTF32 operands, the bare second Linear has no
    epilogue to fuse and stays an ATen addmm, as in the reference)."""

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
        self.launches_per_step = 4          # fused GEMM + two operand expansions + ATen addmm
        self.gemm_launches_per_step = 1
        self.h2d_bytes = rows * d_model * 4
        self.d2h_bytes = rows * d_model * 4

    def _forward(self, x):
        with torch.no_grad():
            return self.compiled(x)

    def step(self):
        return self.graph() if self.graph is not None else self._forward(self.x)

    def use_graphs(self):
        from fuseml_b200.runtime import GraphedCallable

        self.graph = GraphedCallable(self.compiled, self.x)
        return True

    def e2e_step(self):
        self.x_in.copy_(self.x_host, non_blocking=True)
        y = self._forward(self.x_in)
        self.y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()


def make_workload(name, world, scaling):
    if name == "cfg1":
        return SmallFp32MLP()
    if name == "cfg4":
        rows = 8192 if scaling == "weak" else 8192 // world
        return MLPBlock(rows, world=world)
    if name == "cfg5":
        rows = 32768 // world if scaling == "strong" else 32768 // 8  # 4096 rows per GPU, as at 8 GPUs
        if world == 1 and scaling == "strong":
            rows = 32768
        return MLPBlock(rows, blocks=4, reductions=True, world=world)
    if name == "cfg2":
        return ActHeavyGemm()
    if name == "cfg3":
        return GemmRowReduce()
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------------------
# CPU baseline: the oracle's eager fp32 module on the host cores
# --------------------------------------------------------------------------------------

def cpu_baseline(workload_name, budget_s=20.0, steps=None, sample_rows=None):
    """Times the CPU oracle (fp32 eager module = what the reference runs on a CPU) on a
    bounded sample of the workload.  Returns (tokens_per_s, description, cores, ms_per_step, steps)."""
    from oracle import configs

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    full = dict(configs.FULL[workload_name])
    default_rows = {"cfg1": 128, "cfg4": 512, "cfg5": 128, "cfg3": 512, "cfg2": 64}[workload_name]
    rows = sample_rows or default_rows
    full["M"] = rows
    case = configs.make(workload_name, sizes=full)
    with torch.no_grad():
        case.module(*case.args)  # warm-up
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
    times.sort()
    med = times[len(times) // 2]
    desc = (f"{workload_name} at full width, {rows} of the rows per step, fp32 eager PyTorch on "
            f"{cores} threads, median of {n} steps")
    return rows / med, desc, cores, med * 1e3, n


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def samples_so_far(self):
        try:
            return sum(1 for l in open(self.path) if l.strip())
        except Exception:
            return 0

    def wait_for_samples(self, n, timeout_s=3.0):
        """nvidia-smi takes a moment to start: block (bounded) until it has written n samples."""
        t0 = time.perf_counter()
        while self.proc is not None and self.samples_so_far() < n and time.perf_counter() - t0 < timeout_s:
            time.sleep(0.02)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            rows = [l.strip().split(", ") for l in open(self.path).read().strip().splitlines() if l.strip()]
            os.unlink(self.path)
        except Exception:
            return out
        samples, mx = [], None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 7:
                continue
            try:
                clk, mx, watts = float(r[0]), float(r[1]), float(r[2])
            except ValueError:
                continue
            samples.append((clk, watts, {nm for nm, v in zip(names, r[3:7]) if v.strip().lower() == "active"}))
        if samples:
            # "under load" = samples drawing at least half of the highest power seen in the window
            p_max = max(w for _, w, _ in samples)
            loaded = [x for x in samples if x[1] >= 0.5 * p_max] or samples
            clks = sorted(c for c, _, _ in loaded)
            reasons = set().union(*[rs for _, _, rs in loaded])
            out.update(sm_mhz=clks[len(clks) // 2], sm_max_mhz=mx, reasons=sorted(reasons), samples=len(samples),
                       samples_under_load=len(loaded), power_w_max=p_max)
        return out


# --------------------------------------------------------------------------------------

# config.workload of each --workload choice (the same string in both arms)
WORKLOAD_NAMES = {"cfg1": "cfg1_fp32_mlp_small", "cfg2": "cfg2_act_heavy_gemm", "cfg3": "cfg3_gemm_row_reductions",
                  "cfg4": "cfg4_mlp_block", "cfg5": "cfg5_stacked_mlp_x4"}


def run_reference(args):
    """The reference arm: its CPU path for this workload on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    # warm-up passes are part of cpu_baseline(); `steps` timed passes over a bounded sample
    val, desc, cores, ms, n = cpu_baseline(args.workload, steps=min(steps, 20))
    line = {
        "impl": "reference", "metric": "mlp_block_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": n, "warmup": 1, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[args.workload], "note": "CPU path of the reference = eager fp32 module (its compiler returns gm.forward on a CPU)"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="do not capture launch-bound steps in CUDA graphs")
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

    from fuseml_b200 import _native, build as _build, kernels as K

    _build.build()
    _native.load()
    W = max(3, args.warmup)
    steps = max(1, args.steps)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    wl = make_workload(args.workload, world, args.scaling)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n, finish=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        if finish is not None:
            finish()          # make the timing stream wait for work enqueued on other streams
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        return float(ms.item())

    for _ in range(W):
        wl.step()
    wl.check_compiled()
    graphed = False
    if not args.no_graph:
        try:
            graphed = wl.use_graphs()
        except Exception as exc:          # capture is an optimisation, never a requirement
            print(f"[bench] CUDA graph capture failed, stepping eagerly: {exc!r}", file=sys.stderr)
            wl.graphs = None
        for _ in range(3):
            wl.step()
    if rank == 0:
        sampler.wait_for_samples(1)     # started before the workload was built; normally no wait
    launches_before = wl.fused_launches()
    total_ms = timed(wl.step, steps)
    launches_timed = wl.fused_launches() - launches_before
    if graphed:
        launches_timed = wl.gemm_launches_per_step * steps     # replays do not pass through the Python counters
    # The timed region may be shorter than one sampling period (50 ms): repeat the same step,
    # untimed, so that the window under load is at least 0.4 s.  The count is derived from the
    # all-reduced time, so every rank runs the same number of steps (and collectives).
    extra = max(0, int(400.0 / max(total_ms / steps, 1e-3)) - steps)
    for _ in range(min(extra, 20000)):
        wl.step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else {}
    if rank == 0:
        clocks["window"] = "timed region plus untimed repeats of the same step (>= 0.4 s under load)"
    status = K.device_status()
    if status != 0:
        raise SystemExit(f"device status {status:#x}: a bounded wait ran out; numbers would be meaningless")

    for _ in range(2):
        wl.e2e_step()
    wl.e2e_finish()
    e2e_ms = timed(wl.e2e_step, steps, finish=wl.e2e_finish)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_src = load_peaks()
    ms_per_step = total_ms / steps
    value = wl.tokens * world / (ms_per_step * 1e-3)
    launch_ms = ms_per_step / wl.gemm_launches_per_step  # back-to-back launches of the same kernel on one stream
    if wl.bound == "tensor":
        achieved = wl.flops_per_launch / (launch_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_kind": f"bf16_tflops_sustained, {peak_src}", "frac_of_burst_peak": achieved / peaks["bf16_tflops"]}
    else:
        achieved = wl.algo_bytes / (launch_ms * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": f"hbm_gbs, {peak_src}"}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)
    roof["kernel"] = "gemm_epilogue_kernel_v2"
    roof["launch_us"] = launch_ms * 1e3

    line = {
        "metric": "mlp_block_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "rows_per_gpu": wl.tokens, "global_rows": wl.tokens * world,
                   "l2": ("9 MB working set, resident in L2: a latency-bound parity configuration, not a roofline claim"
                          if args.workload == "cfg1" else
                          "inputs larger than L2 (weights + activations per step exceed 126 MB"
                          + ("; weight copies rotated)" if args.workload == "cfg2" else ")")),
                   "parallelism": f"rows sharded over {world} GPU(s), weights replicated",
                   "cuda_graph": bool(graphed),
                   "host_affinity": (f"rank 0 bound to the {len(numa_cores)} cores NVML reports local to its GPU"
                                     if numa_cores else "unchanged")},
        "e2e": {"value": wl.tokens * world / (e2e_ms / steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": wl.h2d_bytes * world, "d2h_bytes_per_step": wl.d2h_bytes * world,
                "ms_per_step": e2e_ms / steps},
        "gpu_launches": launches_timed + (steps if wl.launches_per_step > wl.gemm_launches_per_step else 0),
        "roofline": roof,
        "clocks": clocks,
        "tflops": wl.flops * world / (ms_per_step * 1e-3) / 1e12,
    }
    if not args.no_cpu_baseline:
        try:
            v, desc, cores, ms, n = cpu_baseline(args.workload, budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}
        except Exception as exc:  # the GPU numbers stand on their own
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {exc!r}"}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
