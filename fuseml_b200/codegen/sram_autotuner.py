"""Analytic tile / stage chooser under the shared-memory and TMEM budgets of one SM.

The reference's ``SRAMAutotuner`` (fuseml/codegen/sram_autotuner.py:135-447) enumerated
Triton ``(BLOCK_M, BLOCK_N, BLOCK_K, num_warps, num_stages)`` tuples whose operand tiles fit
a shared-memory budget and scored them without timing.  The same names are kept, rebuilt
around what constrains a tcgen05 kernel:

* shared memory: ``stages * (BM*BK + BK*BN) * bytes`` for the TMA -> MMA ring (227 KB opt-in);
* TMEM: ``acc_buffers * BN`` fp32 columns out of 512 (two buffers let the epilogue of one
  tile overlap the MMAs of the next);
* UMMA shape: M = 128 per CTA, N a multiple of 16 up to 256, ``BK * bytes == 128`` (one swizzle row).

``get_best_config`` returns what the native router (``fuseml_sm100_plan``, the code that
decides at launch) picks for the problem under this tuner's budgets — tile, ring depth, CTA
pairs and split-K included; the functions above it are the budget arithmetic alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Generator

import torch

_DTYPE_BYTES = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.int8: 1}

SMEM_BUDGET_BYTES = 232448          # 227 KB opt-in per CTA on sm_100
TMEM_COLUMNS = 512
_FIXED_SMEM = 4 * 256 * 2 * 4 + 256 + 1024   # column-reduction scratch + barriers + alignment slack
_DEFAULT_SRAM_BUDGET_BYTES = SMEM_BUDGET_BYTES - _FIXED_SMEM

_BLOCK_M_CHOICES = (128,)
_BLOCK_N_CHOICES = (64, 128, 256)
_NUM_STAGES_CHOICES = (2, 3, 4, 5, 6, 8)
_EPILOGUE_WARPS = 4


@dataclass(frozen=True)
class TuneConfig:
    block_m: int
    block_n: int
    block_k: int
    num_warps: int
    num_stages: int
    sram_bytes: int
    tmem_cols: int = 0
    cluster: int = 1
    split_k: int = 1
    bound: str = ""          # "hbm" | "tensor" | "latency": which roofline the router expects to bind
    t_est_us: float = 0.0


def compute_sram_bytes(block_m: int, block_n: int, block_k: int, dtype_bytes: int, num_stages: int) -> int:
    """Ring footprint: one A tile and one B tile per stage."""
    return num_stages * (block_m * block_k + block_k * block_n) * dtype_bytes


def compute_tmem_cols(block_n: int, acc_buffers: int = 2) -> int:
    """fp32 accumulator columns, rounded up to the power of two the allocator hands out."""
    need = block_n * acc_buffers
    return max(32, 1 << (need - 1).bit_length())


def generate_sram_safe_configs(dtype: torch.dtype, sram_budget: int = _DEFAULT_SRAM_BUDGET_BYTES,
                               tmem_budget: int = TMEM_COLUMNS) -> Generator[TuneConfig, None, None]:
    """All configurations that fit both budgets."""
    bpe = _DTYPE_BYTES.get(dtype, 4)
    bk = 128 // bpe if bpe in (2, 4) else 64
    for bm in _BLOCK_M_CHOICES:
        for bn in _BLOCK_N_CHOICES:
            tm = compute_tmem_cols(bn)
            if tm > tmem_budget:
                continue
            for ns in _NUM_STAGES_CHOICES:
                sram = compute_sram_bytes(bm, bn, bk, bpe, ns)
                if sram <= sram_budget:
                    yield TuneConfig(bm, bn, bk, _EPILOGUE_WARPS + 2, ns, sram, tm)


class SRAMAutotuner:
    """Pick the best budget-safe configuration for an (M, N, K, dtype) problem; cached per shape."""

    def __init__(self, sram_budget: int | None = None, sm_count: int = 148,
                 tensor_tflops: float = 2250.0, hbm_gbs: float = 7700.0) -> None:
        self.sram_budget = sram_budget if sram_budget is not None else _DEFAULT_SRAM_BUDGET_BYTES
        self.sm_count = sm_count
        self.tensor_tflops = tensor_tflops
        self.hbm_gbs = hbm_gbs
        self._cache: dict[tuple, TuneConfig] = {}

    def get_best_config(self, M: int, N: int, K: int, dtype: torch.dtype = torch.bfloat16) -> TuneConfig:
        """The native router's plan for an ``M x N x K`` GEMM of ``dtype`` operands (nn.Linear
        layout) under this tuner's shared-memory budget, SM count and peaks.  Host only."""
        key = (int(M), int(N), int(K), dtype)
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        import ctypes as C

        from .. import _native as N_
        from ..kernels import dtype_code

        lib = N_.load()
        bpe = _DTYPE_BYTES.get(dtype, 4)
        code = dtype_code(dtype)
        desc = N_.GemmDesc()
        desc.M, desc.N, desc.K = int(M), int(N), int(K)
        desc.a, desc.b, desc.d = 0x1000, 0x2000, 0x3000          # layout-only query: aligned dummies
        ld = int(K) if (code == N_.F32 or (K * bpe) % 16 == 0) else (int(K) * bpe + 15) // 16 * 16 // bpe
        desc.lda, desc.b_stride_k, desc.b_stride_n, desc.ldd = ld, 1, ld, int(N)
        desc.ab_dtype = desc.out_dtype = code
        props = N_.DeviceProps()
        lib.fuseml_sm100_query(C.byref(props))                     # published B200 figures when there is no device
        props.sm_count = self.sm_count
        props.smem_per_block_optin = self.sram_budget + _FIXED_SMEM
        props.tensor_tflops, props.hbm_gbs = self.tensor_tflops, self.hbm_gbs
        plan = N_.Plan()
        rc = lib.fuseml_sm100_plan(C.byref(desc), C.byref(props), C.byref(plan))
        if rc != N_.OK:
            raise ValueError(f"the router rejects {M} x {N} x {K} {dtype}: {N_.strerror(rc)}")
        kernel_bn = 256 if plan.tile_n > 128 else 128              # the instance that runs the tile
        stage = (plan.tile_m * plan.tile_k + plan.tile_k * (kernel_bn // plan.cluster)) * (4 if code == N_.F32 else bpe)
        if plan.stages * stage > self.sram_budget:
            raise ValueError(f"no configuration fits a shared-memory budget of {self.sram_budget} bytes")
        best = TuneConfig(plan.tile_m, plan.tile_n, plan.tile_k, 2 + 8, plan.stages, plan.stages * stage,
                          plan.tmem_cols, plan.cluster, max(1, plan.split_k),
                          ("hbm", "tensor", "latency")[plan.bound], plan.t_est_us)
        self._cache[key] = best
        return best

    def clear_cache(self) -> None:
        self._cache.clear()

    @property
    def cache_size(self) -> int:
        return len(self._cache)
