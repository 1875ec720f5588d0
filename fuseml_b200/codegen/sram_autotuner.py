"""Analytic tile / stage chooser under the shared-memory and TMEM budgets of one SM.

The reference's ``SRAMAutotuner`` (fuseml/codegen/sram_autotuner.py:135-447) enumerated
Triton ``(BLOCK_M, BLOCK_N, BLOCK_K, num_warps, num_stages)`` tuples whose operand tiles fit
a shared-memory budget and scored them without timing.  The same names are kept, rebuilt
around what constrains a tcgen05 kernel:

* shared memory: ``stages * (BM*BK + BK*BN) * bytes`` for the TMA -> MMA ring (227 KB opt-in);
* TMEM: ``acc_buffers * BN`` fp32 columns out of 512 (two buffers let the epilogue of one
  tile overlap the MMAs of the next);
* UMMA shape: M = 128 per CTA, N a multiple of 16 up to 256, ``BK * bytes == 128`` (one swizzle row).

``get_best_config`` scores candidates with the roofline estimate the native planner uses
(tensor time of the tiles in waves vs. HBM time); the authoritative decision at launch is
``fuseml_sm100_plan`` — this class exposes the same model to Python callers and tests.
"""
from __future__ import annotations

import math
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

    def _score_config(self, cfg: TuneConfig, M: int, N: int, K: int, bpe: int) -> float:
        """Estimated microseconds (lower is better)."""
        tiles = math.ceil(M / cfg.block_m) * math.ceil(N / cfg.block_n)
        waves = math.ceil(tiles / self.sm_count)
        k_pad = math.ceil(K / cfg.block_k) * cfg.block_k
        rate = self.tensor_tflops * 1e12 / self.sm_count * (0.5 if bpe == 4 else 1.0)
        t_tile = 2.0 * cfg.block_m * cfg.block_n * k_pad / rate * 1e6
        t_hbm = bpe * (M * K + K * N + M * N) / (self.hbm_gbs * 1e9) * 1e6
        # a ring too shallow to cover the load latency leaves the tensor pipe waiting
        depth_penalty = 1.0 + max(0, 4 - cfg.num_stages) * 0.15
        narrow_penalty = {256: 1.0, 128: 1.05, 64: 1.15}.get(cfg.block_n, 1.2)
        return max(waves * t_tile * depth_penalty * narrow_penalty, t_hbm)

    def get_best_config(self, M: int, N: int, K: int, dtype: torch.dtype = torch.bfloat16) -> TuneConfig:
        key = (int(M), int(N), int(K), dtype)
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        bpe = _DTYPE_BYTES.get(dtype, 4)
        best, best_t = None, float("inf")
        for cfg in generate_sram_safe_configs(dtype, self.sram_budget):
            if cfg.block_n == 64:
                continue  # no 64-wide kernel instance is built
            t = self._score_config(cfg, M, N, K, bpe)
            # prefer deeper rings at equal time
            if t < best_t - 1e-9 or (abs(t - best_t) <= 1e-9 and best is not None and cfg.num_stages > best.num_stages):
                best, best_t = cfg, t
        if best is None:
            raise ValueError(f"no configuration fits a shared-memory budget of {self.sram_budget} bytes")
        self._cache[key] = best
        return best

    def clear_cache(self) -> None:
        self._cache.clear()

    @property
    def cache_size(self) -> int:
        return len(self._cache)
