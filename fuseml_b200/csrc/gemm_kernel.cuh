// Persistent, warp-specialised GEMM + fused epilogue for sm_100a.
//
//   warp 0      TMA producer: A and B tiles -> 128B-swizzled shared-memory ring
//   warp 1      allocates TMEM; one thread issues tcgen05.mma (fp32 accumulator
//               in TMEM) and commits to the ring's "empty" barriers
//   warps 2..5  epilogue: tcgen05.ld their 32 TMEM lanes (= 32 output rows),
//               run the epilogue program in registers, store / reduce
//
// Two accumulator buffers live in TMEM, so the epilogue of tile i overlaps the
// MMAs of tile i+1.  The accumulator never goes to HBM: only the final dtype
// (or only the reductions) is written.  It replaces the Triton template of the
// reference (fuseml/codegen/kernel_generator.py:1178-1593) and its two cuBLAS Lt
// call sites (fuseml/codegen/cublas_epilogue.py:602-676).
#pragma once

#include "epilogue.cuh"
#include "gemm_params.cuh"
#include "ptx.cuh"

namespace fuseml {

// Where a bounded wait gave up (reported through the status word).
enum : int32_t {
  kWhereProducerEmpty = 0x101,
  kWhereMmaFull = 0x102,
  kWhereMmaTmemEmpty = 0x103,
  kWhereEpilogueTmemFull = 0x104,
  kWhereProducerDrain = 0x105,
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = kTileM * kSwizzleBytes;  // 16 KB
  static constexpr int kBBytes = BN * kSwizzleBytes;      // 32 KB at BN = 256
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  // after the ring: column-reduction scratch, barriers, TMEM base, abort flag
  static constexpr int kColRedBytes = kEpilogueWarps * BN * 2 * 4;
  static constexpr int kBarOffset = kRingBytes + kColRedBytes;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTotalBytes = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamicBytes = kTotalBytes + 1024;  // slack for 1024-byte alignment
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, s));
  return x;
}

// Transposing butterfly: on entry lane r holds v[c] = value(row r, column c);
// on exit lane c holds in v[0] the reduction over the 32 rows of column c.
// 31 shuffles instead of 32 x 5.
template <bool kIsMax>
__device__ __forceinline__ float warp_column_reduce(float (&v)[kChunkN], int lane) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = upper ? v[i] : v[i + s];
      const float keep = upper ? v[i + s] : v[i];
      const float got = __shfl_xor_sync(0xffffffffu, send, s);
      v[i] = kIsMax ? fmaxf(keep, got) : (keep + got);
    }
  }
  return v[0];
}

// FMT: 0 = f16, 1 = bf16, 2 = tf32 (fp32 storage).  B_MN: B tile is MN-major
// in shared memory (row-major [K,N] in global memory) instead of K-major.
template <int BN, int STAGES, int FMT, bool B_MN, bool USES_SAVED>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_epilogue_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int kElemBytes = (FMT == 2) ? 4 : 2;
  constexpr int BK = kSwizzleBytes / kElemBytes;   // 64 (16-bit) or 32 (tf32)
  constexpr int UMMA_K = 32 / kElemBytes;          // 16 or 8: 32 bytes of K per instruction
  constexpr int kKSteps = BK / UMMA_K;             // 4
  constexpr uint32_t kTmemCols = 2 * BN;           // two accumulator buffers
  static_assert(!(B_MN && FMT == 2), "MN-major B is only wired for 16-bit operands");
  static_assert(kTmemCols == 512 || kTmemCols == 256 || kTmemCols == 128, "TMEM columns: power of two");

  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle atoms are 1024 bytes: align the ring.
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  float* colred = reinterpret_cast<float*>(smem + L::kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), kEpilogueWarps);
    }
    *abort_flag = 0u;
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int32_t num_kb = p.num_kb;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int32_t t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        int32_t tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
        const int32_t m0 = tm * kTileM, n0 = tn * BN;
        for (int32_t kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kWhereProducerEmpty)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
          ptx::tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * BK, m0);
          if (!B_MN) {
            ptx::tma_load_2d(b_dst, &tmap_b, full_bar(stage), kb * BK, n0);
          } else {
            // [K,N] row-major: one box = 64 columns (128 bytes) x BK rows.
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              ptx::tma_load_2d(b_dst + j * (BK * kSwizzleBytes), &tmap_b, full_bar(stage), n0 + j * 64, kb * BK);
            }
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Giving up: let copies already in flight land before the CTA exits.
        const uint32_t pending = issued < static_cast<uint32_t>(STAGES) ? issued : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (uint32_t i = 0; i < pending; ++i) {
          if (--s < 0) { s = STAGES - 1; ph ^= 1u; }
          const uint64_t t0 = ptx::globaltimer_ns();
          while (!ptx::mbar_try_wait(full_bar(s), ph)) {
            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
              if (p.status) atomicCAS(p.status, 0, kWhereProducerDrain);
              break;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(FMT, 0u, B_MN ? 1u : 0u, kTileM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int32_t t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        if (!ptx::mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, kWhereMmaTmemEmpty)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int32_t kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, p.status, kWhereMmaFull)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const uint32_t b_addr = a_addr + L::kABytes;
          // K-major: 8-row groups 1024 bytes apart; 32 bytes of K per step.
          const uint64_t a_desc = ptx::make_smem_desc_sw128(a_addr, 16u, 1024u);
          const uint64_t b_desc = B_MN ? ptx::make_smem_desc_sw128(b_addr, BK * kSwizzleBytes, 1024u)
                                       : ptx::make_smem_desc_sw128(b_addr, 16u, 1024u);
          constexpr uint32_t kAStep = 32u >> 4;  // +32 bytes inside the swizzle row
          constexpr uint32_t kBStep = B_MN ? ((UMMA_K * kSwizzleBytes) >> 4) : (32u >> 4);
#pragma unroll
          for (int k = 0; k < kKSteps; ++k) {
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            if (FMT == 2) {
              ptx::mma_tf32_ss(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
            } else {
              ptx::mma_f16_ss(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
            }
          }
          ptx::mma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit(tmem_full_bar(acc));  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id % 4)
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool red_sum = (p.red_kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) != 0;
    const bool red_max = (p.red_kinds & FUSEML_RED_MAX) != 0;
    const bool red_any = red_sum || red_max;
    float all_sum = 0.0f, all_max = -INFINITY;  // AXIS_ALL running partials of this thread
    bool ok = true;
    for (int32_t t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      int32_t tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
      const int32_t m = tm * kTileM + quarter * 32 + lane;
      const int32_t n_tile0 = tn * BN;
      const bool row_ok = m < p.M;
      // After a failed wait the warp keeps walking its tiles without touching
      // TMEM, so that the named barriers below still see all four warps.
      if (ok && !ptx::mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag, p.status, kWhereEpilogueTmemFull)) {
        ok = false;
      }
      ptx::tc_fence_after_sync();
      float row_sum = 0.0f, row_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; ok && c < BN / kChunkN; ++c) {
        const int32_t n0 = n_tile0 + c * kChunkN;
        if (n0 >= p.N) break;  // uniform across the CTA
        uint32_t r[kChunkN];
        ptx::tmem_ld_32x32(tmem_base + lane_base + static_cast<uint32_t>(acc * BN + c * kChunkN), r);
        ptx::tmem_ld_wait();
        float v[kChunkN];
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] = __uint_as_float(r[i]);
        epi::run_program<USES_SAVED>(p, m, n0, row_ok, v);
        if (p.d != nullptr && row_ok) {
          epi::store_chunk(p.d, static_cast<int64_t>(m) * p.ldd, n0, p.N, p.out_dtype, v);
        }
        if (red_any) {
          if (p.red_axis == FUSEML_AXIS_M) {
            // one value per column: fold this warp's 32 rows, park in smem
            float vs[kChunkN], vm[kChunkN];
#pragma unroll
            for (int i = 0; i < kChunkN; ++i) {
              vs[i] = row_ok ? v[i] : 0.0f;
              vm[i] = row_ok ? v[i] : -INFINITY;
            }
            if (red_sum) {
              const float cs = warp_column_reduce<false>(vs, lane);
              colred[(quarter * 2 + 0) * BN + c * kChunkN + lane] = cs;
            }
            if (red_max) {
              const float cm = warp_column_reduce<true>(vm, lane);
              colred[(quarter * 2 + 1) * BN + c * kChunkN + lane] = cm;
            }
          } else {
#pragma unroll
            for (int i = 0; i < kChunkN; ++i) {
              const bool in = (n0 + i < p.N);
              row_sum += in ? v[i] : 0.0f;
              row_max = in ? fmaxf(row_max, v[i]) : row_max;
            }
          }
        }
      }
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && ok) ptx::mbar_arrive(tmem_empty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

      if (red_any) {
        if (p.red_axis == FUSEML_AXIS_N) {
          if (row_ok && ok) {
            const int64_t o = static_cast<int64_t>(tn) * p.M + m;
            if (red_sum) p.red_sum[o] = row_sum;
            if (red_max) p.red_max[o] = row_max;
          }
        } else if (p.red_axis == FUSEML_AXIS_ALL) {
          if (row_ok) {
            all_sum += row_sum;
            all_max = fmaxf(all_max, row_max);
          }
        } else {
          // AXIS_M: combine the four warps' column partials, one thread per column
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int j = threadIdx.x - 64; j < BN; j += kEpilogueWarps * 32) {
            const int32_t n = n_tile0 + j;
            if (n < p.N && ok) {
              const int64_t o = static_cast<int64_t>(tm) * p.N + n;
              if (red_sum) {
                p.red_sum[o] = colred[0 * BN + j] + colred[2 * BN + j] + colred[4 * BN + j] + colred[6 * BN + j];
              }
              if (red_max) {
                p.red_max[o] = fmaxf(fmaxf(colred[1 * BN + j], colred[3 * BN + j]),
                                     fmaxf(colred[5 * BN + j], colred[7 * BN + j]));
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
    if (red_any && p.red_axis == FUSEML_AXIS_ALL) {
      // one partial per CTA: warp shuffle, then the four warps through smem
      const float ws = warp_sum(all_sum);
      const float wm = warp_max(all_max);
      if (lane == 0) {
        colred[quarter * 2 + 0] = ws;
        colred[quarter * 2 + 1] = wm;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        if (red_sum) p.red_sum[blockIdx.x] = colred[0] + colred[2] + colred[4] + colred[6];
        if (red_max) p.red_max[blockIdx.x] = fmaxf(fmaxf(colred[1], colred[3]), fmaxf(colred[5], colred[7]));
      }
    }
  }

  // ------------------------------ tear-down -----------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fuseml
