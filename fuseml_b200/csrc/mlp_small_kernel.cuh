// Both Linears of a small-M MLP block in one kernel: y = prog2(prog1(x W1^T) W2^T), M <= 128 rows.
//
// The intermediate h = prog1(x W1^T) never goes to global memory: every CTA owns slices of the
// intermediate dimension I; for a slice it computes h[:, slice] with the first GEMM (accumulator
// in TMEM), runs the first epilogue program (bias, GELU, ...) on it in registers, writes the
// result into shared memory in the K-major 128-byte-swizzled layout a tcgen05 A operand has, and
// multiplies it at once with W2[:, slice] into a second TMEM accumulator that collects the CTA's
// slices.  The CTA's partial y (fp32, 128 x 256) goes to the workspace in the split-K partial
// layout; splitk_finish_kernel folds the CTAs' partials in index order and runs the second
// program (bias, residual, ...).  Deterministic; no atomics.
//
//   warp 0  one thread: TMA producer.  One ring, two kinds of jobs in program order per slice:
//           K blocks of the first GEMM (x tile 128 x 128 B + W1 rows of the slice) and half K
//           blocks of the second (128 rows of W2 x 128 B; its A operand is h in shared memory)
//   warp 1  one thread: tcgen05.mma issuer for both GEMMs; allocates TMEM
//   warps 2-9  first epilogue (two warps per TMEM lane quarter, alternating 32-column chunks)
//           and the final partial store
//
// fp32 runs as 3xTF32 like the stand-alone kernel: x, W1 and W2 arrive expanded ([hi|lo|hi] and
// [hi|hi|lo] along K); h is split into hi (top 10 mantissa bits) and lo = h - hi on the fly, two
// shared-memory tiles per 32 columns, and the second GEMM runs hi*hi + lo*hi + hi*lo as three K
// blocks against the three copies of W2.
//
// Hazards that need no barrier of their own (single issuing thread, tcgen05.commit covers every
// MMA issued before it): the first GEMM of slice s+1 is issued after the second GEMM of slice s,
// which waited for the epilogue to have read the whole first accumulator; and the epilogue of
// slice s+1 starts after a commit that also covers the MMAs that read the h tiles of slice s.
//
// The reference runs the two Linears as two separately generated kernels with h in HBM between
// them (benchmarks/bench_mlp_block.py:160-182; fuseml/codegen/kernel_launcher.py:640-821).
#pragma once

#include "epilogue.cuh"
#include "gemm_params.cuh"
#include "ptx.cuh"

namespace fuseml {
namespace mlp {

constexpr int kABytes = 128 * 128;            // x tile / h tile / half a W2 tile: 128 rows x 128 bytes of K
constexpr int kHTiles = 4;                     // h tiles of 128 rows x 128 bytes
constexpr int kEpiWarps = 8;                  // two per TMEM lane quarter, alternating 32-column chunks
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr uint32_t kAcc2Col = 0;               // second accumulator: TMEM columns [0, 256)
constexpr uint32_t kAcc1Col = 256;             // first accumulator: TMEM columns [256, 256 + bi)

// Shared memory per operand format.  A ring stage holds one K block of the first GEMM (the x tile,
// 16 KB, and the slice's rows of W1: at most 64 rows for tf32, 128 for 16-bit operands) or one
// half K block of the second (128 rows of W2, 16 KB, at the stage base).  The first GEMM's K loop is
// a chain of load latencies (48 K blocks for the fp32 configuration), so the ring is as deep as
// shared memory allows: six stages of 24 KB for tf32, four of 32 KB for 16-bit operands.
template <bool TF32>
struct Layout {
  static constexpr int kStages = TF32 ? 6 : 4;
  static constexpr int kStageBytes = kABytes + (TF32 ? 64 : 128) * 128;
  static constexpr int kHOffset = kStages * kStageBytes;
  static constexpr int kBarOffset = kHOffset + kHTiles * kABytes;
  static constexpr int kNumBars = 2 * kStages + 3;      // ring full / empty, acc1 full, h full, acc2 full
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

enum : int32_t {
  kWhereMlpProducer = 0x301,
  kWhereMlpMmaFull = 0x302,
  kWhereMlpMmaH = 0x303,
  kWhereMlpEpiAcc1 = 0x304,
  kWhereMlpEpiAcc2 = 0x305,
};

struct MlpParams {
  int32_t M, I, D_out;
  int32_t fmt;          // 0 f16, 1 bf16, 2 tf32 (operands expanded along K)
  int32_t bi;           // slice width: columns of I per slice (16-bit: 64 or 128; tf32: 32 or 64)
  int32_t num_slices;   // I / bi
  int32_t groups;       // CTAs sharing one 256-column chunk of the output; CTA g takes slices g, g + groups, ...
  int32_t n_dchunks;    // ceil(D_out / 256)
  int32_t kb1;          // K blocks of the first GEMM (128 bytes of K each, expansion included)
  int32_t out16;        // 16-bit h: 0 = bf16, 1 = f16
  float* split_ws;      // [groups][n_dchunks][128 x 256] fp32 partial tiles, piece-major
  int32_t* status;
  uint32_t wait_limit_us;
};

// prog1 is a GemmParams of which only the program (n_ops, ops, operands) and N (= I) are used.
template <bool TF32>
__global__ void __launch_bounds__(kThreads, 1)
mlp_small_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w1,
                 const __grid_constant__ CUtensorMap tmap_w2, const __grid_constant__ MlpParams q,
                 const __grid_constant__ GemmParams prog1) {
  using L = Layout<TF32>;
  constexpr int kStages = L::kStages;
  constexpr int kStageBytes = L::kStageBytes;
  constexpr int kHOffset = L::kHOffset;
  constexpr int kBarOffset = L::kBarOffset;
  constexpr int kNumBars = L::kNumBars;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  const uint32_t acc1_full = bar_base + 8u * (2 * kStages);
  const uint32_t h_full = bar_base + 8u * (2 * kStages + 1);
  const uint32_t acc2_full = bar_base + 8u * (2 * kStages + 2);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOffset + kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool tf32 = TF32;
  constexpr int32_t bk = tf32 ? 32 : 64;             // elements per 128-byte row
  const int32_t sub = q.bi / bk;                     // 128-byte column blocks of h per slice
  const int32_t n2 = sub * (tf32 ? 3 : 1) * 2;       // jobs of the second GEMM per slice: K blocks x two 128-row halves of W2
  const int32_t group = static_cast<int32_t>(blockIdx.x) % q.groups;
  const int32_t dchunk = static_cast<int32_t>(blockIdx.x) / q.groups;
  const int32_t d0 = dchunk * 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
    ptx::mbar_init(acc1_full, 1);
    ptx::mbar_init(h_full, kEpiWarps);  // one arrival per epilogue warp
    ptx::mbar_init(acc2_full, 1);
    abort_flag[0] = 0u;
    abort_flag[1] = q.wait_limit_us;
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w1);
    ptx::prefetch_tensormap(&tmap_w2);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int32_t s = group; s < q.num_slices && ok; s += q.groups) {
        for (int32_t job = 0; job < q.kb1 + n2; ++job) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, q.status, kWhereMlpProducer)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          if (job < q.kb1) {
            // first GEMM: x[:, K block] and the slice's rows of W1
            ptx::mbar_arrive_expect_tx(full_bar(stage), kABytes + q.bi * 128);
            ptx::tma_load_2d(a_dst, &tmap_x, full_bar(stage), job * bk, 0);
            ptx::tma_load_2d(b_dst, &tmap_w1, full_bar(stage), job * bk, s * q.bi);
          } else {
            // second GEMM: 128 rows of W2 (half of the output chunk), the slice's columns (for
            // tf32: copy j of the expansion), at the stage base
            const int32_t r = (job - q.kb1) >> 1, half = (job - q.kb1) & 1;
            const int32_t t = tf32 ? r / 3 : r, j = tf32 ? r % 3 : 0;
            ptx::mbar_arrive_expect_tx(full_bar(stage), kABytes);
            ptx::tma_load_2d(a_dst, &tmap_w2, full_bar(stage), j * q.I + s * q.bi + t * bk, d0 + half * 128);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------------
    if (ptx::elect_one()) {
      const uint32_t fmt = static_cast<uint32_t>(q.fmt);
      const uint32_t idesc1 = ptx::make_idesc(fmt, 0u, 0u, 128, static_cast<uint32_t>(q.bi));
      const uint32_t idesc2 = ptx::make_idesc(fmt, 0u, 0u, 128, 128u);
      const uint64_t a_desc0 = ptx::make_smem_desc_sw128(smem_base, 16u, 1024u);
      const uint64_t b_desc0 = ptx::make_smem_desc_sw128(smem_base + kABytes, 16u, 1024u);
      const uint64_t h_desc0 = ptx::make_smem_desc_sw128(smem_base + kHOffset, 16u, 1024u);
      int stage = 0;
      uint32_t phase = 0, h_phase = 0;
      bool ok = true, any = false;
      bool first2[2] = {true, true};
      auto issue4 = [&](uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool fresh) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t accumulate = (!fresh || k > 0) ? 1u : 0u;
          if constexpr (tf32) ptx::mma_tf32_ss(d_tmem, a_desc + k * 2, b_desc + k * 2, idesc, accumulate);
          else ptx::mma_f16_ss(d_tmem, a_desc + k * 2, b_desc + k * 2, idesc, accumulate);
        }
      };
      for (int32_t s = group; s < q.num_slices && ok; s += q.groups) {
        any = true;
        for (int32_t kb = 0; kb < q.kb1; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, q.status, kWhereMlpMmaFull)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint64_t off = static_cast<uint64_t>(stage) * (kStageBytes >> 4);
          issue4(tmem_base + kAcc1Col, a_desc0 + off, b_desc0 + off, idesc1, kb == 0);
          ptx::mma_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit(acc1_full);
        // h of this slice: written by the epilogue warps into the h tiles
        if (!ptx::mbar_wait(h_full, h_phase, abort_flag, q.status, kWhereMlpMmaH)) { ok = false; break; }
        h_phase ^= 1u;
        ptx::tc_fence_after_sync();
        for (int32_t job = 0; job < n2; ++job) {
          if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, q.status, kWhereMlpMmaFull)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          // tf32: K block r = 3 t + j multiplies [hi | lo | hi][j] of h column block t with copy j of W2
          const int32_t r = job >> 1, half = job & 1;
          const int32_t t = tf32 ? r / 3 : r, j = tf32 ? r % 3 : 0;
          const int32_t tile = tf32 ? (2 * t + (j == 1 ? 1 : 0)) : t;
          const uint64_t off = static_cast<uint64_t>(stage) * (kStageBytes >> 4);
          issue4(tmem_base + kAcc2Col + static_cast<uint32_t>(half * 128), h_desc0 + static_cast<uint64_t>(tile) * (kABytes >> 4),
                 a_desc0 + off, idesc2, first2[half]);
          first2[half] = false;
          ptx::mma_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (ok && any) ptx::mma_commit(acc2_full);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue warps -------------------------------------------
    const int quarter = warp & 3;                         // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;                     // which of the quarter's two warps
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_ok = row < q.M;
    uint32_t acc1_phase = 0;
    bool ok = true, any = false;
    uint8_t* h_base = smem + kHOffset;
    for (int32_t s = group; s < q.num_slices; s += q.groups) {
      any = true;
      if (ok && !ptx::mbar_wait(acc1_full, acc1_phase, abort_flag, q.status, kWhereMlpEpiAcc1, true)) ok = false;
      acc1_phase ^= 1u;
      if (!ok) continue;
      ptx::tc_fence_after_sync();
      for (int32_t c = half; c < q.bi / 32; c += 2) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + lane_base + kAcc1Col + static_cast<uint32_t>(c * 32), r);
        ptx::tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        const int32_t n0 = s * q.bi + c * 32;               // column of I
        epi::run_program<epi::kProgGeneric, 32>(prog1, row, n0, row_ok, v, nullptr, 0);
        if (tf32) {
          // one 128-byte row of the hi tile and of the lo tile of column block c
          uint8_t* hi_row = h_base + (2 * c) * kABytes + row * 128;
          uint8_t* lo_row = hi_row + kABytes;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              hi[e] = __uint_as_float(__float_as_uint(v[4 * j + e]) & 0xffffe000u);
              lo[e] = v[4 * j + e] - hi[e];
            }
            const int piece = (j ^ (row & 7)) << 4;
            *reinterpret_cast<float4*>(hi_row + piece) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4*>(lo_row + piece) = make_float4(lo[0], lo[1], lo[2], lo[3]);
          }
        } else {
          // 32 columns = 64 bytes = four 16-byte pieces of the row of tile c / 2
          uint8_t* h_row = h_base + (c >> 1) * kABytes + row * 128;
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (q.out16 == 0) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              packed[i] = *reinterpret_cast<const uint32_t*>(&hh);
            } else {
              const __half2 hh = __floats2half2_rn(fminf(fmaxf(v[2 * i], -65504.0f), 65504.0f),
                                                   fminf(fmaxf(v[2 * i + 1], -65504.0f), 65504.0f));
              packed[i] = *reinterpret_cast<const uint32_t*>(&hh);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int piece = (((c & 1) * 4 + j) ^ (row & 7)) << 4;
            *reinterpret_cast<uint4*>(h_row + piece) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          }
        }
      }
      // publish the tiles to the tensor core (async proxy) and hand the slice to the MMA thread
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(h_full);
    }
    // the CTA's partial y: raw fp32 accumulator to the workspace, [group][chunk][column / 4][row][4]
    if (any && ok && ptx::mbar_wait(acc2_full, 0u, abort_flag, q.status, kWhereMlpEpiAcc2, true)) {
      ptx::tc_fence_after_sync();
      float4* tile = reinterpret_cast<float4*>(q.split_ws + (static_cast<int64_t>(group) * q.n_dchunks + dchunk) * (128 * 256));
      for (int32_t c = half; c < 256 / 32; c += 2) {
        if (d0 + c * 32 >= q.D_out) break;
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + lane_base + kAcc2Col + static_cast<uint32_t>(c * 32), r);
        ptx::tmem_ld_wait();
        float4* dst = tile + static_cast<int64_t>(c) * 8 * 128 + row;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i * 128] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                     __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
      }
    }
  }

  // ------------------------------ tear-down -------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mlp
}  // namespace fuseml
