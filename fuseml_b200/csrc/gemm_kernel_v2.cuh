// Persistent, warp-specialised GEMM + fused epilogue for sm_100a, one CTA or a CTA pair per tile.
//
//   warp 0      TMA producer: A and B tiles -> 128B-swizzled shared-memory ring
//   warp 1      allocates TMEM; one thread (of the pair's leader CTA) issues tcgen05.mma with
//               the fp32 accumulator in TMEM and frees ring stages with tcgen05.commit
//   warps 2..   epilogue (EW = 8 warps: two per TMEM lane quarter on alternating 32-column
//               chunks; EW = 16: four per quarter on 16-column chunks): tcgen05.ld, epilogue
//               program in registers, 16-byte stores / reductions.  In launches where no CTA
//               gets a second tile (EW = 16) the residual and output tiles move by TMA through
//               the drained operand ring instead of row-per-thread global accesses.
//
// CG = 1: the CTA computes a 128 x BN tile.  CG = 2 (cluster of two CTAs, cta_group::2): the
// pair computes 256 x BN; each CTA loads its own 128 rows of A and its own BN/2 columns of B,
// the MMA reads B from both CTAs' shared memory, so every SM ingests a third less operand data
// per flop.  No TMA multicast is used: each CTA fetches only what it alone needs.
// Two accumulator buffers live in TMEM, so the epilogue of tile i overlaps the MMAs of tile
// i+1.  Replaces the Triton template of the reference (fuseml/codegen/kernel_generator.py:
// 1178-1593) and its cuBLAS Lt call sites (fuseml/codegen/cublas_epilogue.py:602-676).
#pragma once

#include <type_traits>

#include "epilogue.cuh"
#include "gemm_params.cuh"
#include "ptx.cuh"

namespace fuseml {
namespace v2 {

// Epilogue warps per CTA: 8 (two per TMEM lane quarter, 32-column chunks) or 16 (four per
// quarter, 16-column chunks: half the registers per thread, twice the warps to hide the latency
// of an epilogue that nothing overlaps - a CTA's only tile).
constexpr int threads_for(int epi_warps) { return 64 + epi_warps * 32; }   // 320 or 576

enum : int32_t {
  kWhereProducerEmpty = 0x201,
  kWhereMmaFull = 0x202,
  kWhereMmaTmemEmpty = 0x203,
  kWhereEpilogueTmemFull = 0x204,
  kWhereProducerDrain = 0x205,
  kWhereEpilogueTileIn = 0x206,
  kWhereStoreBox = 0x207,
  kWhereStreamKPart = 0x208,
};

// Optional stall counters (diagnostic builds only, -DFUSEML_STALL_COUNTERS): per CTA
//   [0] MMA thread: cycles from first to last tile   [1] ... waiting for operands (full barriers)
//   [2] ... waiting for a free accumulator buffer     [3] epilogue warp 2: waiting for the accumulator
//   [4] epilogue warp 2: working                       [5] producer: waiting for a free ring stage
//   [6] wall clock (ns) at kernel entry                [7] wall clock (ns) just before the CTA exits
//   [8] ... after set-up (barriers, TMEM, cluster sync) [9] ... when the MMA thread has issued everything
//   [10] ... when epilogue warp 2 is done               [11] ... after the tear-down barriers
//   [12..15] epilogue warp 2, cycles: TMEM load | epilogue program | store / tile write | waiting for K-split parts
#ifdef FUSEML_STALL_COUNTERS
__device__ unsigned long long g_stall[1024][16];
#define FUSEML_STALL_T0() const long long stall_t0 = clock64()
#define FUSEML_STALL_ADD(var) var += clock64() - stall_t0
#else
#define FUSEML_STALL_T0() do {} while (0)
#define FUSEML_STALL_ADD(var) do {} while (0)
#endif

template <int BN, int STAGES, int CG>
struct Smem {
  static constexpr int kABytes = kTileM * kSwizzleBytes;          // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / CG) * kSwizzleBytes;       // this CTA's share of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kColRedBytes = 4 * 2 * BN * 4;             // [quarter][sum|max][BN]
  static constexpr int kStagedBytes = 2 * 2 * BN * 4;             // [acc buffer][row vector][BN] fp32
  static constexpr int kBarOffset = kRingBytes + kColRedBytes + kStagedBytes;
  static constexpr int kNumBars = 2 * STAGES + 5 + 4;             // ring full/empty, TMEM full/empty x 2, tile in, 4 output boxes
  static constexpr int kTotalBytes = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamicBytes = kTotalBytes + 1024;
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

// Transposing butterfly: lane r holds v[c] = value(row r, column c) on entry; lane c holds the
// reduction over the 32 rows of column c in v[0] on exit (31 shuffles).
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

// Ask L2 for the operand bytes one thread's row of the tile will read in the epilogue, long
// before the accumulator is ready (the epilogue warps are idle during the K loop).
__device__ __forceinline__ void prefetch_operands(const GemmParams& p, int64_t m, int32_t n_tile0, int32_t bn,
                                                  bool row_ok, int lane) {
  for (int op = 0; op < p.n_ops; ++op) {
    const int32_t code = p.ops[op].opcode;
    if (code != FUSEML_OP_ADD_T && code != FUSEML_OP_MUL_T && code != FUSEML_OP_SUB_T && code != FUSEML_OP_RSUB_T &&
        code != FUSEML_OP_GELU_ERF_BWD_T)
      continue;
    const EpiOperand& o = p.operands[p.ops[op].slot];
    if (o.stride_n != 1) continue;
    const int eb = o.dtype == FUSEML_F32 ? 4 : 2;
    const int32_t cols = (n_tile0 + bn <= p.N) ? bn : (p.N - n_tile0);
    if (cols <= 0) continue;
    if (o.stride_m == 0) {
      // one row shared by everybody: a few lanes cover it
      const char* base = reinterpret_cast<const char*>(o.ptr) + static_cast<int64_t>(n_tile0) * eb;
      if (lane * 128 < cols * eb) ptx::prefetch_l2(base + lane * 128);
    } else if (row_ok) {
      const char* base = reinterpret_cast<const char*>(o.ptr) + (m * o.stride_m + n_tile0) * eb;
      for (int b = 0; b < cols * eb; b += 128) ptx::prefetch_l2(base + b);
    }
  }
}

// LAYOUT: 0 = A and B K-major (activations x nn.Linear weight view), 1 = B row-major [K,N]
// (MN-major tiles), 2 = A stored [K,M] as well (both MN-major: weight gradients, dY^T @ X).  PROG:
// how the epilogue program runs (epi::kProg*).  CG: CTAs per tile (1 or 2).  EW: epilogue warps.
// The operand format (f16 / bf16 / tf32) is a run-time value (GemmParams::fmt): it only selects
// the instruction descriptor, the MMA kind and the K extent of a stage.
template <int BN, int STAGES, int LAYOUT, int PROG, int CG, int EW>
__global__ void __launch_bounds__(threads_for(EW), 1)
gemm_epilogue_kernel_v2(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_r, const __grid_constant__ CUtensorMap tmap_d,
                        const __grid_constant__ GemmParams p) {
  using L = Smem<BN, STAGES, CG>;
  constexpr bool B_MN = LAYOUT >= 1;
  constexpr bool A_MN = LAYOUT == 2;
  // the K-split last wave exists for CTA pairs with eight epilogue warps whose program keeps no
  // second value register (the host never asks the other instances for it: their registers
  // have no room for the walk's extra state)
  constexpr bool kStreamK = (CG == 2 && EW == 8 && PROG != epi::kProgGenericSaved);
  const bool tf32 = p.fmt == 2;
  const int32_t BK = tf32 ? 32 : 64;             // elements per 128-byte stage row
  constexpr int kKSteps = 4;                      // MMAs per stage: 32 bytes of K each (16 x 16-bit or 8 x tf32)
  constexpr int BN_CTA = BN / CG;                 // most B columns one CTA loads (sizes shared memory)
  constexpr uint32_t kTmemCols = 2 * BN;
  static_assert(EW == 8 || EW == 16, "two or four epilogue warps per TMEM lane quarter");
  static_assert(EW == 8 || L::kStageBytes % (kTileM * kSwizzleBytes) == 0, "tile I/O packs whole boxes into ring stages");
  constexpr uint32_t kMnBoxBytes = 64 * kSwizzleBytes;   // MN-major B (16-bit operands only): one 64 k x 64 n box
  constexpr int kEpiWarps = EW;
  constexpr int kEpiSplit = EW / 4;             // warps sharing one TMEM lane quarter
  constexpr int CH = (EW == 16) ? 16 : 32;      // accumulator columns per chunk
  static_assert(CG == 1 || CG == 2, "one CTA or a CTA pair");
  static_assert(!B_MN || (BN_CTA % 64 == 0), "MN-major B is loaded in 64-column boxes");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tile_in_bar = bar_base + 8u * (2 * STAGES + 4);
  auto box_bar = [&](int j) { return bar_base + 8u * (2 * STAGES + 5 + j); };   // output box j written by all epilogue warps
  // tile I/O through the drained ring (sixteen-warp instance only; see GemmParams::io_flags)
  // (only when every tile walker really has at most one tile: the launch may have been given
  // fewer CTA pairs than the host asked for)
  const bool lone_tile = p.num_tiles <= static_cast<int32_t>(gridDim.x) / CG;
  const bool tile_in = (EW == 16) && lone_tile && (p.io_flags & 1) != 0;
  const bool tile_out = (EW == 16) && lone_tile && (p.io_flags & 2) != 0;
  constexpr int kBoxBytes = kTileM * kSwizzleBytes;   // 128 rows x 64 16-bit columns
  constexpr int kBoxesPerStage = L::kStageBytes / kBoxBytes;   // 2 (pairs, 128-wide) or 3 (256-wide single CTA)
  const int32_t tile_boxes = p.bn / 64;               // boxes of this CTA's tile (tile I/O needs bn % 64 == 0)
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  float* colred = reinterpret_cast<float*>(smem + L::kRingBytes);
  float* staged_base = reinterpret_cast<float*>(smem + L::kRingBytes + L::kColRedBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef FUSEML_STALL_COUNTERS
  if (threadIdx.x == 0) g_stall[blockIdx.x][6] = ptx::globaltimer_ns();
#endif
  const uint32_t cta_rank = (CG == 2) ? ptx::cluster_ctarank() : 0u;
  const bool is_leader = (cta_rank == 0);
  const int32_t unit = blockIdx.x / CG;            // tile walker id (CTA or pair)
  const int32_t num_units = gridDim.x / CG;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);    // leader: one expect_tx arrival covering both CTAs' bytes
      ptx::mbar_init(empty_bar(s), 1);   // one commit arrival (multicast to both CTAs when paired)
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), kEpiWarps * CG);   // leader collects both CTAs' epilogue warps
    }
    ptx::mbar_init(tile_in_bar, 1);
    for (int j = 0; j < 4; ++j) ptx::mbar_init(box_bar(j), kEpiWarps);
    abort_flag[0] = 0u;
    abort_flag[1] = p.wait_limit_us;
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    if (tile_in) ptx::prefetch_tensormap(&tmap_r);
    if (tile_out) ptx::prefetch_tensormap(&tmap_d);
  }
  if (warp == 1) {
    if (CG == 2) {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) {   // the peer's barriers must exist before anything signals them
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after_sync();
  // Everything above touched only this CTA's shared memory, TMEM and the kernel parameters; it
  // may overlap the tail of the previous kernel of the stream.  From here on global memory is
  // read and written: wait for the previous kernel first.
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const uint32_t tmem_base = *tmem_base_slot;
#ifdef FUSEML_STALL_COUNTERS
  if (threadIdx.x == 32) g_stall[blockIdx.x][8] = ptx::globaltimer_ns();
#endif
  // Every role walks the same list of work items (WorkWalk): whole tiles in waves, then (stream-K
  // launches) a range of the K blocks of the last, ragged wave's tiles; or the single
  // (tile, K slice) item of a split-K launch.
  const bool splitk = p.split_k > 1;
  const int32_t k_slice = splitk ? unit / p.num_tiles : 0;
  // The tile width is a run-time value (a multiple of 32, at most BN): the router may shave it
  // so that the number of tiles fits the number of CTA pairs without a ragged last wave.
  const int32_t bn = p.bn;
  const int32_t bn_cta = bn / CG;
  const int32_t n_boxes = (bn_cta + 63) / 64;                          // MN-major: 64-column TMA boxes
  const uint32_t stage_tx = L::kABytes + (B_MN ? n_boxes * kMnBoxBytes : bn_cta * kSwizzleBytes);

  if (warp == 0) {
    // ------------------------------ TMA producer (every CTA) -----------------------------
    if (ptx::elect_one()) {
      int stage = 0;
      uint32_t phase = 0, issued = 0;
      bool ok = true;
      const uint64_t pol_stream = ptx::policy_evict_first();
      const uint64_t pol_keep = ptx::policy_evict_last();
      const uint64_t pol_normal = ptx::policy_evict_normal();
      long long st_empty = 0;
      WorkWalk walk;
      walk.template init<kStreamK>(p, unit, num_units);
      WorkItem w;
      while (ok && walk.next(&w)) {
        const int32_t kb_begin = w.kb0, kb_end = w.kb1;
        int32_t tm, tn;
        tile_coords(w.tile, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
        const int32_t m0 = tm * (kTileM * CG) + static_cast<int32_t>(cta_rank) * kTileM;
        const int32_t n0 = tn * bn + static_cast<int32_t>(cta_rank) * bn_cta;
        for (int32_t kb = kb_begin; kb < kb_end; ++kb) {
          FUSEML_STALL_T0();
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kWhereProducerEmpty)) {
            ok = false;
            break;
          }
          FUSEML_STALL_ADD(st_empty);
          // host-injected failure (diagnostics): the last K block of the last tile is never
          // loaded and its barrier never armed; nothing is in flight when the MMA thread gives up
          if (p.drop_last_load && kb == kb_end - 1 && w.last) break;
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          // one load helper for both modes: completion bytes go to `bar` (for a pair: the
          // leader's barrier, addressed through the cluster window)
          const uint32_t bar = (CG == 2) ? ptx::mapa(full_bar(stage), 0) : full_bar(stage);
          if (CG == 1 || is_leader) ptx::mbar_arrive_expect_tx(full_bar(stage), CG * stage_tx);
          // L2 policy per operand: 0 = default (plain load), 1 = evict-first (pure stream),
          // 2 = evict-last (keep resident).  The loads are spelled out per case: routing them
          // through a helper with run-time policy and box-count tests made the issue of the four
          // MN-major boxes slow enough to starve the tensor core.
          const uint64_t pol_a = p.a_stream == 1 ? pol_stream : (p.a_stream == 2 ? pol_keep : pol_normal);
          const uint64_t pol_b = p.b_stream == 1 ? pol_stream : pol_keep;
          if (A_MN) {
            // A stored [K, M]: two boxes of 64 k x 64 m (the same shape as an MN-major B box)
#pragma unroll
            for (int j = 0; j < kTileM / 64; ++j) {
              if (CG == 1) ptx::tma_load_2d_hint(a_dst + j * kMnBoxBytes, &tmap_a, bar, m0 + j * 64, kb * BK, pol_a);
              else ptx::tma_load_2d_pair_hint(a_dst + j * kMnBoxBytes, &tmap_a, bar, m0 + j * 64, kb * BK, pol_a);
            }
          }
          if (CG == 1) {
            if (A_MN) {}
            else if (p.a_stream == 0) ptx::tma_load_2d(a_dst, &tmap_a, bar, kb * BK, m0);
            else ptx::tma_load_2d_hint(a_dst, &tmap_a, bar, kb * BK, m0, pol_a);
            if (!B_MN) {
              if (p.b_stream == 0) ptx::tma_load_2d(b_dst, &tmap_b, bar, kb * BK, n0);
              else ptx::tma_load_2d_hint(b_dst, &tmap_b, bar, kb * BK, n0, pol_b);
            } else if (p.b_stream == 0 && n_boxes == BN_CTA / 64) {
#pragma unroll
              for (int j = 0; j < BN_CTA / 64; ++j)
                ptx::tma_load_2d(b_dst + j * kMnBoxBytes, &tmap_b, bar, n0 + j * 64, kb * BK);
            } else {
              for (int j = 0; j < n_boxes; ++j)
                ptx::tma_load_2d_hint(b_dst + j * kMnBoxBytes, &tmap_b, bar, n0 + j * 64, kb * BK, pol_b);
            }
          } else {
            if (A_MN) {}
            else if (p.a_stream == 0) ptx::tma_load_2d_pair(a_dst, &tmap_a, bar, kb * BK, m0);
            else ptx::tma_load_2d_pair_hint(a_dst, &tmap_a, bar, kb * BK, m0, pol_a);
            if (!B_MN) {
              if (p.b_stream == 0) ptx::tma_load_2d_pair(b_dst, &tmap_b, bar, kb * BK, n0);
              else ptx::tma_load_2d_pair_hint(b_dst, &tmap_b, bar, kb * BK, n0, pol_b);
            } else if (p.b_stream == 0 && n_boxes == BN_CTA / 64) {
#pragma unroll
              for (int j = 0; j < BN_CTA / 64; ++j)
                ptx::tma_load_2d_pair(b_dst + j * kMnBoxBytes, &tmap_b, bar, n0 + j * 64, kb * BK);
            } else {
              for (int j = 0; j < n_boxes; ++j)
                ptx::tma_load_2d_pair_hint(b_dst + j * kMnBoxBytes, &tmap_b, bar, n0 + j * 64, kb * BK, pol_b);
            }
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (EW == 16 && tile_in && ok && unit < p.num_tiles) {
        // This CTA's only tile: as the last MMAs drain the ring, bring the tile of the matrix
        // operand (residual) into the freed stages: a box of 128 rows x 64 columns is 16 KB, a
        // stage holds two or three of them, the tile has bn / 64.
        int32_t tm, tn;
        tile_coords(unit, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
        const int32_t m0 = tm * (kTileM * CG) + static_cast<int32_t>(cta_rank) * kTileM;
        const int32_t n_tile0 = tn * bn;
        ptx::mbar_arrive_expect_tx(tile_in_bar, static_cast<uint32_t>(tile_boxes) * kBoxBytes);
        for (int i = 0; i < STAGES && ok; ++i) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kWhereProducerEmpty)) {
            ok = false;
            break;
          }
          // the boxes that live in this stage's memory (box j sits at j * 16 KB from the ring base)
          for (int j = stage * kBoxesPerStage; j < (stage + 1) * kBoxesPerStage && j < tile_boxes; ++j)
            ptx::tma_load_2d(smem_base + j * kBoxBytes, &tmap_r, tile_in_bar, n_tile0 + j * 64, m0);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (EW == 16 && tile_out && ok && unit < p.num_tiles) {
        // This CTA's only tile, on its way out: every 64-column box of the output tile is written
        // to the drained ring by all epilogue warps (one arrival each on the box's barrier); this
        // thread, idle by now, stores each box as soon as it is complete, so that only the last
        // box's store is left when the epilogue warps finish and nobody waits at a CTA barrier.
        int32_t tm, tn;
        tile_coords(unit, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
        const int32_t row0 = (tm * CG + static_cast<int32_t>(cta_rank)) * kTileM;
        const int32_t n_tile0 = tn * bn;
        for (int j = 0; j < tile_boxes; ++j) {
          // (after a failed wait elsewhere the epilogue warps still arrive, without having
          // written anything: store nothing then)
          if (!ptx::mbar_wait(box_bar(j), 0u, abort_flag, p.status, kWhereStoreBox, true) || *abort_flag) {
            ok = false;
            break;
          }
          if (n_tile0 + j * 64 < p.N) {
            ptx::tma_store_2d(&tmap_d, smem_base + j * kBoxBytes, n_tile0 + j * 64, row0);
            ptx::bulk_commit_group();
          }
        }
        ptx::bulk_wait_read_all();   // the boxes must stay in shared memory until the copies have read them
      }
#ifdef FUSEML_STALL_COUNTERS
      g_stall[blockIdx.x][5] = st_empty;
#else
      (void)st_empty;
#endif
      if (!ok && is_leader) {
        // Giving up: let copies already in flight land before the CTA exits (a pair's bytes are all
        // counted on the leader's barriers, and the partner cannot leave before the final cluster
        // barrier, so the leader's wait covers both).
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
    // ------------------------------ MMA issuer (leader CTA only) ---------------------------
    // The loop body exists twice, once per MMA kind: a test of the format inside the K loop
    // costs the single issuing thread about 3 % of a tensor-bound GEMM.
    auto mma_role = [&](auto tf32_tag) {
      constexpr bool kTf32 = decltype(tf32_tag)::value;
      const uint32_t idesc = ptx::make_idesc(static_cast<uint32_t>(p.fmt), A_MN ? 1u : 0u, B_MN ? 1u : 0u, kTileM * CG, static_cast<uint32_t>(bn));
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long st_full = 0, st_tmem = 0;
      bool ready = false;   // the next ring stage is already known to be full
      const uint64_t a_desc0 = A_MN ? ptx::make_smem_desc_sw128(smem_base, kMnBoxBytes, 1024u)
                                    : ptx::make_smem_desc_sw128(smem_base, 16u, 1024u);
      const uint64_t b_desc0 = B_MN ? ptx::make_smem_desc_sw128(smem_base + L::kABytes, kMnBoxBytes, 1024u)
                                    : ptx::make_smem_desc_sw128(smem_base + L::kABytes, 16u, 1024u);
#ifdef FUSEML_STALL_COUNTERS
      const long long st_begin = clock64();
#endif
      WorkWalk walk;
      walk.template init<kStreamK>(p, unit, num_units);
      WorkItem w;
      while (ok && walk.next(&w)) {
        const int32_t kb_begin = w.kb0, kb_end = w.kb1;
        {
          FUSEML_STALL_T0();
          if (!ptx::mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, kWhereMmaTmemEmpty)) {
            ok = false;
            break;
          }
          FUSEML_STALL_ADD(st_tmem);
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int32_t kb = kb_begin; kb < kb_end; ++kb) {
          // `ready` carries the result of a probe issued just before the previous K block's MMAs:
          // the barrier's round trip overlaps their issue instead of preceding the next ones
          if (!ready) {
            FUSEML_STALL_T0();
            if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, p.status, kWhereMmaFull)) {
              ok = false;
              break;
            }
            FUSEML_STALL_ADD(st_full);
          }
          ptx::tc_fence_after_sync();
          const int next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
          const uint32_t next_phase = (stage + 1 == STAGES) ? (phase ^ 1u) : phase;
          const bool next_ready = ptx::mbar_try_wait(full_bar(next_stage), next_phase);
          // the start-address field (address >> 4, 14 bits) is the only part of a descriptor
          // that changes from stage to stage
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage) * (L::kStageBytes >> 4);
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage) * (L::kStageBytes >> 4);
          constexpr uint32_t kAStep = A_MN ? ((16 * kSwizzleBytes) >> 4) : (32u >> 4);
          constexpr uint32_t kBStep = B_MN ? ((16 * kSwizzleBytes) >> 4) : (32u >> 4);
#pragma unroll
          for (int k = 0; k < kKSteps; ++k) {
            const uint32_t accumulate = (kb > kb_begin || k > 0) ? 1u : 0u;
            if (CG == 2) {
              if (kTf32) ptx::mma_tf32_ss_pair(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
              else ptx::mma_f16_ss_pair(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
            } else {
              if (kTf32) ptx::mma_tf32_ss(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
              else ptx::mma_f16_ss(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, idesc, accumulate);
            }
          }
          if (CG == 2) ptx::mma_commit_pair(empty_bar(stage)); else ptx::mma_commit(empty_bar(stage));
          stage = next_stage;
          phase = next_phase;
          ready = next_ready;
        }
        if (!ok) break;
        if (CG == 2) ptx::mma_commit_pair(tmem_full_bar(acc)); else ptx::mma_commit(tmem_full_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
#ifdef FUSEML_STALL_COUNTERS
      g_stall[blockIdx.x][0] = clock64() - st_begin;
      g_stall[blockIdx.x][9] = ptx::globaltimer_ns();
      g_stall[blockIdx.x][1] = st_full;
      g_stall[blockIdx.x][2] = st_tmem;
#else
      (void)st_full; (void)st_tmem;
#endif
    };
    if (is_leader && ptx::elect_one()) {
      if (tf32) mma_role(std::true_type{}); else mma_role(std::false_type{});
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (every CTA, 8 warps) --------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;          // TMEM lanes a warp may read: 32 * (warp id % 4)
    const int half = ew >> 2;              // which of the two warps of this quarter
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t lead_tmem_empty0 = (CG == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool red_sum = (p.red_kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) != 0;
    const bool red_max = (p.red_kinds & FUSEML_RED_MAX) != 0;
    const bool red_any = red_sum || red_max;
    float all_sum = 0.0f, all_max = -INFINITY;
    bool ok = true;
    long long st_wait = 0, st_work = 0;
#ifdef FUSEML_STALL_COUNTERS
    long long st_ld = 0, st_prog = 0, st_store = 0, st_tail = 0;
#endif
    // Split-K: this K slice's raw fp32 accumulator goes to the workspace in a layout made for
    // the two kernels that touch it, [slice][tile][32-column chunk][16-byte piece][row][4]: one
    // warp-level store writes 32 consecutive 16-byte pieces (512 contiguous bytes) instead of
    // 32 pieces in 32 different rows, and splitk_finish_kernel reads them back the same way.
    float* const split_tile = splitk ? p.split_ws + static_cast<int64_t>(k_slice) * p.num_tiles * (kTileM * bn) : nullptr;
    WorkWalk walk;
    walk.template init<kStreamK>(p, unit, num_units);
    WorkItem w;
    while (walk.next(&w)) {
      const int32_t t = w.tile;
      const bool sk_later = kStreamK && w.kind == 2;       // raw store, no program, no reductions
      const bool sk_first = kStreamK && w.kind == 1;       // add the later parts, then the usual epilogue
      // exchange: raw store of the half this unit does not finish (pass 0), then the partner's part
      // is added to the other half and the epilogue runs on it (pass 1)
      const bool sk_xchg = kStreamK && w.kind == 4;
      const int32_t left_chunks = (bn / CH + 1) / 2;
      const bool right_side = w.kb0 != 0;
      int32_t tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
      const int32_t tm128 = tm * CG + static_cast<int32_t>(cta_rank);   // index of this CTA's 128-row block
      const int32_t m = tm128 * kTileM + quarter * 32 + lane;
      const int32_t n_tile0 = tn * bn;
      const bool row_ok = m < p.M;
      if (half == 0) prefetch_operands(p, m, n_tile0, bn, row_ok, lane);
      // Row vectors (bias): stage this tile's slice in shared memory as fp32 while the K loop
      // runs.  Two buffers (by accumulator parity) and one barrier per tile suffice: nobody
      // passes the next tile's barrier before every warp has finished reading this one.
      float* staged = staged_base + acc * (2 * BN);
      if (p.vec_slot[0] >= 0) {
        const int idx = threadIdx.x - 64;
        if (idx < bn) {
          const int32_t n = n_tile0 + idx;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int32_t slot = p.vec_slot[j];
            if (slot >= 0)
              staged[j * BN + idx] = n < p.N ? epi::load_scalar(p.operands[slot].ptr, n, p.operands[slot].dtype) : 0.0f;
          }
        }
        asm volatile("bar.sync 2, %0;" ::"n"(32 * EW) : "memory");
      }
      // After a failed wait the warp keeps walking its tiles without touching TMEM, so that the
      // named barriers below still see all eight warps.
      {
        FUSEML_STALL_T0();
        if (ok && !ptx::mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag, p.status, kWhereEpilogueTmemFull, true)) {
          ok = false;
        }
        FUSEML_STALL_ADD(st_wait);
      }
      FUSEML_STALL_T0();
      ptx::tc_fence_after_sync();
      float row_sum = 0.0f, row_max = -INFINITY;
      // Tile I/O through shared memory (see GemmParams::io_flags): every warp then walks all its
      // chunks, active or not, because the storing thread counts sixteen arrivals per 64-column box.
      const bool staged_io = tile_in || tile_out;
      if (tile_in && ok &&
          !ptx::mbar_wait(tile_in_bar, 0u, abort_flag, p.status, kWhereEpilogueTileIn, true)) {
        ok = false;
      }
      // bounded wait for `count` parts in consecutive workspace slots (normally complete by now:
      // their K ranges are no longer than this unit's)
      auto wait_parts = [&](int32_t first_slot, int32_t count) {
#ifdef FUSEML_STALL_COUNTERS
        const long long flag_t0 = clock64();
#endif
        for (int32_t j = 0; j < count && ok; ++j) {
          const uint32_t* flag = p.sk_flags + (static_cast<int64_t>(first_slot + j) * CG + cta_rank);
          const uint64_t t0 = ptx::globaltimer_ns();
          while (ptx::ld_acquire_gpu(flag) == 0u) {
            __nanosleep(64);
            const uint32_t limit_us = abort_flag[1];
            if (*abort_flag || ptx::globaltimer_ns() - t0 > (limit_us ? static_cast<uint64_t>(limit_us) * 1000ull : ptx::kWaitLimitNs)) {
              if (!*abort_flag) { *abort_flag = 1u; if (p.status) atomicCAS(p.status, 0, kWhereStreamKPart); }
              ok = false;
              break;
            }
          }
        }
#ifdef FUSEML_STALL_COUNTERS
        st_tail += clock64() - flag_t0;
#endif
      };
      // publish the raw part in slot `slot`: the barrier orders every epilogue thread's stores
      // before thread 64's fence, and the fence (cumulative) orders them before the flag for
      // whoever reads the flag and fences in turn.  One fence per CTA: a fence per thread waits
      // for the thread's own stores under a saturated memory system, 256 times over.
      auto publish_part = [&](int32_t slot) {
        asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
        if (threadIdx.x == 64 && ok) {
          __threadfence();
          *reinterpret_cast<volatile uint32_t*>(p.sk_flags + (static_cast<int64_t>(slot) * CG + cta_rank)) = 1u;
        }
      };
      if (sk_first && ok) wait_parts(w.slot, w.after);
      const int32_t part_slot0 = sk_xchg ? w.after : w.slot;
      const int32_t part_count = sk_xchg ? 1 : w.after;
#pragma unroll 1
      for (int pass = 0; pass < (sk_xchg ? 2 : 1); ++pass) {
      if (sk_xchg && pass == 1) {
        publish_part(w.slot);
        if (ok) wait_parts(w.after, 1);
      }
      const bool raw_store = sk_later || (sk_xchg && pass == 0);
      const bool add_parts = sk_first || (sk_xchg && pass == 1);
#pragma unroll 1
      for (int c = half; (ok || staged_io) && c < bn / CH; c += kEpiSplit) {
        const int32_t n0 = n_tile0 + c * CH;
        const bool active = ok && n0 < p.N;   // uniform across the warp
        if (!active && !staged_io) break;
        if (sk_xchg && (((c >= left_chunks) == right_side) != (pass == 1))) continue;   // the other pass's half
        // this thread's 16 columns inside the swizzled 128 x 64 box (box = chunk / 4)
        uint8_t* piece = smem + (c >> 2) * kBoxBytes + (quarter * 32 + lane) * kSwizzleBytes +
                         ((((c & 3) * 2) ^ (lane & 7)) << 4);
        if (active) {
          // Pull this thread's 64-byte slices of the matrix operand (residual) for this chunk and
          // for the warp's next one into L1 now: by the time the program reaches the op, the
          // load hits L1 instead of waiting on L2.  Costs no registers.
          if (p.mat_slot >= 0 && row_ok && !tile_in) {
            const EpiOperand& mo = p.operands[p.mat_slot];
            const char* mp = reinterpret_cast<const char*>(mo.ptr) + (static_cast<int64_t>(m) * mo.stride_m + n0) * 2;
            if (c == half) { ptx::prefetch_l1(mp); ptx::prefetch_l1(mp + 2 * CH - 1); }
            if (n0 + kEpiSplit * CH < p.N) {
              ptx::prefetch_l1(mp + kEpiSplit * CH * 2);
              ptx::prefetch_l1(mp + kEpiSplit * CH * 2 + 2 * CH - 1);
            }
          }
#ifdef FUSEML_STALL_COUNTERS
          const long long c0 = clock64();
#endif
          uint32_t r[CH];
          ptx::tmem_ld_32x32(tmem_base + lane_base + static_cast<uint32_t>(acc * BN + c * CH), r);
          ptx::tmem_ld_wait();
          float v[CH];
#pragma unroll
          for (int i = 0; i < CH; ++i) v[i] = __uint_as_float(r[i]);
#ifdef FUSEML_STALL_COUNTERS
          const long long c1 = clock64();
#endif
          if (add_parts) {
            // later parts in slot order: the sum does not depend on which unit finished first
            for (int32_t j = 0; j < part_count; ++j) {
              const float4* src = reinterpret_cast<const float4*>(p.sk_ws + (static_cast<int64_t>(part_slot0 + j) * CG + cta_rank) * (kTileM * BN)) +
                                  static_cast<int64_t>(c) * (CH / 4) * kTileM + (quarter * 32 + lane);
              float4 x[CH / 4];
#pragma unroll
              for (int i = 0; i < CH / 4; ++i) x[i] = __ldcg(src + i * kTileM);
#pragma unroll
              for (int i = 0; i < CH / 4; ++i) {
                v[4 * i + 0] += x[i].x;
                v[4 * i + 1] += x[i].y;
                v[4 * i + 2] += x[i].z;
                v[4 * i + 3] += x[i].w;
              }
            }
          }
          if (!raw_store) epi::run_program<PROG, CH>(p, m, n0, row_ok, v, staged + c * CH, BN, tile_in ? piece : nullptr);
#ifdef FUSEML_STALL_COUNTERS
          const long long c2 = clock64();
#endif
          if (raw_store) {
            float4* dst = reinterpret_cast<float4*>(p.sk_ws + (static_cast<int64_t>(w.slot) * CG + cta_rank) * (kTileM * BN)) +
                          static_cast<int64_t>(c) * (CH / 4) * kTileM + (quarter * 32 + lane);
#pragma unroll
            for (int i = 0; i < CH / 4; ++i)
              dst[i * kTileM] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else if (tile_out) {
            if constexpr (CH == 16) epi::store_tile_smem(v, piece, p.out_dtype);
          } else if (splitk) {
            float4* dst = reinterpret_cast<float4*>(split_tile + static_cast<int64_t>(t) * (kTileM * bn)) +
                          static_cast<int64_t>(c) * (CH / 4) * kTileM + (quarter * 32 + lane);
#pragma unroll
            for (int i = 0; i < CH / 4; ++i)
              dst[i * kTileM] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else if (p.d != nullptr && row_ok) {
            epi::store_chunk<CH>(p.d, static_cast<int64_t>(m) * p.ldd, n0, p.N, p.out_dtype, v);
          }
#ifdef FUSEML_STALL_COUNTERS
          st_ld += c1 - c0;
          st_prog += c2 - c1;
          st_store += clock64() - c2;
#endif
          if (red_any && !raw_store) {
            if (p.red_axis == FUSEML_AXIS_M) {
              // column reductions transpose 32 x 32 blocks in registers: 32-column chunks only (the
              // host never picks the 16-warp instance for them)
              if constexpr (CH == 32) {
                float vs[CH], vm[CH];
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                  vs[i] = row_ok ? v[i] : 0.0f;
                  vm[i] = row_ok ? v[i] : -INFINITY;
                }
                if (red_sum) colred[(quarter * 2 + 0) * BN + c * CH + lane] = warp_column_reduce<false>(vs, lane);
                if (red_max) colred[(quarter * 2 + 1) * BN + c * CH + lane] = warp_column_reduce<true>(vm, lane);
              }
            } else if (n0 + CH <= p.N) {
              // full chunk: pairwise packed adds (two chains), maxima as a tree
              epi::f32x2 s0 = epi::pack2(v[0], v[1]), s1 = epi::pack2(v[2], v[3]);
              float m0 = fmaxf(v[0], v[1]), m1 = fmaxf(v[2], v[3]);
#pragma unroll
              for (int i = 4; i < CH; i += 4) {
                s0 = epi::add2(s0, epi::pack2(v[i], v[i + 1]));
                s1 = epi::add2(s1, epi::pack2(v[i + 2], v[i + 3]));
                m0 = fmaxf(m0, fmaxf(v[i], v[i + 1]));
                m1 = fmaxf(m1, fmaxf(v[i + 2], v[i + 3]));
              }
              float lo, hi;
              epi::unpack2(epi::add2(s0, s1), lo, hi);
              row_sum += lo + hi;
              row_max = fmaxf(row_max, fmaxf(m0, m1));
            } else {
#pragma unroll
              for (int i = 0; i < CH; ++i) {
                const bool in = (n0 + i < p.N);
                row_sum += in ? v[i] : 0.0f;
                row_max = in ? fmaxf(row_max, v[i]) : row_max;
              }
            }
          }
        }
        if (EW == 16 && tile_out) {
          // this warp's share of output box c / 4 is in shared memory (or the chunk lies past N):
          // publish it to the async proxy and tell the storing thread.  No CTA-wide barrier: the
          // sixteen warps stay out of step, one warp's exp/rcp overlapping another's FMAs.
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(box_bar(c >> 2));
        }
      }
      }   // pass
      if (sk_later) publish_part(w.slot);
      // accumulator drained: hand the TMEM buffer back to the (leader's) MMA thread
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && ok) {
        if (CG == 2) ptx::mbar_arrive_cluster(lead_tmem_empty0 + 8u * acc);
        else ptx::mbar_arrive(tmem_empty_bar(acc));
      }
      FUSEML_STALL_ADD(st_work);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

      if (red_any && !sk_later) {
        if (p.red_axis == FUSEML_AXIS_N) {
          // two warps share a row: each writes its own partial slot
          if (row_ok && ok) {
            const int64_t o = (static_cast<int64_t>(tn) * kEpiSplit + half) * p.M + m;
            if (red_sum) p.red_sum[o] = row_sum;
            if (red_max) p.red_max[o] = row_max;
          }
        } else if (p.red_axis == FUSEML_AXIS_ALL) {
          if (row_ok) {
            all_sum += row_sum;
            all_max = fmaxf(all_max, row_max);
          }
        } else {
          // AXIS_M: combine the four quarters' column partials, one thread per column
          asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
          for (int j = threadIdx.x - 64; j < bn; j += kEpiWarps * 32) {
            const int32_t n = n_tile0 + j;
            if (n < p.N && ok && tm128 * kTileM < p.M) {
              const int64_t o = static_cast<int64_t>(tm128) * p.N + n;
              if (red_sum)
                p.red_sum[o] = colred[0 * BN + j] + colred[2 * BN + j] + colred[4 * BN + j] + colred[6 * BN + j];
              if (red_max)
                p.red_max[o] = fmaxf(fmaxf(colred[1 * BN + j], colred[3 * BN + j]),
                                     fmaxf(colred[5 * BN + j], colred[7 * BN + j]));
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
        }
      }
    }
#ifdef FUSEML_STALL_COUNTERS
    if (warp == 2 && lane == 0) {
      g_stall[blockIdx.x][3] = st_wait;
      g_stall[blockIdx.x][4] = st_work;
      g_stall[blockIdx.x][10] = ptx::globaltimer_ns();
      g_stall[blockIdx.x][12] = st_ld;
      g_stall[blockIdx.x][13] = st_prog;
      g_stall[blockIdx.x][14] = st_store;
      g_stall[blockIdx.x][15] = st_tail;
    }
#else
    (void)st_wait; (void)st_work;
#endif
    if (red_any && p.red_axis == FUSEML_AXIS_ALL) {
      const float ws = warp_sum(all_sum);
      const float wm = warp_max(all_max);
      if (lane == 0) {
        colred[ew * 2 + 0] = ws;
        colred[ew * 2 + 1] = wm;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
      if (threadIdx.x == 64) {
        float s = 0.0f, mx = -INFINITY;
        for (int w = 0; w < kEpiWarps; ++w) { s += colred[w * 2]; mx = fmaxf(mx, colred[w * 2 + 1]); }
        if (red_sum) p.red_sum[blockIdx.x] = s;
        if (red_max) p.red_max[blockIdx.x] = mx;
      }
    }
  }

  // ------------------------------ tear-down ---------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) {   // neither CTA may leave while its partner can still touch its memory
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
#ifdef FUSEML_STALL_COUNTERS
  if (threadIdx.x == 32) g_stall[blockIdx.x][11] = ptx::globaltimer_ns();
#endif
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (CG == 2) ptx::tmem_dealloc_pair(tmem_base, kTmemCols); else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
#ifdef FUSEML_STALL_COUNTERS
  if (threadIdx.x == 32) g_stall[blockIdx.x][7] = ptx::globaltimer_ns();
#endif
}

}  // namespace v2
}  // namespace fuseml
