// Device-side parameter block of the fused GEMM kernels.  It is filled on the
// host from the public fuseml_gemm_desc_t + fuseml_plan_t and passed by value
// (kernel parameter space), so a launch reads no host memory and needs no
// device-side allocation.
#pragma once

#include <stdint.h>

#include "../../include/fuseml_sm100.h"

namespace fuseml {

constexpr int kTileM = 128;        // UMMA M with cta_group::1: one TMEM lane per row
constexpr int kSwizzleBytes = 128; // K extent of one shared-memory stage, in bytes
constexpr int kChunkN = 32;        // accumulator columns one tcgen05.ld brings in

struct EpiOperand {
  const void* ptr;
  int64_t stride_m;
  int64_t stride_n;
  int32_t dtype;
  int32_t writable;
};

struct GemmParams {
  int32_t M, N, K;
  int32_t tiles_m, tiles_n, num_tiles, group_m, num_kb;
  int32_t bn;        // tile width actually used (multiple of 32, at most the kernel's BN)
  void* d;           // may be null (reduction-only chains)
  int64_t ldd;
  int32_t out_dtype;
  int32_t n_ops;
  fuseml_epi_op_t ops[FUSEML_MAX_EPI_OPS];
  EpiOperand operands[FUSEML_MAX_OPERANDS];
  // reductions: partials go to `red_sum` / `red_max` (inside the caller's
  // workspace); a finalize kernel folds them afterwards.
  int32_t red_kinds;
  int32_t red_axis;
  float* red_sum;    // [partials][len]
  float* red_max;    // [partials][len]
  int32_t uses_saved;  // program contains SAVE/SWAP/*_SAVED
  int32_t fmt;         // operand format of the MMA: 0 = f16, 1 = bf16, 2 = tf32 (fp32 storage, 32 elements per stage)
  // Operand fetch ahead of use (ops[i].reserved selects the path: 0 = load where the op runs):
  //   vec_slot[j] (reserved = 1 + j): a row vector (bias) - its slice for the tile is staged in
  //     shared memory as fp32 once per tile, while the K loop is still running;
  //   mat_slot (reserved = 3): a full [M,N] 16-bit operand (residual) - each thread's 64-byte
  //     slices are prefetched into L1 one chunk ahead of their use.
  int32_t vec_slot[2];
  int32_t mat_slot;
  // L2 policy of the operand loads: 0 = default, 1 = evict-first (an operand every element of
  // which is read by one or two tiles only: keeping it would push reusable data out of L2),
  // 2 = evict-last (the small operand everybody re-reads while the other one streams past)
  int32_t a_stream, b_stream;
  // Tile I/O through shared memory (sixteen-warp instance, a CTA's only tile, tile width 256):
  //   bit 0: the matrix operand (mat_slot) is brought in by TMA into the drained operand ring;
  //   bit 1: the output tile is written to the ring and stored by TMA.
  // Both replace row-per-thread global accesses (32 cache lines per warp-level instruction) by
  // bulk copies of 128 x 64 boxes.
  int32_t io_flags;
  // Split-K: split_k > 1 CTAs share one tile's K loop; work item t = tile + num_tiles * slice,
  // slice s covers K blocks [s * kb_per_split, ...); each CTA stores its raw fp32 accumulator
  // to split_ws[s][tile][column / 4][row][4] and splitk_finish_kernel folds the slices and runs
  // the epilogue.
  int32_t split_k;
  int32_t kb_per_split;
  float* split_ws;
  // K-split last wave (CTA pairs, stream_k != 0): the tiles of a ragged last wave are shared
  // between all units by K ranges (see WorkWalk).  A unit that computes a later part of a tile
  // stores its raw fp32 accumulator to workspace slot s (per CTA: 128 x BN floats at
  // sk_ws[s * CG + rank], the split-K piece-major layout) and raises sk_flags[s * CG + rank];
  // the unit that owns the tile adds the parts to its accumulator in slot order and runs the
  // epilogue.  (Contiguous K ranges of equal length for every unit, tried first, put the units
  // at different K positions, lose the sharing of operands through L2 and run slower than the
  // ragged wave.)
  int32_t stream_k;
  float* sk_ws;
  uint32_t* sk_flags;   // one per CTA, zeroed by the host before the launch
  int32_t* status;     // device status word (bounded-wait time-outs)
  // Diagnostics (fuseml_sm100_set_diagnostics; both 0 in normal operation): the wall-clock limit
  // of a bounded wait in microseconds (0 = the built-in two seconds), and a host-injected
  // failure: the producer issues no load for the last K block of its last tile, so that the MMA
  // thread waits on a barrier that nothing completes while no copy is in flight.
  uint32_t wait_limit_us;
  int32_t drop_last_load;
};

// Tile id -> (tile row, tile column).  Tiles are walked in groups of
// `group_m` tile rows: CTAs that run at the same time then share a narrow band
// of B columns and a short stack of A row blocks, which keeps both resident in
// L2 (same idea as the GROUP_SIZE_M swizzle of the reference,
// fuseml/codegen/kernel_generator.py:1278-1286).
// group_m < 0 (FUSEML_PLAN_GROUP_N): bands of -group_m tile columns instead, columns fastest
// inside a band, all rows of one band before the next band.
__host__ __device__ inline void tile_coords(int32_t t, int32_t tiles_m, int32_t tiles_n, int32_t group_m,
                                            int32_t* tm, int32_t* tn) {
  if (group_m < 0) {
    const int32_t g = -group_m;
    const int32_t band_size = g * tiles_m;
    const int32_t band = t / band_size;
    const int32_t first_n = band * g;
    const int32_t cols = (tiles_n - first_n) < g ? (tiles_n - first_n) : g;
    const int32_t r = t - band * band_size;
    *tn = first_n + (r % cols);
    *tm = r / cols;
    return;
  }
  const int32_t group_size = group_m * tiles_n;
  const int32_t group_id = t / group_size;
  const int32_t first_m = group_id * group_m;
  const int32_t rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int32_t r = t - group_id * group_size;
  *tm = first_m + (r % rows);
  *tn = r / rows;
}

// One unit's (CTA's or CTA pair's) walk over its work; the three roles of a CTA run the same walk.
//   kind 0  a whole tile, K blocks [0, num_kb)
//   kind 1  the first part of a K-split tile: this unit finishes the tile after adding the
//           `after` later parts, which other units left in workspace slots slot .. slot+after-1
//   kind 2  a later part of a K-split tile: the raw accumulator goes to workspace slot `slot`
//   kind 3  a split-K slice (every CTA has exactly one; folded by splitk_finish_kernel)
//   kind 4  one of the two K halves of an exchanged tile: the unit stores the raw accumulator of
//           the columns it does not finish to workspace slot `slot`, then adds the partner's
//           part from slot `after` to the half of the columns it does finish (the left half of
//           the tile when kb0 == 0, the right half otherwise) and runs the epilogue on it
//
// K-split last wave (GemmParams::stream_k): T tiles on U units leave R = T % U tiles for the last
// wave; the whole waves before it are walked as usual.
//   R <= U / 2  every last-wave tile is cut into S = U / R equal K slices, one per unit; the unit
//               with slice 0 finishes the tile (slot of a later slice = its unit index).  With
//               S = 2 and no fused reduction the two units exchange halves instead (kind 4): each
//               publishes and each finishes half a tile, so neither the pass through the
//               workspace nor the epilogue of a whole tile is left to one of them.
//   R >  U / 2  owner units 0..R-1 take K blocks [0, num_kb - L) of their tile, where
//               L = 3/4 num_kb (U - R) / U; the R L blocks left over form one stream in tile order that
//               the U - R helper units share in equal contiguous runs.  A run crosses tile
//               boundaries, so a helper walks several short parts; the part of tile t done by
//               helper h goes to slot t + h (parts are ordered in both, so the sum is unique), and
//               a tile's leftover lies in at most two helpers' runs.
// Either way every unit's last-wave work starts at the same time and takes about the same time,
// owners walk K in step (they share B through L2), and sums run in slot order.
struct WorkItem {
  int32_t tile, kb0, kb1, kind, after, slot;
  bool last;            // the unit's last item
};

struct WorkWalk {
  int32_t unit, units, num_kb, dp_tiles;
  int32_t next_dp;      // next whole tile
  int32_t sk_tile, sk_kb0, sk_kb1, sk_kind, sk_after, sk_slot;   // the unit's one part of a last-wave tile (sk_tile < 0: none)
  int32_t hp_pos, hp_end, hp_len, hp_own, hp_index;              // a helper's run of left-over K blocks (hp_pos >= hp_end: none)
  int32_t splitk_tile, splitk_kb0, splitk_kb1;                   // split-K item (kind 3), -1 when taken

  // SK = false compiles the K-split last wave out (kernel instances that never run it: their
  // register budget has no room for the walk's extra state)
  template <bool SK = true>
  __host__ __device__ void init(const GemmParams& p, int32_t unit_, int32_t units_) {
    unit = unit_; units = units_; num_kb = p.num_kb;
    splitk_tile = -1; splitk_kb0 = splitk_kb1 = 0;
    sk_tile = -1; sk_kb0 = sk_kb1 = sk_kind = sk_after = sk_slot = 0;
    hp_pos = hp_end = hp_len = hp_own = hp_index = 0;
    if (p.split_k > 1) {
      const int32_t slice = unit / p.num_tiles;
      splitk_tile = unit % p.num_tiles;
      splitk_kb0 = slice * p.kb_per_split;
      splitk_kb1 = splitk_kb0 + p.kb_per_split < num_kb ? splitk_kb0 + p.kb_per_split : num_kb;
      dp_tiles = 0;
      next_dp = 0;
      return;
    }
    const int32_t rem = (SK && p.stream_k) ? p.num_tiles % units : 0;
    const int32_t slices = rem > 0 ? units / rem : 0;       // K slices per last-wave tile
    dp_tiles = p.num_tiles;
    next_dp = unit;
    if (slices >= 2) {
      dp_tiles = p.num_tiles - rem;
      if (unit < rem * slices) {
        const int32_t per = (num_kb + slices - 1) / slices;
        const int32_t used = (num_kb + per - 1) / per;          // slices that are not empty
        const int32_t slice = unit % slices;
        if (slice < used) {
          sk_tile = dp_tiles + unit / slices;
          sk_kb0 = slice * per;
          sk_kb1 = sk_kb0 + per < num_kb ? sk_kb0 + per : num_kb;
          sk_kind = (used == 1) ? 0 : (slice == 0 ? 1 : 2);
          sk_after = slice == 0 ? used - 1 : 0;
          sk_slot = slice == 0 ? unit + 1 : unit;
          if (slices == 2 && used == 2 && p.red_kinds == 0) {
            sk_kind = 4;
            sk_slot = unit;
            sk_after = unit ^ 1;       // units 2j and 2j + 1 share tile j of the last wave
          }
        }
      }
    } else if (slices == 1 && rem < units) {
      const int32_t idle = units - rem;
      // L: 3/4 of the even share.  A helper's K blocks come slower than an owner's (its operands
      // are shared with nobody through L2; measured 0.41 against 0.36 us per block) and each of its
      // parts ends with a store of the raw accumulator.
      const int32_t left = static_cast<int32_t>(static_cast<int64_t>(num_kb) * idle * 3 / (static_cast<int64_t>(units) * 4));
      if (left >= 1) {
        dp_tiles = p.num_tiles - rem;
        const int32_t run = (rem * left + idle - 1) / idle;       // K blocks per helper (>= left, as rem > idle)
        if (unit < rem) {
          const int32_t h0 = unit * left / run, h1 = ((unit + 1) * left - 1) / run;
          sk_tile = dp_tiles + unit;
          sk_kb0 = 0;
          sk_kb1 = num_kb - left;
          sk_kind = 1;
          sk_after = h1 - h0 + 1;
          sk_slot = unit + h0;
        } else {
          hp_index = unit - rem;
          hp_len = left;
          hp_own = num_kb - left;
          hp_pos = hp_index * run;
          hp_end = hp_pos + run < rem * left ? hp_pos + run : rem * left;
        }
      }
    }
  }

  __host__ __device__ bool next(WorkItem* w) {
    if (splitk_tile >= 0) {
      *w = WorkItem{splitk_tile, splitk_kb0, splitk_kb1, 3, 0, 0, true};
      splitk_tile = -1;
      dp_tiles = 0;
      sk_tile = -1;
      return true;
    }
    if (next_dp < dp_tiles) {
      const int32_t t = next_dp;
      next_dp += units;
      *w = WorkItem{t, 0, num_kb, 0, 0, 0, next_dp >= dp_tiles && sk_tile < 0 && hp_pos >= hp_end};
      return true;
    }
    if (sk_tile >= 0) {
      *w = WorkItem{sk_tile, sk_kb0, sk_kb1, sk_kind, sk_after, sk_slot, true};
      sk_tile = -1;
      return true;
    }
    if (hp_pos < hp_end) {
      const int32_t t = hp_pos / hp_len;
      const int32_t stop = hp_end < (t + 1) * hp_len ? hp_end : (t + 1) * hp_len;
      *w = WorkItem{dp_tiles + t, hp_own + (hp_pos - t * hp_len), hp_own + (stop - t * hp_len), 2, 0, t + hp_index, stop == hp_end};
      hp_pos = stop;
      return true;
    }
    return false;
  }
};

}  // namespace fuseml
