// Second kernel of a split-K launch: folds the K slices' fp32 partial tiles in a fixed order
// (slice 0, 1, 2, ...: the result does not depend on which CTA finished first), runs the
// epilogue program on the sum and stores the output.  One thread per output row and 16
// columns.
//
// The reference has no counterpart (its Triton template always walks the whole K loop in one
// program, fuseml/codegen/kernel_generator.py:1454-1542).
#pragma once

#include "epilogue.cuh"
#include "gemm_params.cuh"

namespace fuseml {

constexpr int kFinishChunk = 16;      // columns per thread; 8 for small problems (twice the threads)

// Partial tiles are stored as [slice][tile][16-byte piece = column / 4][row][4 floats] (see the
// GEMM kernel): a thread takes one row and four consecutive pieces (16 columns); threads that
// are neighbours in a warp take neighbouring rows, so every load instruction of a warp reads
// 512 contiguous bytes.
template <bool USES_SAVED, int CHUNK = kFinishChunk>
__global__ void __launch_bounds__(256) splitk_finish_kernel(const __grid_constant__ GemmParams p) {
  constexpr int kFinishChunk = CHUNK;                                 // shadows the default: columns per thread
  const int32_t groups_per_tile = p.bn / kFinishChunk;               // column groups in a tile
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int32_t row = static_cast<int32_t>(idx % kTileM);
  const int64_t rest = idx / kTileM;
  const int32_t group = static_cast<int32_t>(rest % groups_per_tile);
  const int64_t tile = rest / groups_per_tile;
  if (tile >= p.num_tiles) return;
  int32_t tm, tn;
  tile_coords(static_cast<int32_t>(tile), p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
  const int64_t m = static_cast<int64_t>(tm) * kTileM + row;
  const int32_t n0 = tn * p.bn + group * kFinishChunk;
  if (m >= p.M || n0 >= p.N) return;
  const int64_t tile_floats = static_cast<int64_t>(kTileM) * p.bn;
  const int64_t slice_floats = static_cast<int64_t>(p.num_tiles) * tile_floats;
  const float4* src = reinterpret_cast<const float4*>(p.split_ws + tile * tile_floats) +
                      static_cast<int64_t>(group) * (kFinishChunk / 4) * kTileM + row;
  float v[kFinishChunk];
#pragma unroll
  for (int i = 0; i < kFinishChunk; ++i) v[i] = 0.0f;
  // Four slices' loads are issued before the first is added (sixteen 16-byte loads in flight per
  // thread: the pass is bound by load latency, not bandwidth); the additions keep slice order.
  constexpr int kBatch = 4;
  for (int s0 = 0; s0 < p.split_k; s0 += kBatch) {
    float4 x[kBatch][kFinishChunk / 4];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const float4* q = src + static_cast<int64_t>(s0 + u) * (slice_floats / 4);
#pragma unroll
      for (int i = 0; i < kFinishChunk / 4; ++i)
        x[u][i] = (s0 + u < p.split_k) ? __ldcs(q + i * kTileM) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);   // read once
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (s0 + u < p.split_k) {
#pragma unroll
        for (int i = 0; i < kFinishChunk / 4; ++i) {
          v[4 * i + 0] += x[u][i].x;
          v[4 * i + 1] += x[u][i].y;
          v[4 * i + 2] += x[u][i].z;
          v[4 * i + 3] += x[u][i].w;
        }
      }
    }
  }
  epi::run_program<USES_SAVED ? epi::kProgGenericSaved : epi::kProgGeneric, kFinishChunk>(p, m, n0, true, v, nullptr, 0);
  if (p.d != nullptr) epi::store_chunk<kFinishChunk>(p.d, m * p.ldd, n0, p.N, p.out_dtype, v);
}

}  // namespace fuseml
