// Second kernel of a split-K launch: folds the K slices' fp32 partial tiles in a fixed order
// (slice 0, 1, 2, ...: the result does not depend on which CTA finished first), runs the
// epilogue program on the sum and stores the output.  One thread per output row and 16
// columns; neighbouring threads take neighbouring chunks of the same row, so the partials are
// read and the output is written in contiguous 64-byte / 32-byte pieces.
//
// The reference has no counterpart (its Triton template always walks the whole K loop in one
// program, fuseml/codegen/kernel_generator.py:1454-1542).
#pragma once

#include "epilogue.cuh"
#include "gemm_params.cuh"

namespace fuseml {

constexpr int kFinishChunk = 16;

template <bool USES_SAVED>
__global__ void __launch_bounds__(256) splitk_finish_kernel(const __grid_constant__ GemmParams p) {
  const int64_t chunks_per_row = (p.N + kFinishChunk - 1) / kFinishChunk;
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= chunks_per_row * p.M) return;
  const int64_t m = idx / chunks_per_row;
  const int32_t n0 = static_cast<int32_t>(idx - m * chunks_per_row) * kFinishChunk;
  const int64_t slice = static_cast<int64_t>(p.M) * p.N;
  const float* src = p.split_ws + m * p.N + n0;
  float v[kFinishChunk];
#pragma unroll
  for (int i = 0; i < kFinishChunk; ++i) v[i] = 0.0f;
  const bool full = (n0 + kFinishChunk <= p.N);
  if (full && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (slice & 3) == 0) {
    for (int s = 0; s < p.split_k; ++s) {
      const float4* q = reinterpret_cast<const float4*>(src + s * slice);
#pragma unroll
      for (int i = 0; i < kFinishChunk / 4; ++i) {
        const float4 x = __ldcs(q + i);   // read once: do not keep the partials in cache
        v[4 * i + 0] += x.x;
        v[4 * i + 1] += x.y;
        v[4 * i + 2] += x.z;
        v[4 * i + 3] += x.w;
      }
    }
  } else {
    for (int s = 0; s < p.split_k; ++s) {
#pragma unroll
      for (int i = 0; i < kFinishChunk; ++i) {
        if (n0 + i < p.N) v[i] += src[s * slice + i];
      }
    }
  }
  epi::run_program<USES_SAVED, kFinishChunk>(p, m, n0, true, v, nullptr, 0);
  if (p.d != nullptr) epi::store_chunk<kFinishChunk>(p.d, m * p.ldd, n0, p.N, p.out_dtype, v);
}

}  // namespace fuseml
