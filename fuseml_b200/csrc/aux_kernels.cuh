// Small helper kernels around the fused GEMM: folding reduction partials,
// the stand-alone reduction tail, and the hi|lo|hi expansion of fp32 operands.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "../../include/fuseml_sm100.h"

namespace fuseml {

// out[i] = fold over j of partial[j*len + i].  Sums are folded in double so the
// result does not depend on how many partials there were.  mean = sum * inv_count.
// The reference folds with global atomics instead
// (fuseml/codegen/kernel_generator.py:1959-2017), which is order-dependent.
__global__ void reduce_finalize_kernel(const float* __restrict__ psum, const float* __restrict__ pmax,
                                       int64_t partials, int64_t len, double inv_count,
                                       float* __restrict__ out_sum, float* __restrict__ out_max,
                                       float* __restrict__ out_mean) {
  if (len == 1) {
    // one scalar: whole block cooperates over the partials
    __shared__ double s_sum[32];
    __shared__ float s_max[32];
    if (blockIdx.x != 0) return;
    double acc = 0.0;
    float mx = -INFINITY;
    for (int64_t j = threadIdx.x; j < partials; j += blockDim.x) {
      if (psum) acc += static_cast<double>(psum[j]);
      if (pmax) mx = fmaxf(mx, pmax[j]);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      acc += __shfl_xor_sync(0xffffffffu, acc, s);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_sum[warp] = acc; s_max[warp] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int nw = (blockDim.x + 31) >> 5;
      double a = 0.0;
      float m = -INFINITY;
      for (int w = 0; w < nw; ++w) { a += s_sum[w]; m = fmaxf(m, s_max[w]); }
      if (out_sum) out_sum[0] = static_cast<float>(a);
      if (out_mean) out_mean[0] = static_cast<float>(a * inv_count);
      if (out_max) out_max[0] = m;
    }
    return;
  }
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < len;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    double acc = 0.0;
    float mx = -INFINITY;
    for (int64_t j = 0; j < partials; ++j) {
      if (psum) acc += static_cast<double>(psum[j * len + i]);
      if (pmax) mx = fmaxf(mx, pmax[j * len + i]);
    }
    if (out_sum) out_sum[i] = static_cast<float>(acc);
    if (out_mean) out_mean[i] = static_cast<float>(acc * inv_count);
    if (out_max) out_max[i] = mx;
  }
}

// Neutral elements for partial arrays (0 for sums, -inf for maxima).
__global__ void fill_neutral_kernel(float* __restrict__ psum, float* __restrict__ pmax, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (psum) psum[i] = 0.0f;
    if (pmax) pmax[i] = -INFINITY;
  }
}

__device__ __forceinline__ float tail_load(const void* x, int64_t idx, int32_t dtype) {
  if (dtype == FUSEML_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[idx]);
  if (dtype == FUSEML_F16) return __half2float(reinterpret_cast<const __half*>(x)[idx]);
  return reinterpret_cast<const float*>(x)[idx];
}

// Streams rows of x[M,N] (leading dimension ldx): each block folds whole rows,
// 16-byte loads where the row start is aligned.  mode 0: one result per row
// written straight to the outputs; mode 1: one partial per block (folded by
// reduce_finalize_kernel afterwards).
__global__ void reduce_rows_kernel(const void* __restrict__ x, int32_t dtype, int64_t M, int64_t N, int64_t ldx,
                                   int32_t mode, double inv_count, float* __restrict__ out_sum,
                                   float* __restrict__ out_max, float* __restrict__ out_mean) {
  __shared__ float s_sum[32];
  __shared__ float s_max[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  const int eb = dtype == FUSEML_F32 ? 4 : 2;
  const int vec = 16 / eb;
  float blk_sum = 0.0f, blk_max = -INFINITY;
  for (int64_t m = blockIdx.x; m < M; m += gridDim.x) {
    const char* row = reinterpret_cast<const char*>(x) + m * ldx * eb;
    float acc = 0.0f, mx = -INFINITY;
    int64_t n_vec = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
      n_vec = N / vec;
      for (int64_t i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (dtype == FUSEML_F32) {
            const float f = __uint_as_float(w[j]);
            acc += f; mx = fmaxf(mx, f);
          } else {
            float2 f;
            if (dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            acc += f.x + f.y; mx = fmaxf(mx, fmaxf(f.x, f.y));
          }
        }
      }
    }
    for (int64_t n = n_vec * vec + threadIdx.x; n < N; n += blockDim.x) {
      const float f = tail_load(x, m * ldx + n, dtype);
      acc += f; mx = fmaxf(mx, f);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      acc += __shfl_xor_sync(0xffffffffu, acc, s);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    }
    if (lane == 0) { s_sum[warp] = acc; s_max[warp] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.0f, b = -INFINITY;
      for (int w = 0; w < nw; ++w) { a += s_sum[w]; b = fmaxf(b, s_max[w]); }
      if (mode == 0) {
        if (out_sum) out_sum[m] = a;
        if (out_mean) out_mean[m] = static_cast<float>(a * inv_count);
        if (out_max) out_max[m] = b;
      } else {
        blk_sum += a; blk_max = fmaxf(blk_max, b);
      }
    }
    __syncthreads();
  }
  if (mode == 1 && threadIdx.x == 0) {
    if (out_sum) out_sum[blockIdx.x] = blk_sum;
    if (out_max) out_max[blockIdx.x] = blk_max;
  }
}

// Column reductions: thread = one column, block.y slices the rows; writes
// partial[slice][N].
__global__ void reduce_cols_kernel(const void* __restrict__ x, int32_t dtype, int64_t M, int64_t N, int64_t ldx,
                                   int64_t rows_per_slice, float* __restrict__ psum, float* __restrict__ pmax) {
  const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (n >= N) return;
  const int64_t m0 = blockIdx.y * rows_per_slice;
  const int64_t m1 = (m0 + rows_per_slice < M) ? (m0 + rows_per_slice) : M;
  float acc = 0.0f, mx = -INFINITY;
  for (int64_t m = m0; m < m1; ++m) {
    const float f = tail_load(x, m * ldx + n, dtype);
    acc += f; mx = fmaxf(mx, f);
  }
  if (psum) psum[blockIdx.y * N + n] = acc;
  if (pmax) pmax[blockIdx.y * N + n] = mx;
}

// fp32 -> three-term TF32 expansion along K.  For a source matrix S[rows, K]
// (element (r,k) at src[r*stride_r + k*stride_k]) writes dst[r, 0:3K] as
//   variant 0 (A side): [ hi | lo | hi ]      variant 1 (B side): [ hi | hi | lo ]
// where hi keeps the top 10 mantissa bits (exactly a TF32 value) and lo = x - hi.
// A TF32 GEMM over the 3K-long rows then computes hi*hi + lo*hi + hi*lo, i.e. the
// fp32 product to ~2^-21 relative, with fp32 accumulation.
struct SplitJob {
  const float* src;
  int64_t rows, K, stride_r, stride_k;
  int32_t variant;     // 0: [hi|lo|hi] (the A side), 1: [hi|hi|lo] (the B side)
  float* dst;
  int64_t ld;
  int32_t blocks;      // blocks of the launch that work on this job (0 = none)
};

// Up to three operands in one launch: blocks [0, a.blocks) expand a, the next b.blocks expand b,
// the rest c (a job with blocks == 0 is skipped).
__global__ void split_tf32_kernel(const SplitJob a, const SplitJob b, const SplitJob c) {
  const int32_t bx = static_cast<int32_t>(blockIdx.x);
  const int which = bx < a.blocks ? 0 : (bx < a.blocks + b.blocks ? 1 : 2);
  // every field is selected on its own: a reference to one of the three parameter structs chosen
  // at run time makes the compiler copy them to local memory (measured: 13 us per launch)
#define FUSEML_PICK(f) (which == 0 ? a.f : (which == 1 ? b.f : c.f))
  const float* __restrict__ src = FUSEML_PICK(src);
  float* __restrict__ dst = FUSEML_PICK(dst);
  const int64_t rows = FUSEML_PICK(rows), K = FUSEML_PICK(K), stride_r = FUSEML_PICK(stride_r), stride_k = FUSEML_PICK(stride_k);
  const int64_t ld = FUSEML_PICK(ld);
  const int32_t variant = FUSEML_PICK(variant), blocks = FUSEML_PICK(blocks);
#undef FUSEML_PICK
  const int64_t block = which == 0 ? bx : (which == 1 ? bx - a.blocks : bx - a.blocks - b.blocks);
  const int64_t total = rows * K;
  for (int64_t i = block * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(blocks) * blockDim.x) {
    // when K is the strided dimension of the source, walk rows fastest so that reads coalesce
    int64_t r, k;
    if (stride_k == 1) { r = i / K; k = i - r * K; } else { k = i / rows; r = i - k * rows; }
    const float x = src[r * stride_r + k * stride_k];
    const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    const float lo = x - hi;
    float* o = dst + r * ld;
    o[k] = hi;
    o[K + k] = variant == 0 ? lo : hi;
    o[2 * K + k] = variant == 0 ? hi : lo;
  }
}

}  // namespace fuseml
