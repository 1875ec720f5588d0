// Epilogue virtual machine: runs a short program over 32 accumulator columns of
// one output row held in registers.  The opcode switch is uniform across the
// warp (same program for every element), the element loops are fully unrolled,
// so the interpretation overhead is a handful of instructions per op per 32
// elements.  Semantics follow the reference's emitters
// (fuseml/codegen/kernel_generator.py:1599-1903): everything is evaluated in
// fp32 and cast once at the store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_params.cuh"

namespace fuseml {
namespace epi {

// 1 + erf(z) without cancellation for negative z: Abramowitz-Stegun 7.1.26 gives
// erfc(|z|) = poly(t) * exp(-z^2), t = 1/(1 + p|z|), |error| < 1.5e-7; then
// 1 + erf(z) = erfc(|z|) for z < 0 and 2 - erfc(|z|) otherwise.  Two special-function-unit
// ops and six FMAs per element, no divergent branch (erff() costs about three times as much).
__device__ __forceinline__ float one_plus_erf(float z) {
  const float a = fabsf(z);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, a, 1.0f));  // MUFU.RCP (an IEEE-rounded reciprocal costs several times more)
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float erfc_a = poly * t * __expf(-a * a);
  return z < 0.0f ? erfc_a : 2.0f - erfc_a;
}
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * one_plus_erf(x * 0.70710678118654752440f);
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

__device__ __forceinline__ float load_scalar(const void* p, int64_t idx, int32_t dtype) {
  if (dtype == FUSEML_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  if (dtype == FUSEML_F16) return __half2float(reinterpret_cast<const __half*>(p)[idx]);
  return reinterpret_cast<const float*>(p)[idx];
}

// v[i] = combine(v[i], operand[m, n0 + i]) for the 32 columns of a chunk, without a 32-element
// temporary: values are folded in as each 16-byte word is unpacked.  combine is a*b for MUL and
// sa*a + sb*b otherwise (ADD: 1,1; SUB: 1,-1; RSUB: -1,1).  Columns >= N are left alone.  The
// fast path (unit column stride, 16-byte aligned, full chunk) uses 128-bit loads; with
// stride_m == 0 all lanes hit the same address and the load broadcasts.
__device__ __forceinline__ float combine(bool mul, float sa, float sb, float a, float b) {
  return mul ? a * b : fmaf(sb, b, sa * a);
}

__device__ __forceinline__ void fold_operand_chunk(float (&v)[kChunkN], int32_t code, const EpiOperand& o, int64_t m,
                                                   int32_t n0, int32_t N) {
  const bool mul = code == FUSEML_OP_MUL_T;
  const float sa = code == FUSEML_OP_RSUB_T ? -1.0f : 1.0f;
  const float sb = code == FUSEML_OP_SUB_T ? -1.0f : 1.0f;
  const int64_t base = m * o.stride_m + static_cast<int64_t>(n0) * o.stride_n;
  const bool full = (n0 + kChunkN <= N);
  if (o.stride_n == 1 && full) {
    if (o.dtype == FUSEML_F32) {
      const float* p = reinterpret_cast<const float*>(o.ptr) + base;
      if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < kChunkN / 4; ++i) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(p) + i);
          v[4 * i + 0] = combine(mul, sa, sb, v[4 * i + 0], q.x);
          v[4 * i + 1] = combine(mul, sa, sb, v[4 * i + 1], q.y);
          v[4 * i + 2] = combine(mul, sa, sb, v[4 * i + 2], q.z);
          v[4 * i + 3] = combine(mul, sa, sb, v[4 * i + 3], q.w);
        }
        return;
      }
    } else {
      const uint16_t* p = reinterpret_cast<const uint16_t*>(o.ptr) + base;
      if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < kChunkN / 8; ++i) {
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + i);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f;
            if (o.dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[8 * i + 2 * j] = combine(mul, sa, sb, v[8 * i + 2 * j], f.x);
            v[8 * i + 2 * j + 1] = combine(mul, sa, sb, v[8 * i + 2 * j + 1], f.y);
          }
        }
        return;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kChunkN; ++i) {
    if (n0 + i < N)
      v[i] = combine(mul, sa, sb, v[i], load_scalar(o.ptr, base + static_cast<int64_t>(i) * o.stride_n, o.dtype));
  }
}

// v[i] (+|*)= src[i], src = 32 fp32 values staged in shared memory (same address for every
// lane: the reads broadcast)
template <bool kMul>
__device__ __forceinline__ void fold_staged(float (&v)[kChunkN], const float* src) {
#pragma unroll
  for (int i = 0; i < kChunkN / 4; ++i) {
    const float4 q = reinterpret_cast<const float4*>(src)[i];
    v[4 * i + 0] = kMul ? v[4 * i + 0] * q.x : v[4 * i + 0] + q.x;
    v[4 * i + 1] = kMul ? v[4 * i + 1] * q.y : v[4 * i + 1] + q.y;
    v[4 * i + 2] = kMul ? v[4 * i + 2] * q.z : v[4 * i + 2] + q.z;
    v[4 * i + 3] = kMul ? v[4 * i + 3] * q.w : v[4 * i + 3] + q.w;
  }
}

// Stores v[0..31] to row pointer `row` (element index n0 .. n0+31) in `dtype`.
// fp16 saturates to +-65504 before the cast, as the reference does
// (fuseml/codegen/kernel_generator.py:1575-1581).
__device__ __forceinline__ void store_chunk(void* base_ptr, int64_t row_off, int32_t n0, int32_t N,
                                            int32_t dtype, const float (&v)[kChunkN]) {
  const bool full = (n0 + kChunkN <= N);
  if (dtype == FUSEML_F32) {
    float* p = reinterpret_cast<float*>(base_ptr) + row_off + n0;
    if (full && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < kChunkN / 4; ++i) {
        reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kChunkN; ++i) if (n0 + i < N) p[i] = v[i];
    }
    return;
  }
  uint32_t packed[kChunkN / 2];
  if (dtype == FUSEML_BF16) {
#pragma unroll
    for (int i = 0; i < kChunkN / 2; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kChunkN / 2; ++i) {
      const float a = fminf(fmaxf(v[2 * i], -65504.0f), 65504.0f);
      const float b = fminf(fmaxf(v[2 * i + 1], -65504.0f), 65504.0f);
      const __half2 h = __floats2half2_rn(a, b);
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  uint16_t* p = reinterpret_cast<uint16_t*>(base_ptr) + row_off + n0;
  if (full && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
    for (int i = 0; i < kChunkN / 8; ++i) {
      reinterpret_cast<uint4*>(p)[i] =
          make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kChunkN; ++i) {
      if (n0 + i < N) p[i] = static_cast<uint16_t>((packed[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu);
    }
  }
}

// Runs the program on one chunk.  `row_ok` is false for rows past M: their
// operand loads and aux stores are skipped (values are don't-care).
// `staged` points at this chunk's 32 columns of the row vectors staged in shared memory
// (vector j at staged + j * staged_stride).
template <bool kUsesSaved>
__device__ __forceinline__ void run_program(const GemmParams& p, int64_t m, int32_t n0, bool row_ok,
                                            float (&v)[kChunkN], const float* staged, int32_t staged_stride) {
  float s[kUsesSaved ? kChunkN : 1];
  if (kUsesSaved) {
#pragma unroll
    for (int i = 0; i < (kUsesSaved ? kChunkN : 1); ++i) s[i] = 0.0f;
  }
  for (int op = 0; op < p.n_ops; ++op) {
    const int32_t code = p.ops[op].opcode;
    switch (code) {
      case FUSEML_OP_RELU:
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] = v[i] > 0.0f ? v[i] : 0.0f;
        break;
      case FUSEML_OP_GELU_ERF:
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] = gelu_erf(v[i]);
        break;
      case FUSEML_OP_GELU_TANH:
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] = gelu_tanh(v[i]);
        break;
      case FUSEML_OP_SIGMOID:
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] = sigmoid(v[i]);
        break;
      case FUSEML_OP_ADD_IMM: {
        const float c = p.ops[op].imm;
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] += c;
      } break;
      case FUSEML_OP_MUL_IMM: {
        const float c = p.ops[op].imm;
#pragma unroll
        for (int i = 0; i < kChunkN; ++i) v[i] *= c;
      } break;
      case FUSEML_OP_ADD_T:
      case FUSEML_OP_MUL_T:
      case FUSEML_OP_SUB_T:
      case FUSEML_OP_RSUB_T: {
        const int32_t pre = p.ops[op].reserved;
        if (pre == 1 || pre == 2) {
          const float* src = staged + (pre - 1) * staged_stride;
          if (code == FUSEML_OP_ADD_T) fold_staged<false>(v, src); else fold_staged<true>(v, src);
        } else if (row_ok) {
          fold_operand_chunk(v, code, p.operands[p.ops[op].slot], m, n0, p.N);
        }
      } break;
      case FUSEML_OP_STORE_AUX: {
        if (row_ok) {
          const EpiOperand& o = p.operands[p.ops[op].slot];
          store_chunk(const_cast<void*>(o.ptr), m * o.stride_m, n0, p.N, o.dtype, v);
        }
      } break;
      case FUSEML_OP_SAVE:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < kChunkN; ++i) s[i] = v[i];
        }
        break;
      case FUSEML_OP_SWAP:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < kChunkN; ++i) { const float x = v[i]; v[i] = s[i]; s[i] = x; }
        }
        break;
      case FUSEML_OP_ADD_SAVED:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < kChunkN; ++i) v[i] += s[i];
        }
        break;
      case FUSEML_OP_MUL_SAVED:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < kChunkN; ++i) v[i] *= s[i];
        }
        break;
      default:
        break;
    }
  }
}

}  // namespace epi
}  // namespace fuseml
