// Epilogue virtual machine: runs a short program over a chunk of CH (32 or 16) accumulator
// columns of one output row held in registers.  The opcode switch is uniform across the
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

// ---- packed fp32 arithmetic (two lanes per instruction, sm_100) ---------------------------
// Epilogue instructions compete for issue slots with the single threads that feed TMA and the
// tensor core (measured: every issue cycle of epilogue arithmetic per scheduler costs about one
// cycle of MMA time), so the element-wise math is written over pairs of columns with the
// f32x2 forms of add/mul/fma; only the special-function ops and bit operations stay scalar.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 r, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
}
__device__ __forceinline__ f32x2 splat2(float c) { return pack2(c, c); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// GELU (erf form) of two values: 0.5 x (1 + erf(x / sqrt 2)).
// erf through Abramowitz-Stegun 7.1.26: erfc(|z|) = poly(t) exp(-z^2), t = 1/(1 + p|z|),
// |error| < 1.5e-7, and erf(z) = copysign(1 - erfc(|z|), z) (no cancellation for either sign).
// With z = x / sqrt 2 folded into the constants: t = 1/(1 + (p/sqrt 2)|x|),
// exp(-z^2) = 2^(-(log2 e / 2) x^2).  Two special-function ops per element; the rest is ten
// packed instructions per pair.
__device__ __forceinline__ void gelu_erf2(float& x0, float& x1) {
  const f32x2 x = pack2(x0, x1);
  const f32x2 ax = pack2(fabsf(x0), fabsf(x1));
  const f32x2 den = fma2(ax, splat2(0.3275911f * 0.70710678118654752440f), splat2(1.0f));
  float d0, d1;
  unpack2(den, d0, d1);
  const f32x2 t = pack2(rcp_approx(d0), rcp_approx(d1));
  f32x2 poly = fma2(t, splat2(1.061405429f), splat2(-1.453152027f));
  poly = fma2(poly, t, splat2(1.421413741f));
  poly = fma2(poly, t, splat2(-0.284496736f));
  poly = fma2(poly, t, splat2(0.254829592f));
  poly = mul2(poly, t);
  float a0, a1;
  unpack2(mul2(mul2(x, x), splat2(-0.5f * 1.4426950408889634f)), a0, a1);
  const f32x2 e = pack2(ex2_approx(a0), ex2_approx(a1));
  float r0, r1;
  unpack2(fma2(poly, mul2(e, splat2(-1.0f)), splat2(1.0f)), r0, r1);   // 1 - erfc(|z|) = |erf z|
  const f32x2 erf = pack2(copysignf(r0, x0), copysignf(r1, x1));
  const f32x2 hx = mul2(x, splat2(0.5f));
  unpack2(fma2(hx, erf, hx), x0, x1);
}

// GELU (tanh form): 0.5 x (1 + tanh u), u = k0 (x + k1 x^3).  0.5 (1 + tanh u) = 1 / (1 + e^(-2u)),
// so gelu = x / (1 + 2^(x (c0 + c1 x^2))) with c0 = -2 k0 log2 e, c1 = c0 k1.
__device__ __forceinline__ void gelu_tanh2(float& x0, float& x1) {
  const float c0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const f32x2 x = pack2(x0, x1);
  const f32x2 w = mul2(x, fma2(mul2(x, x), splat2(c0 * 0.044715f), splat2(c0)));
  float w0, w1;
  unpack2(w, w0, w1);
  // 2^w overflows to +inf for very negative x: x / inf = -0, the correct limit
  const f32x2 den = add2(pack2(ex2_approx(w0), ex2_approx(w1)), splat2(1.0f));
  float d0, d1;
  unpack2(den, d0, d1);
  unpack2(mul2(x, pack2(rcp_approx(d0), rcp_approx(d1))), x0, x1);
}

// sigmoid: 1 / (1 + 2^(-x log2 e))
__device__ __forceinline__ void sigmoid2(float& x0, float& x1) {
  float w0, w1;
  unpack2(mul2(pack2(x0, x1), splat2(-1.4426950408889634f)), w0, w1);
  const f32x2 den = add2(pack2(ex2_approx(w0), ex2_approx(w1)), splat2(1.0f));
  float d0, d1;
  unpack2(den, d0, d1);
  x0 = rcp_approx(d0);
  x1 = rcp_approx(d1);
}

// gelu_erf(x) * sigmoid(x) of two values with two special-function ops per element instead of
// four: erf through Abramowitz-Stegun 7.1.28, erfc(|z|) = 1 / P(|z|)^16 with a degree-6
// polynomial P (|error| < 3e-7, no exponential), and one reciprocal shared with the sigmoid:
//   r = 1 / (P^16 (1 + 2^(-x log2 e))),  erfc = (1 + 2^(-x log2 e)) r,  sigmoid = P^16 r.
// z = x / sqrt 2 is folded into the coefficients.  |x| is clamped at 4 sqrt 2 (erf is 1 to fp32
// beyond) and the exponent at 64 so that the product of the two denominators stays finite.
// The rest is packed arithmetic on the FMA pipe, which the special-function unit runs beside.
__device__ __forceinline__ void gelu_erf_times_sigmoid2(float& x0, float& x1) {
  const f32x2 x = pack2(x0, x1);
  const f32x2 ax = pack2(fminf(fabsf(x0), 5.65685424949238f), fminf(fabsf(x1), 5.65685424949238f));
  f32x2 pq = fma2(ax, splat2(0.0000430638f * 0.125f), splat2(0.0002765672f * 0.17677669529663688f));
  pq = fma2(pq, ax, splat2(0.0001520143f * 0.25f));
  pq = fma2(pq, ax, splat2(0.0092705272f * 0.35355339059327373f));
  pq = fma2(pq, ax, splat2(0.0422820123f * 0.5f));
  pq = fma2(pq, ax, splat2(0.0705230784f * 0.70710678118654752440f));
  pq = fma2(pq, ax, splat2(1.0f));
  pq = mul2(pq, pq);
  pq = mul2(pq, pq);
  pq = mul2(pq, pq);
  pq = mul2(pq, pq);                                            // P^16 <= 5.6e7
  float w0, w1;
  unpack2(mul2(x, splat2(-1.4426950408889634f)), w0, w1);
  const f32x2 den = add2(pack2(ex2_approx(fminf(w0, 64.0f)), ex2_approx(fminf(w1, 64.0f))), splat2(1.0f));
  float q0, q1;
  unpack2(mul2(pq, den), q0, q1);
  const f32x2 r = pack2(rcp_approx(q0), rcp_approx(q1));
  float e0, e1;
  unpack2(fma2(mul2(den, r), splat2(-1.0f), splat2(1.0f)), e0, e1);   // 1 - erfc(|z|) = |erf z|
  const f32x2 erf = pack2(copysignf(e0, x0), copysignf(e1, x1));
  const f32x2 hx = mul2(x, splat2(0.5f));
  unpack2(mul2(fma2(hx, erf, hx), mul2(pq, r)), x0, x1);
}

__device__ __forceinline__ float load_scalar(const void* p, int64_t idx, int32_t dtype) {
  if (dtype == FUSEML_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  if (dtype == FUSEML_F16) return __half2float(reinterpret_cast<const __half*>(p)[idx]);
  return reinterpret_cast<const float*>(p)[idx];
}

// v[i] = combine(v[i], operand[m, n0 + i]) for the CH columns of a chunk, without a CH-element
// temporary: values are folded in as each 16-byte word is unpacked.  combine is a*b for MUL and
// sa*a + sb*b otherwise (ADD: 1,1; SUB: 1,-1; RSUB: -1,1).  Columns >= N are left alone.  The
// fast path (unit column stride, 16-byte aligned, full chunk) uses 128-bit loads; with
// stride_m == 0 all lanes hit the same address and the load broadcasts.
__device__ __forceinline__ float combine(bool mul, float sa, float sb, float a, float b) {
  return mul ? a * b : fmaf(sb, b, sa * a);
}

// the same over a pair of columns: one packed instruction
__device__ __forceinline__ void combine2(bool mul, f32x2 sa, f32x2 sb, float& a0, float& a1, float b0, float b1) {
  const f32x2 a = pack2(a0, a1), b = pack2(b0, b1);
  unpack2(mul ? mul2(a, b) : fma2(sb, b, mul2(sa, a)), a0, a1);
}

template <int CH>
__device__ __forceinline__ void fold_operand_chunk(float (&v)[CH], int32_t code, const EpiOperand& o, int64_t m,
                                                   int32_t n0, int32_t N) {
  const bool mul = code == FUSEML_OP_MUL_T;
  const float sa = code == FUSEML_OP_RSUB_T ? -1.0f : 1.0f;
  const float sb = code == FUSEML_OP_SUB_T ? -1.0f : 1.0f;
  const f32x2 sa2 = splat2(sa), sb2 = splat2(sb);
  const int64_t base = m * o.stride_m + static_cast<int64_t>(n0) * o.stride_n;
  const bool full = (n0 + CH <= N);
  if (o.stride_n == 1 && full) {
    if (o.dtype == FUSEML_F32) {
      const float* p = reinterpret_cast<const float*>(o.ptr) + base;
      if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < CH / 4; ++i) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(p) + i);
          combine2(mul, sa2, sb2, v[4 * i + 0], v[4 * i + 1], q.x, q.y);
          combine2(mul, sa2, sb2, v[4 * i + 2], v[4 * i + 3], q.z, q.w);
        }
        return;
      }
    } else {
      const uint16_t* p = reinterpret_cast<const uint16_t*>(o.ptr) + base;
      if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < CH / 8; ++i) {
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + i);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f;
            if (o.dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            combine2(mul, sa2, sb2, v[8 * i + 2 * j], v[8 * i + 2 * j + 1], f.x, f.y);
          }
        }
        return;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    if (n0 + i < N)
      v[i] = combine(mul, sa, sb, v[i], load_scalar(o.ptr, base + static_cast<int64_t>(i) * o.stride_n, o.dtype));
  }
}

// Derivative of GELU (erf form) at two points: gelu'(x) = Phi(x) + x phi(x)
//   = 0.5 (1 + erf(x / sqrt 2)) + x exp(-x^2 / 2) / sqrt(2 pi),
// with the same erfc approximation as gelu_erf2; the exponential is shared by both terms.
__device__ __forceinline__ void gelu_erf_grad2(float& x0, float& x1) {
  const f32x2 x = pack2(x0, x1);
  const f32x2 ax = pack2(fabsf(x0), fabsf(x1));
  const f32x2 den = fma2(ax, splat2(0.3275911f * 0.70710678118654752440f), splat2(1.0f));
  float d0, d1;
  unpack2(den, d0, d1);
  const f32x2 t = pack2(rcp_approx(d0), rcp_approx(d1));
  f32x2 poly = fma2(t, splat2(1.061405429f), splat2(-1.453152027f));
  poly = fma2(poly, t, splat2(1.421413741f));
  poly = fma2(poly, t, splat2(-0.284496736f));
  poly = fma2(poly, t, splat2(0.254829592f));
  poly = mul2(poly, t);
  float a0, a1;
  unpack2(mul2(mul2(x, x), splat2(-0.5f * 1.4426950408889634f)), a0, a1);
  const f32x2 e = pack2(ex2_approx(a0), ex2_approx(a1));                 // exp(-x^2 / 2)
  float r0, r1;
  unpack2(fma2(poly, mul2(e, splat2(-1.0f)), splat2(1.0f)), r0, r1);   // |erf(x / sqrt 2)|
  const f32x2 erf = pack2(copysignf(r0, x0), copysignf(r1, x1));
  const f32x2 cdf = fma2(erf, splat2(0.5f), splat2(0.5f));
  unpack2(fma2(mul2(x, e), splat2(0.3989422804014327f), cdf), x0, x1);
}

// t[i] = operand[m, n0 + i] as fp32 for the CH columns of a chunk (0 for columns >= N).
template <int CH>
__device__ __forceinline__ void load_operand_chunk(float (&t)[CH], const EpiOperand& o, int64_t m, int32_t n0, int32_t N) {
  const int64_t base = m * o.stride_m + static_cast<int64_t>(n0) * o.stride_n;
  if (o.stride_n == 1 && n0 + CH <= N && o.dtype != FUSEML_F32) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(o.ptr) + base;
    if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < CH / 8; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f;
          if (o.dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
          else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          t[8 * i + 2 * j] = f.x;
          t[8 * i + 2 * j + 1] = f.y;
        }
      }
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < CH; ++i)
    t[i] = (n0 + i < N) ? load_scalar(o.ptr, base + static_cast<int64_t>(i) * o.stride_n, o.dtype) : 0.0f;
}

// v[i] (+|*)= src[i], src = CH fp32 values staged in shared memory (same address for every
// lane: the reads broadcast)
template <bool kMul, int CH>
__device__ __forceinline__ void fold_staged(float (&v)[CH], const float* src) {
#pragma unroll
  for (int i = 0; i < CH / 4; ++i) {
    const float4 q = reinterpret_cast<const float4*>(src)[i];
    const f32x2 lo = pack2(v[4 * i + 0], v[4 * i + 1]), hi = pack2(v[4 * i + 2], v[4 * i + 3]);
    const f32x2 qlo = pack2(q.x, q.y), qhi = pack2(q.z, q.w);
    unpack2(kMul ? mul2(lo, qlo) : add2(lo, qlo), v[4 * i + 0], v[4 * i + 1]);
    unpack2(kMul ? mul2(hi, qhi) : add2(hi, qhi), v[4 * i + 2], v[4 * i + 3]);
  }
}

// The 16 columns of one row of a 128 x 64 box of 16-bit values in shared memory, 128-byte
// swizzle: `piece` points at the first 16-byte piece, the second one sits at piece ^ 16.
__device__ __forceinline__ void fold_tile_smem(float (&v)[16], bool mul, const uint8_t* piece, int32_t dtype) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<uintptr_t>(piece) ^ (h ? 16u : 0u));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f;
      if (dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
      else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      const f32x2 a = pack2(v[8 * h + 2 * j], v[8 * h + 2 * j + 1]), b = pack2(f.x, f.y);
      unpack2(mul ? mul2(a, b) : add2(a, b), v[8 * h + 2 * j], v[8 * h + 2 * j + 1]);
    }
  }
}
__device__ __forceinline__ void store_tile_smem(const float (&v)[16], uint8_t* piece, int32_t dtype) {
  uint32_t packed[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (dtype == FUSEML_BF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(fminf(fmaxf(v[2 * i], -65504.0f), 65504.0f),
                                          fminf(fmaxf(v[2 * i + 1], -65504.0f), 65504.0f));
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  *reinterpret_cast<uint4*>(piece) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  *reinterpret_cast<uint4*>(reinterpret_cast<uintptr_t>(piece) ^ 16u) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// Stores v[0..CH-1] to row pointer `row` (element index n0 .. n0+CH-1) in `dtype`.
// fp16 saturates to +-65504 before the cast, as the reference does
// (fuseml/codegen/kernel_generator.py:1575-1581).
template <int CH>
__device__ __forceinline__ void store_chunk(void* base_ptr, int64_t row_off, int32_t n0, int32_t N,
                                            int32_t dtype, const float (&v)[CH]) {
  const bool full = (n0 + CH <= N);
  if (dtype == FUSEML_F32) {
    float* p = reinterpret_cast<float*>(base_ptr) + row_off + n0;
    if (full && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < CH / 4; ++i) {
        reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) if (n0 + i < N) p[i] = v[i];
    }
    return;
  }
  uint32_t packed[CH / 2];
  if (dtype == FUSEML_BF16) {
#pragma unroll
    for (int i = 0; i < CH / 2; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int i = 0; i < CH / 2; ++i) {
      const float a = fminf(fmaxf(v[2 * i], -65504.0f), 65504.0f);
      const float b = fminf(fmaxf(v[2 * i + 1], -65504.0f), 65504.0f);
      const __half2 h = __floats2half2_rn(a, b);
      packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  uint16_t* p = reinterpret_cast<uint16_t*>(base_ptr) + row_off + n0;
  if (full && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
    for (int i = 0; i < CH / 8; ++i) {
      reinterpret_cast<uint4*>(p)[i] =
          make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      if (n0 + i < N) p[i] = static_cast<uint16_t>((packed[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu);
    }
  }
}

// Runs the program on one chunk.  `row_ok` is false for rows past M: their
// operand loads and aux stores are skipped (values are don't-care).
// `staged` points at this chunk's columns of the row vectors staged in shared memory
// (vector j at staged + j * staged_stride); `mat_piece`, when not null, at this thread's 16
// columns of the matrix operand in a swizzled shared-memory box (ops with reserved == 3).
// How the program is executed (a template argument of the kernels): by the interpreter below,
// without or with the second value register, or as straight-line code for the chains the
// benchmark configurations lower to.  In the interpreter every op is a basic block of its own:
// the loads of an op cannot start before the previous op's arithmetic has drained, and a cheap
// op (bias add, residual add) costs several hundred cycles per chunk in dispatch and exposed
// latency (measured: 323 and 590 cycles per 16-column chunk for four warps per scheduler).  The
// straight-line forms fetch their operands first and leave the scheduling to the compiler.
enum : int {
  kProgGeneric = 0,        // interpreter, no SAVE / SWAP / *_SAVED in the program
  kProgGenericSaved = 1,   // interpreter with the second value register
  kProgBiasGelu = 2,       // ADD_T(staged row vector), GELU_ERF
  kProgBiasAdd = 3,        // ADD_T(staged row vector), ADD_T(matrix)
  kProgBiasGeluSigAdd = 4, // ADD_T(staged row vector), GELU_ERF_MUL_SIGMOID, ADD_T(matrix)
  kProgCount = 5
};

template <int PROG, int CH>
__device__ __forceinline__ void run_program(const GemmParams& p, int64_t m, int32_t n0, bool row_ok,
                                            float (&v)[CH], const float* staged, int32_t staged_stride,
                                            const uint8_t* mat_piece = nullptr) {
  if constexpr (PROG >= kProgBiasGelu) {
    // ---- straight-line forms: operands first, then the arithmetic ----
    constexpr int kMatOp = (PROG == kProgBiasAdd) ? 1 : 2;       // index of the matrix ADD_T
    float4 bias[CH / 4];
#pragma unroll
    for (int i = 0; i < CH / 4; ++i) bias[i] = reinterpret_cast<const float4*>(staged)[i];
    uint4 mat[2];
    bool mat_regs = false;
    if constexpr (PROG != kProgBiasGelu && CH == 16) {
      if (mat_piece != nullptr) {
        mat[0] = *reinterpret_cast<const uint4*>(mat_piece);
        mat[1] = *reinterpret_cast<const uint4*>(reinterpret_cast<uintptr_t>(mat_piece) ^ 16u);
        mat_regs = true;
      }
    }
#pragma unroll
    for (int i = 0; i < CH / 4; ++i) {
      unpack2(add2(pack2(v[4 * i + 0], v[4 * i + 1]), pack2(bias[i].x, bias[i].y)), v[4 * i + 0], v[4 * i + 1]);
      unpack2(add2(pack2(v[4 * i + 2], v[4 * i + 3]), pack2(bias[i].z, bias[i].w)), v[4 * i + 2], v[4 * i + 3]);
    }
    if constexpr (PROG == kProgBiasGelu) {
#pragma unroll
      for (int i = 0; i < CH; i += 2) gelu_erf2(v[i], v[i + 1]);
    } else {
      if constexpr (PROG == kProgBiasGeluSigAdd) {
#pragma unroll
        for (int i = 0; i < CH; i += 2) gelu_erf_times_sigmoid2(v[i], v[i + 1]);
      }
      const EpiOperand& mo = p.operands[p.ops[kMatOp].slot];
      if (mat_regs) {
        if constexpr (CH == 16) {
          const uint32_t w[8] = {mat[0].x, mat[0].y, mat[0].z, mat[0].w, mat[1].x, mat[1].y, mat[1].z, mat[1].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float2 f;
            if (mo.dtype == FUSEML_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            unpack2(add2(pack2(v[2 * j], v[2 * j + 1]), pack2(f.x, f.y)), v[2 * j], v[2 * j + 1]);
          }
        }
      } else if (row_ok) {
        fold_operand_chunk<CH>(v, FUSEML_OP_ADD_T, mo, m, n0, p.N);
      }
    }
    return;
  }
  constexpr bool kUsesSaved = (PROG == kProgGenericSaved);
  float s[kUsesSaved ? CH : 1];
  if (kUsesSaved) {
#pragma unroll
    for (int i = 0; i < (kUsesSaved ? CH : 1); ++i) s[i] = 0.0f;
  }
  for (int op = 0; op < p.n_ops; ++op) {
    const int32_t code = p.ops[op].opcode;
    switch (code) {
      case FUSEML_OP_RELU:
#pragma unroll
        for (int i = 0; i < CH; ++i) v[i] = v[i] > 0.0f ? v[i] : 0.0f;
        break;
      case FUSEML_OP_GELU_ERF:
#pragma unroll
        for (int i = 0; i < CH; i += 2) gelu_erf2(v[i], v[i + 1]);
        break;
      case FUSEML_OP_GELU_TANH:
#pragma unroll
        for (int i = 0; i < CH; i += 2) gelu_tanh2(v[i], v[i + 1]);
        break;
      case FUSEML_OP_SIGMOID:
#pragma unroll
        for (int i = 0; i < CH; i += 2) sigmoid2(v[i], v[i + 1]);
        break;
      case FUSEML_OP_GELU_ERF_MUL_SIGMOID:
#pragma unroll
        for (int i = 0; i < CH; i += 2) gelu_erf_times_sigmoid2(v[i], v[i + 1]);
        break;
      case FUSEML_OP_ADD_IMM: {
        const float c = p.ops[op].imm;
#pragma unroll
        for (int i = 0; i < CH; i += 2) unpack2(add2(pack2(v[i], v[i + 1]), splat2(c)), v[i], v[i + 1]);
      } break;
      case FUSEML_OP_MUL_IMM: {
        const float c = p.ops[op].imm;
#pragma unroll
        for (int i = 0; i < CH; i += 2) unpack2(mul2(pack2(v[i], v[i + 1]), splat2(c)), v[i], v[i + 1]);
      } break;
      case FUSEML_OP_ADD_T:
      case FUSEML_OP_MUL_T:
      case FUSEML_OP_SUB_T:
      case FUSEML_OP_RSUB_T: {
        const int32_t pre = p.ops[op].reserved;
        if (pre == 1 || pre == 2) {
          const float* src = staged + (pre - 1) * staged_stride;
          if (code == FUSEML_OP_ADD_T) fold_staged<false, CH>(v, src); else fold_staged<true, CH>(v, src);
        } else if (pre == 3 && mat_piece != nullptr) {
          // this thread's slice of the matrix operand, brought into shared memory by TMA
          if constexpr (CH == 16) fold_tile_smem(v, code == FUSEML_OP_MUL_T, mat_piece, p.operands[p.ops[op].slot].dtype);
        } else if (row_ok) {
          fold_operand_chunk<CH>(v, code, p.operands[p.ops[op].slot], m, n0, p.N);
        }
      } break;
      case FUSEML_OP_GELU_ERF_BWD_T: {
        if (row_ok) {
          float t[CH];
          load_operand_chunk<CH>(t, p.operands[p.ops[op].slot], m, n0, p.N);
#pragma unroll
          for (int i = 0; i < CH; i += 2) {
            gelu_erf_grad2(t[i], t[i + 1]);
            unpack2(mul2(pack2(v[i], v[i + 1]), pack2(t[i], t[i + 1])), v[i], v[i + 1]);
          }
        }
      } break;
      case FUSEML_OP_STORE_AUX: {
        if (row_ok) {
          const EpiOperand& o = p.operands[p.ops[op].slot];
          store_chunk<CH>(const_cast<void*>(o.ptr), m * o.stride_m, n0, p.N, o.dtype, v);
        }
      } break;
      case FUSEML_OP_SAVE:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < CH; ++i) s[i] = v[i];
        }
        break;
      case FUSEML_OP_SWAP:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < CH; ++i) { const float x = v[i]; v[i] = s[i]; s[i] = x; }
        }
        break;
      case FUSEML_OP_ADD_SAVED:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < CH; i += 2)
            unpack2(add2(pack2(v[i], v[i + 1]), pack2(s[i], s[i + 1])), v[i], v[i + 1]);
        }
        break;
      case FUSEML_OP_MUL_SAVED:
        if (kUsesSaved) {
#pragma unroll
          for (int i = 0; i < CH; i += 2)
            unpack2(mul2(pack2(v[i], v[i + 1]), pack2(s[i], s[i + 1])), v[i], v[i + 1]);
        }
        break;
      default:
        break;
    }
  }
}

}  // namespace epi
}  // namespace fuseml
