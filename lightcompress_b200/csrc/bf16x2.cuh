// Packed bf16x2 forms of the integer quantise / dequantise chain, for bf16 tensors.
//
// On a bf16 tensor most of the reference's ops are bf16 ops already, so they map one-to-one onto packed
// instructions with the same round-to-nearest-even: round(u) (h2rint), + zero point (HADD2), clamp
// (HMNMX2 with NaN propagation), q - z (HSUB2) and * scale (HMUL2).  Only the quotient w / s needs fp32
// (reciprocal and one correction, see div_rint<__nv_bfloat16>: exact when w and s are bf16 values and
// the context is not `exact`); the two quotients are rounded to bf16 by one conversion.
#pragma once

#include "lc_common.cuh"

namespace lc {

__device__ __forceinline__ __nv_bfloat162 bf2_of(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t u32_of(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// per-context constants as bf16 pairs
struct QuantCtx2 {
  __nv_bfloat162 s, z, qmin, qmax;
};
__device__ __forceinline__ QuantCtx2 make_ctx2(const QuantCtx& c, QRange qr) {
  QuantCtx2 p;
  p.s = __float2bfloat162_rn(c.s);
  p.z = __float2bfloat162_rn(c.z);
  p.qmin = __float2bfloat162_rn(qr.qmin);
  p.qmax = __float2bfloat162_rn(qr.qmax);
  return p;
}

// clamp(round(w / s) + z, qmin, qmax) for two values; c must not be `exact`
__device__ __forceinline__ __nv_bfloat162 quant2(float w0, float w1, const QuantCtx& c, const QuantCtx2& p) {
  const float a0 = __fmul_rn(w0, c.r), a1 = __fmul_rn(w1, c.r);
  const float u0 = __fmaf_rn(__fmaf_rn(-a0, c.s, w0), c.r, a0);
  const float u1 = __fmaf_rn(__fmaf_rn(-a1, c.s, w1), c.r, a1);
  const __nv_bfloat162 t = h2rint(__floats2bfloat162_rn(u0, u1));
  return __hmin2_nan(__hmax2_nan(__hadd2(t, p.z), p.qmin), p.qmax);
}

// (q - z) * s
__device__ __forceinline__ __nv_bfloat162 dequant2(__nv_bfloat162 q, const QuantCtx2& p) {
  return __hmul2(__hsub2(q, p.z), p.s);
}

}  // namespace lc
