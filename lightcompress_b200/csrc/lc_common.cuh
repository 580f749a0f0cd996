// Shared helpers for the sm_100a kernels: status codes, element-type traits and the
// "compute in fp32, round to the tensor dtype after every op" arithmetic that makes the
// fused kernels bit-identical to a chain of separate torch ops.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lc_b200.h"

#define LC_API __attribute__((visibility("default")))

#define LC_CHECK_CUDA(expr)                      \
  do {                                           \
    cudaError_t _e = (expr);                     \
    if (_e != cudaSuccess) return LC_ERR_CUDA;   \
  } while (0)

#define LC_LAUNCH_CHECK()                              \
  do {                                                 \
    if (cudaGetLastError() != cudaSuccess) return LC_ERR_CUDA; \
  } while (0)

namespace lc {

constexpr int kNumSMsB200 = 148;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_size(int dt) { return dt == LC_F32 ? 4 : 2; }

// ---- element traits -------------------------------------------------------------------------
template <typename T> struct Elem;

template <> struct Elem<float> {
  static constexpr int kPerVec = 4;  // elements per 16-byte vector
  __device__ __forceinline__ static float to_f(float v) { return v; }
  __device__ __forceinline__ static float from_f(float v) { return v; }
  // round an fp32 intermediate to the tensor dtype and come back to fp32
  __device__ __forceinline__ static float rnd(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  __device__ __forceinline__ static float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Elem<__half> {
  static constexpr int kPerVec = 8;
  __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
  __device__ __forceinline__ static float rnd(float v) { return __half2float(__float2half_rn(v)); }
};

// max / min that propagate NaN like torch.amax / torch.amin (one FMNMX.NAN each)
__device__ __forceinline__ float nan_max(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float nan_min(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// torch.clamp(x, lo, hi) = min(max(x, lo), hi) with NaN passed through
__device__ __forceinline__ float clampf(float x, float lo, float hi) { return nan_min(nan_max(x, lo), hi); }

// ---- integer quantisation parameters (IntegerQuantizer.get_qparams) ---------------------------
struct QRange {
  float qmin, qmax;
};
__host__ __device__ inline QRange int_qrange(int bits, int sym) {
  QRange r;
  if (sym) {
    r.qmin = -(float)(1 << (bits - 1));
    r.qmax = (float)((1 << (bits - 1)) - 1);
  } else {
    r.qmin = 0.f;
    r.qmax = (float)((1 << bits) - 1);
  }
  return r;
}

// scale / zero from a group's min and max, every op rounded to T.
template <typename T>
__device__ __forceinline__ void int_qparams(float mn, float mx, QRange qr, int sym, float& s, float& z) {
  using E = Elem<T>;
  if (sym) {
    float a = nan_max(fabsf(mx), fabsf(mn));
    a = E::rnd(nan_max(a, 1e-5f));      // clamp(min=1e-5) on a tensor of dtype T
    s = E::rnd(__fdiv_rn(a, qr.qmax));
    z = 0.f;
  } else {
    float d = E::rnd(__fsub_rn(mx, mn));
    d = E::rnd(nan_max(d, 1e-5f));
    s = E::rnd(__fdiv_rn(d, __fsub_rn(qr.qmax, qr.qmin)));
    float t = E::rnd(__fdiv_rn(mn, s));
    t = rintf(t);
    t = E::rnd(__fsub_rn(qr.qmin, t));
    z = clampf(t, qr.qmin, qr.qmax);
  }
}

// clamp(round(w / s) + z, qmin, qmax); returns the code as a float holding an integer
template <typename T>
__device__ __forceinline__ float int_quant(float w, float s, float z, QRange qr) {
  using E = Elem<T>;
  float u = E::rnd(__fdiv_rn(w, s));
  u = rintf(u);
  u = E::rnd(__fadd_rn(u, z));
  return clampf(u, qr.qmin, qr.qmax);
}

// (q - z) * s
template <typename T>
__device__ __forceinline__ float int_dequant(float q, float s, float z) {
  using E = Elem<T>;
  return E::rnd(__fmul_rn(E::rnd(__fsub_rn(q, z)), s));
}

// ---- fast exact quantisation ---------------------------------------------------------------------
// The element-wise cost of the fused kernels is dominated by the IEEE division w / s.  The scale is
// shared by a whole group, so its reciprocal is computed once (QuantCtx) and each element uses
//   q0 = w * r;  e = fma(-q0, s, w);  q1 = fma(e, r, q0)
// which is within one ulp of RN(w / s) and almost always equal to it.  The result only feeds a
// rounding (to T, then to an integer), so it can differ from the exact path only when q1 sits
// within an ulp of a rounding boundary; those elements (and non-finite ones) take the IEEE
// division.  Codes and dequantised values therefore stay bit-identical to the reference's.
struct QuantCtx {
  float s, z, r;   // scale, zero point, 1/s
  bool exact;      // use the IEEE division for every element of the group
};

// absmax: largest |w| the context will be used on (NaN / inf allowed: they select the exact path)
__device__ __forceinline__ QuantCtx make_quant_ctx(float s, float z, float absmax) {
  QuantCtx c;
  c.s = s;
  c.z = z;
  c.r = __frcp_rn(s);
  // Keep the IEEE division when the reciprocal would lose accuracy (tiny / huge / non-finite
  // scale) or when w * r could overflow or is not finite; every comparison is false for NaN.
  c.exact = !(s > 1e-30f && s < 1e30f) || !(__fmul_rn(absmax, c.r) < 1e37f);
  return c;
}

// IEEE division kept out of line: the rare slow path must be a real branch, not a predicated
// copy of the whole division sequence in every element's instruction stream.
static __device__ __noinline__ float ieee_div(float a, float b) { return __fdiv_rn(a, b); }

// rint(rnd_T(w / s)) -- exactly what torch.round(w / s) gives on a tensor of dtype T.
// In the saturated region (|result| > 1024) the integer may be off by one; it is clamped anyway.
template <typename T>
__device__ __forceinline__ float div_rint(float w, const QuantCtx& c);

template <>
__device__ __forceinline__ float div_rint<float>(float w, const QuantCtx& c) {
  if (c.exact) return rintf(ieee_div(w, c.s));
  const float q0 = __fmul_rn(w, c.r);
  const float e = __fmaf_rn(-q0, c.s, w);
  const float q1 = __fmaf_rn(e, c.r, q0);
  float k = rintf(q1);
  // within 1e-4 of a half-integer (more than an ulp for |q1| <= 1024), or NaN / inf
  if (!(fabsf(fabsf(__fsub_rn(q1, k)) - 0.5f) >= 1e-4f)) k = rintf(ieee_div(w, c.s));
  return k;
}

template <>
__device__ __forceinline__ float div_rint<__nv_bfloat16>(float w, const QuantCtx& c) {
  if (c.exact) return rintf(Elem<__nv_bfloat16>::rnd(ieee_div(w, c.s)));
  // w and s are bf16 values (8-bit significands a, b).  The quotient a/b is either exactly a
  // bf16 rounding midpoint (9 significant bits) or at least 1/(512*255) ~ 7.7e-6 away from every
  // midpoint in relative terms -- 64 fp32 ulps.  q1 is within one ulp of RN(w/s) and equals the
  // quotient whenever that is representable, so rounding q1 to bf16 gives the reference's value
  // with no boundary check.
  const float q0 = __fmul_rn(w, c.r);
  const float e = __fmaf_rn(-q0, c.s, w);
  const float q1 = __fmaf_rn(e, c.r, q0);
  return rintf(Elem<__nv_bfloat16>::rnd(q1));
}

template <>
__device__ __forceinline__ float div_rint<__half>(float w, const QuantCtx& c) {
  return rintf(Elem<__half>::rnd(__fdiv_rn(w, c.s)));   // fp16 keeps the inline IEEE division
}

// clamp(round(w / s) + z, qmin, qmax) through the fast division.  For codes of at most 8 bits the
// sum of two integers needs no rounding to T: it is exact up to 256 and saturates beyond.
template <typename T>
__device__ __forceinline__ float int_quant_fast(float w, const QuantCtx& c, QRange qr) {
  return clampf(__fadd_rn(div_rint<T>(w, c), c.z), qr.qmin, qr.qmax);
}

// (q - z) * s rounded to T; q - z is an integer of magnitude <= 255, exact in every T.
template <typename T>
__device__ __forceinline__ float int_dequant_fast(float q, const QuantCtx& c) {
  return __fmul_rn(__fsub_rn(q, c.z), c.s);   // the caller's conversion to T is the rounding
}

__device__ __forceinline__ int code_to_int(float q) { return (q != q) ? 0 : __float2int_rn(q); }

}  // namespace lc
