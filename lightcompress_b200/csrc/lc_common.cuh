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

// max / min that propagate NaN like torch.amax / torch.amin
__device__ __forceinline__ float nan_max(float a, float b) { return (a > b || a != a) ? a : b; }
__device__ __forceinline__ float nan_min(float a, float b) { return (a < b || a != a) ? a : b; }
// torch.clamp(x, lo, hi) = min(max(x, lo), hi) with NaN passed through
__device__ __forceinline__ float clampf(float x, float lo, float hi) {
  return (x != x) ? x : fminf(fmaxf(x, lo), hi);
}

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

__device__ __forceinline__ int code_to_int(float q) { return (q != q) ? 0 : __float2int_rn(q); }

}  // namespace lc
