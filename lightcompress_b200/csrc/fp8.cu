// Family 1 (float): FP8 e4m3 per-row quant / dequant for per_channel weights and per_token
// activations.  One CTA per row; the row stays in registers between the abs-max reduction and
// the quantise pass, so HBM is read once.  Rows that are not 16-byte vectorisable take the
// scalar two-pass kernel.
#include <cuda_fp8.h>

#include <type_traits>

#include "lc_common.cuh"

namespace lc {
namespace {

struct Fp8Args {
  const void* in;
  void* fake_out;
  void* codes_out;
  void* scales_out;
  int64_t rows, cols;
};

// scale = clamp(absmax, 1e-5) / 448 in dtype T; a scale that rounds to zero becomes 1
// (FloatQuantizer.get_qparams / quant, quant.py:544-551, :1061).
template <typename T>
__device__ __forceinline__ float fp8_scale(float absmax) {
  using E = Elem<T>;
  float a = E::rnd(nan_max(absmax, 1e-5f));
  float s = E::rnd(__fdiv_rn(a, 448.f));
  return (s == 0.f) ? 1.f : s;
}

// rnd_T(w / s).  For bf16 the reciprocal-based quotient rounds to the same bf16 value as the IEEE
// one (see div_rint<__nv_bfloat16>); the other types keep the IEEE division.
template <typename T>
__device__ __forceinline__ float fp8_div(float w, float s, float r, bool exact) {
  return Elem<T>::rnd(__fdiv_rn(w, s));
}
template <>
__device__ __forceinline__ float fp8_div<__nv_bfloat16>(float w, float s, float r, bool exact) {
  if (exact) return Elem<__nv_bfloat16>::rnd(ieee_div(w, s));
  const float q0 = __fmul_rn(w, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-q0, s, w), r, q0);
  return Elem<__nv_bfloat16>::rnd(q1);
}

// u = w / s + 0 in T, q = e4m3(u) as fp32, fake = T(q * s)
template <typename T>
__device__ __forceinline__ void fp8_one(float w, float s, float r, bool exact, float& fake, uint8_t& code) {
  using E = Elem<T>;
  float u = fp8_div<T>(w, s, r, exact);
  u = E::rnd(__fadd_rn(u, 0.f));
  const __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(u, __NV_SATFINITE, __NV_E4M3);
  code = (uint8_t)c;
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
  const float q = __half2float(__half(hr));
  fake = E::rnd(__fmul_rn(__fsub_rn(q, 0.f), s));
}

__device__ __forceinline__ float block_absmax(float a, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = nan_max(a, __shfl_xor_sync(0xffffffffu, a, o));
  if (lane == 0) smem[warp] = a;
  __syncthreads();
  a = smem[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) a = nan_max(a, smem[w]);
  __syncthreads();
  return a;
}

// bf16 rows: quotient in fp32 (reciprocal + one correction), everything else packed bf16x2 -- the
// reference's ops on a bf16 tensor are bf16 ops: u = w/s, u + 0, e4m3 round, q * s.
__device__ __forceinline__ void fp8_bf16_vec(const uint4& raw, float s, float rs, __nv_bfloat162 s2, uint4& fake,
                                             uint2& codes) {
  const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[4];
  uint16_t cpair[4];
  const __nv_bfloat162 zero2 = __float2bfloat162_rn(0.f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float w0 = __uint_as_float(in[j] << 16), w1 = __uint_as_float(in[j] & 0xffff0000u);
    const float a0 = __fmul_rn(w0, rs), a1 = __fmul_rn(w1, rs);
    const float u0 = __fmaf_rn(__fmaf_rn(-a0, s, w0), rs, a0);
    const float u1 = __fmaf_rn(__fmaf_rn(-a1, s, w1), rs, a1);
    const __nv_bfloat162 u2 = __hadd2(__floats2bfloat162_rn(u0, u1), zero2);
    const __nv_fp8x2_storage_t c2 =
        __nv_cvt_bfloat16raw2_to_fp8x2(*reinterpret_cast<const __nv_bfloat162_raw*>(&u2), __NV_SATFINITE, __NV_E4M3);
    cpair[j] = (uint16_t)c2;
    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(c2, __NV_E4M3);
    const float2 qf = __half22float2(*reinterpret_cast<const __half2*>(&hr));
    const __nv_bfloat162 q2 = __floats2bfloat162_rn(qf.x, qf.y);   // e4m3 values are exact in bf16
    const __nv_bfloat162 f2 = __hmul2(__hsub2(q2, zero2), s2);
    o[j] = *reinterpret_cast<const uint32_t*>(&f2);
  }
  fake = make_uint4(o[0], o[1], o[2], o[3]);
  codes = make_uint2((uint32_t)cpair[0] | ((uint32_t)cpair[1] << 16), (uint32_t)cpair[2] | ((uint32_t)cpair[3] << 16));
}

template <typename T, int V>
__global__ void __launch_bounds__(256) fp8_row_vec_kernel(Fp8Args a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec;
  __shared__ float smem[8];
  const int64_t nvec = a.cols / N;
  for (int64_t r = blockIdx.x; r < a.rows; r += gridDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(a.in) + r * nvec;
    uint4 v[V];
    float am = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) v[k] = __ldcs(in + i);
    }
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      // packed: |x| and the NaN-propagating maximum on two bf16 values per instruction
      __nv_bfloat162 am2 = __float2bfloat162_rn(0.f);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const int64_t i = threadIdx.x + (int64_t)k * 256;
        if (i < nvec) {
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
          for (int e = 0; e < 4; ++e) am2 = __hmax2_nan(am2, __habs2(p2[e]));
        }
      }
      am = nan_max(__low2float(am2), __high2float(am2));
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const int64_t i = threadIdx.x + (int64_t)k * 256;
        if (i < nvec) {
          const T* p = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
          for (int e = 0; e < N; ++e) am = nan_max(am, fabsf(E::to_f(p[e])));
        }
      }
    }
    am = block_absmax(am, smem);
    const float s = fp8_scale<T>(am);
    const float rs = __frcp_rn(s);
    const bool exact = !(s > 1e-30f && s < 1e30f) || !(__fmul_rn(am, rs) < 1e37f);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      if (!exact) {
        const __nv_bfloat162 s2 = __float2bfloat162_rn(s);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec) {
            uint4 fake;
            uint2 cds;
            fp8_bf16_vec(v[k], s, rs, s2, fake, cds);
            const int64_t vidx = r * nvec + i;
            if (a.fake_out) __stcs(reinterpret_cast<uint4*>(a.fake_out) + vidx, fake);
            if (a.codes_out) *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(a.codes_out) + vidx * 8) = cds;
          }
        }
        if (threadIdx.x == 0 && a.scales_out) reinterpret_cast<T*>(a.scales_out)[r] = E::from_f(s);
        continue;
      }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) {
        const T* p = reinterpret_cast<const T*>(&v[k]);
        uint4 outv;
        T* o = reinterpret_cast<T*>(&outv);
        uint8_t codes[N];
#pragma unroll
        for (int e = 0; e < N; ++e) {
          float fake;
          fp8_one<T>(E::to_f(p[e]), s, rs, exact, fake, codes[e]);
          o[e] = E::from_f(fake);
        }
        const int64_t vidx = r * nvec + i;
        if (a.fake_out) __stcs(reinterpret_cast<uint4*>(a.fake_out) + vidx, outv);
        if (a.codes_out) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(a.codes_out) + vidx * N;
          uint32_t w0 = codes[0] | (codes[1] << 8) | (codes[2] << 16) | ((uint32_t)codes[3] << 24);
          if (N == 4) {
            *reinterpret_cast<uint32_t*>(dst) = w0;
          } else {
            uint32_t w1 = codes[N - 4] | (codes[N - 3] << 8) | (codes[N - 2] << 16) | ((uint32_t)codes[N - 1] << 24);
            *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
          }
        }
      }
    }
    if (threadIdx.x == 0 && a.scales_out) reinterpret_cast<T*>(a.scales_out)[r] = E::from_f(s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fp8_generic_kernel(Fp8Args a) {
  using E = Elem<T>;
  __shared__ float smem[8];
  for (int64_t r = blockIdx.x; r < a.rows; r += gridDim.x) {
    const T* in = reinterpret_cast<const T*>(a.in) + r * a.cols;
    float am = 0.f;
    for (int64_t i = threadIdx.x; i < a.cols; i += 256) am = nan_max(am, fabsf(E::to_f(in[i])));
    am = block_absmax(am, smem);
    const float s = fp8_scale<T>(am);
    const float rs = __frcp_rn(s);
    const bool exact = !(s > 1e-30f && s < 1e30f) || !(__fmul_rn(am, rs) < 1e37f);
    for (int64_t i = threadIdx.x; i < a.cols; i += 256) {
      float fake;
      uint8_t code;
      fp8_one<T>(E::to_f(in[i]), s, rs, exact, fake, code);
      if (a.fake_out) reinterpret_cast<T*>(a.fake_out)[r * a.cols + i] = E::from_f(fake);
      if (a.codes_out) reinterpret_cast<uint8_t*>(a.codes_out)[r * a.cols + i] = code;
    }
    if (threadIdx.x == 0 && a.scales_out) reinterpret_cast<T*>(a.scales_out)[r] = E::from_f(s);
  }
}

template <typename T>
int dispatch(const Fp8Args& a, cudaStream_t st) {
  constexpr int N = Elem<T>::kPerVec;
  int64_t blocks = a.rows;
  const int64_t cap = (int64_t)kNumSMsB200 * 8 * 8;
  if (blocks > cap) blocks = cap;
  const bool vec_ok = aligned16(a.in) && (!a.fake_out || aligned16(a.fake_out)) &&
                      (!a.codes_out || aligned16(a.codes_out)) && (a.cols % N == 0);
  const int64_t nvec = a.cols / N;
  if (vec_ok && nvec <= 256 * 16) {
    if (nvec <= 256) fp8_row_vec_kernel<T, 1><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 512) fp8_row_vec_kernel<T, 2><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 1024) fp8_row_vec_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 2048) fp8_row_vec_kernel<T, 8><<<(unsigned)blocks, 256, 0, st>>>(a);
    else fp8_row_vec_kernel<T, 16><<<(unsigned)blocks, 256, 0, st>>>(a);
  } else {
    fp8_generic_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(a);
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_fp8_e4m3_quant(const void* in, int dtype, int64_t rows, int64_t cols, void* fake_out,
                                 void* codes_out, void* scales_out, lc_stream_t stream) {
  using namespace lc;
  if (rows < 0 || cols < 0) return LC_ERR_ARG;
  if (dtype != LC_F32 && dtype != LC_BF16 && dtype != LC_F16) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (in == nullptr) return LC_ERR_ARG;
  Fp8Args a{in, fake_out, codes_out, scales_out, rows, cols};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return dispatch<float>(a, st);
    case LC_BF16: return dispatch<__nv_bfloat16>(a, st);
    default: return dispatch<__half>(a, st);
  }
}
