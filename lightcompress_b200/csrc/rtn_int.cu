// Family 1: single-pass integer quant / dequant (RTN) for per-group, per-channel and
// per-token granularity.  HBM-bound: every input element is read once with a 128-bit load
// and every requested output is written once.
//
// Three kernels:
//   group_vec_kernel  group of up to 2 KB: a sub-warp of L lanes owns a group, V vectors per lane,
//                     min/max by xor-shuffles, all lanes derive (scale, zero) redundantly.
//   row_vec_kernel    long rows (per_channel / per_token, or groups > 512 bytes): one CTA per
//                     row segment, the segment stays in registers between reduce and quantise.
//   generic_kernel    any shape / alignment: scalar loads, two passes (second pass hits L2).
#include <type_traits>

#include "lc_common.cuh"

namespace lc {
namespace {

template <typename T> struct Vec16 { uint4 raw; };

template <typename T, int N>
__device__ __forceinline__ void unpack(const uint4& v, float (&f)[N]) {
  const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = Elem<T>::to_f(p[i]);
}
template <typename T, int N>
__device__ __forceinline__ uint4 pack(const float (&f)[N]) {
  uint4 v;
  T* p = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < N; ++i) p[i] = Elem<T>::from_f(f[i]);
  return v;
}

struct QuantArgs {
  const void* col_scale;  // optional per-column multiplier applied (and rounded to T) before everything else
  const void* in;
  const void* scales_in;
  const void* zeros_in;
  void* fake_out;
  void* codes_out;
  void* scales_out;
  void* zeros_out;
  int64_t rows, cols, group, n_groups_total;
  int bits, sym, code_fmt;
  QRange qr;
};

// Writes the codes of one 16-byte input vector (N elements starting at element index e0).
template <int N>
__device__ __forceinline__ void store_codes(const QuantArgs& a, int64_t e0, const float (&q)[N]) {
  if (a.code_fmt == LC_CODES_I32) {
    int32_t* dst = reinterpret_cast<int32_t*>(a.codes_out) + e0;
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      int4 v = make_int4(code_to_int(q[i]), code_to_int(q[i + 1]), code_to_int(q[i + 2]), code_to_int(q[i + 3]));
      *reinterpret_cast<int4*>(dst + i) = v;
    }
  } else if (a.code_fmt == LC_CODES_I8) {
    uint32_t w[N / 4];
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      w[i / 4] = (uint32_t)(code_to_int(q[i]) & 0xff) | ((uint32_t)(code_to_int(q[i + 1]) & 0xff) << 8) |
                 ((uint32_t)(code_to_int(q[i + 2]) & 0xff) << 16) | ((uint32_t)(code_to_int(q[i + 3]) & 0xff) << 24);
    }
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.codes_out) + e0;
    if (N == 4) {
      *reinterpret_cast<uint32_t*>(dst) = w[0];
    } else {
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[N / 4 - 1]);
    }
  } else if (a.code_fmt == LC_CODES_PACK4) {
    const int qmin = (int)a.qr.qmin;
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) w |= (uint32_t)((code_to_int(q[i]) - qmin) & 0xf) << (4 * i);
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.codes_out) + (e0 >> 1);
    if (N == 4) {
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)w;
    } else {
      *reinterpret_cast<uint32_t*>(dst) = w;
    }
  }
}

// ---- kernel A: L lanes per group, V 16-byte vectors per lane -------------------------------------
// Lane j of a group reads vectors j, j+L, j+2L, ... so that every load instruction of a warp
// covers whole 128-byte lines; the V loads of a thread are independent and issued back to back.
template <typename T, int L, int V>
__global__ void __launch_bounds__(256) group_vec_kernel(QuantArgs a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec;
  constexpr int GV = L * V;  // vectors per group
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int sub = lane % L;  // lane inside the group
  const int64_t groups_per_sweep = nthreads / L;
  const int64_t groups_per_row = a.cols / a.group;
  const uint4* in = reinterpret_cast<const uint4*>(a.in);
  const T* s_in = reinterpret_cast<const T*>(a.scales_in);
  const T* z_in = reinterpret_cast<const T*>(a.zeros_in);
  const bool is_static = a.scales_in != nullptr;

  // The loop bound is warp-uniform (first group of the warp) because every lane must reach the
  // full-mask shuffles below; lanes whose own group is past the end are masked by `ok`.
  for (int64_t gw = (tid - lane) / L; gw < a.n_groups_total; gw += groups_per_sweep) {
    const int64_t g = gw + lane / L;
    const bool ok = g < a.n_groups_total;
    float f[V][N];
    float mx = -INFINITY, mn = INFINITY;
    if (ok) {
      uint4 v[V];
      const uint4* src = in + g * GV + sub;
#pragma unroll
      for (int k = 0; k < V; ++k) v[k] = __ldcs(src + L * k);
      if (a.col_scale) {
        // w <- rnd_T(w * s[col]) (the in-place mul_ of AWQ's scaling_weight); groups tile the row
        const int64_t vec_in_row = (g % groups_per_row) * GV + sub;
        const uint4* sc = reinterpret_cast<const uint4*>(a.col_scale) + vec_in_row;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          float w[N], m[N];
          unpack<T, N>(v[k], w);
          unpack<T, N>(__ldg(sc + L * k), m);
#pragma unroll
          for (int i = 0; i < N; ++i) w[i] = E::rnd(__fmul_rn(w[i], m[i]));
          v[k] = pack<T, N>(w);
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) {
        unpack<T, N>(v[k], f[k]);
#pragma unroll
        for (int i = 0; i < N; ++i) {
          mx = nan_max(mx, f[k][i]);
          mn = nan_min(mn, f[k][i]);
        }
      }
    }
    QuantCtx c;
    if (!is_static) {
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) {
        mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      }
      float s, z;
      int_qparams<T>(mn, mx, a.qr, a.sym, s, z);
      c = make_quant_ctx(s, z, nan_max(fabsf(mx), fabsf(mn)));
    } else if (ok) {
      const float s = E::to_f(s_in[g]);
      const float z = (a.sym || z_in == nullptr) ? 0.f : E::to_f(z_in[g]);
      // this thread's own elements decide whether its fast path is safe
      c = make_quant_ctx(s, z, nan_max(fabsf(mx), fabsf(mn)));
    }
    if (!ok) continue;
    const int64_t vbase = g * GV + sub;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float q[N], d[N];
#pragma unroll
      for (int i = 0; i < N; ++i) {
        q[i] = int_quant_fast<T>(f[k][i], c, a.qr);
        d[i] = int_dequant_fast<T>(q[i], c);
      }
      const int64_t vidx = vbase + L * k;
      if (a.fake_out) __stcs(reinterpret_cast<uint4*>(a.fake_out) + vidx, pack<T, N>(d));
      if (a.codes_out) store_codes<N>(a, vidx * N, q);
    }
    if (sub == 0) {
      if (a.scales_out) reinterpret_cast<T*>(a.scales_out)[g] = E::from_f(c.s);
      if (a.zeros_out) reinterpret_cast<T*>(a.zeros_out)[g] = E::from_f(c.z);
    }
  }
}

// ---- kernel A2: bf16, dynamic, dequantised output only -- packed bf16x2 arithmetic ------------------
// For bf16 tensors most of the reference's ops are bf16 ops already, so they map one-to-one onto
// packed bf16x2 instructions with the same round-to-nearest-even: the optional pre-scale w*s[col]
// (HMUL2), round(u) (h2rint), + zero (HADD2), clamp (HMNMX2 with NaN propagation), (q - z) (HSUB2,
// exact) and * scale (HMUL2).  Only the quotient w / s needs fp32 (reciprocal + one correction,
// see div_rint<__nv_bfloat16>); it is rounded to bf16 two at a time by one conversion.
__device__ __forceinline__ __nv_bfloat162 as_bf2(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// quantise + dequantise one 16-byte vector of bf16 values with packed arithmetic (group not `exact`)
__device__ __forceinline__ uint4 bf16_qdq_vec(const uint4& raw, const QuantCtx& c, __nv_bfloat162 s2, __nv_bfloat162 z2,
                                              __nv_bfloat162 qmin2, __nv_bfloat162 qmax2) {
  const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float w0 = __uint_as_float(in[j] << 16), w1 = __uint_as_float(in[j] & 0xffff0000u);
    const float a0 = __fmul_rn(w0, c.r), a1 = __fmul_rn(w1, c.r);
    const float u0 = __fmaf_rn(__fmaf_rn(-a0, c.s, w0), c.r, a0);
    const float u1 = __fmaf_rn(__fmaf_rn(-a1, c.s, w1), c.r, a1);
    __nv_bfloat162 t = h2rint(__floats2bfloat162_rn(u0, u1));
    t = __hmin2_nan(__hmax2_nan(__hadd2(t, z2), qmin2), qmax2);
    o[j] = as_u32(__hmul2(__hsub2(t, z2), s2));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int L, int V>
__global__ void __launch_bounds__(256) group_vec_bf16_fake_kernel(QuantArgs a) {
  using T = __nv_bfloat16;
  using E = Elem<T>;
  constexpr int GV = L * V;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int sub = lane % L;
  const int64_t groups_per_sweep = nthreads / L;
  const int64_t groups_per_row = a.cols / a.group;
  const uint4* in = reinterpret_cast<const uint4*>(a.in);
  const __nv_bfloat162 qmin2 = __float2bfloat162_rn(a.qr.qmin), qmax2 = __float2bfloat162_rn(a.qr.qmax);

  for (int64_t gw = (tid - lane) / L; gw < a.n_groups_total; gw += groups_per_sweep) {
    const int64_t g = gw + lane / L;
    const bool ok = g < a.n_groups_total;
    uint32_t v[V][4];
    __nv_bfloat162 mx2 = __float2bfloat162_rn(-INFINITY), mn2 = __float2bfloat162_rn(INFINITY);
    if (ok) {
      const uint4* src = in + g * GV + sub;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const uint4 t = __ldcs(src + L * k);
        v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
      }
      if (a.col_scale) {
        const uint4* sc = reinterpret_cast<const uint4*>(a.col_scale) + (g % groups_per_row) * GV + sub;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const uint4 m = __ldg(sc + L * k);
          v[k][0] = as_u32(__hmul2(as_bf2(v[k][0]), as_bf2(m.x)));
          v[k][1] = as_u32(__hmul2(as_bf2(v[k][1]), as_bf2(m.y)));
          v[k][2] = as_u32(__hmul2(as_bf2(v[k][2]), as_bf2(m.z)));
          v[k][3] = as_u32(__hmul2(as_bf2(v[k][3]), as_bf2(m.w)));
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mx2 = __hmax2_nan(mx2, as_bf2(v[k][j]));
          mn2 = __hmin2_nan(mn2, as_bf2(v[k][j]));
        }
    }
    float mx = nan_max(__low2float(mx2), __high2float(mx2));
    float mn = nan_min(__low2float(mn2), __high2float(mn2));
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) {
      mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    float s, z;
    int_qparams<T>(mn, mx, a.qr, a.sym, s, z);
    const QuantCtx c = make_quant_ctx(s, z, nan_max(fabsf(mx), fabsf(mn)));
    if (!ok) continue;
    const int64_t vbase = g * GV + sub;
    const __nv_bfloat162 s2 = __float2bfloat162_rn(s), z2 = __float2bfloat162_rn(z);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      uint32_t o[4];
      if (!c.exact) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w0 = __uint_as_float(v[k][j] << 16), w1 = __uint_as_float(v[k][j] & 0xffff0000u);
          const float a0 = __fmul_rn(w0, c.r), a1 = __fmul_rn(w1, c.r);
          const float u0 = __fmaf_rn(__fmaf_rn(-a0, s, w0), c.r, a0);
          const float u1 = __fmaf_rn(__fmaf_rn(-a1, s, w1), c.r, a1);
          __nv_bfloat162 t = h2rint(__floats2bfloat162_rn(u0, u1));
          t = __hmin2_nan(__hmax2_nan(__hadd2(t, z2), qmin2), qmax2);
          o[j] = as_u32(__hmul2(__hsub2(t, z2), s2));
        }
      } else {
        // tiny / huge / non-finite group: the scalar path with the IEEE division
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w0 = __uint_as_float(v[k][j] << 16), w1 = __uint_as_float(v[k][j] & 0xffff0000u);
          const float d0 = int_dequant_fast<T>(int_quant_fast<T>(w0, c, a.qr), c);
          const float d1 = int_dequant_fast<T>(int_quant_fast<T>(w1, c, a.qr), c);
          o[j] = as_u32(__floats2bfloat162_rn(d0, d1));
        }
      }
      __stcs(reinterpret_cast<uint4*>(a.fake_out) + vbase + L * k, make_uint4(o[0], o[1], o[2], o[3]));
    }
    if (sub == 0) {
      if (a.scales_out) reinterpret_cast<T*>(a.scales_out)[g] = E::from_f(s);
      if (a.zeros_out) reinterpret_cast<T*>(a.zeros_out)[g] = E::from_f(z);
    }
  }
}

// ---- kernel B: one CTA per group (a long row segment), V vectors per thread in registers ------
template <typename T, int V>
__global__ void __launch_bounds__(256) row_vec_kernel(QuantArgs a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec;
  __shared__ float s_mx[8], s_mn[8];
  const int64_t nvec = a.group / N;  // vectors per group
  const T* s_in = reinterpret_cast<const T*>(a.scales_in);
  const T* z_in = reinterpret_cast<const T*>(a.zeros_in);
  const bool is_static = a.scales_in != nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int64_t g = blockIdx.x; g < a.n_groups_total; g += gridDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(a.in) + g * nvec;
    uint4 v[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) v[k] = __ldcs(in + i);
    }
    float s, z;
    float mx_all = 0.f, mn_all = 0.f;
    if (!is_static) {
      float mx = -INFINITY, mn = INFINITY;
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        // packed NaN-propagating max / min on two bf16 values per instruction
        __nv_bfloat162 mx2 = __float2bfloat162_rn(-INFINITY), mn2 = __float2bfloat162_rn(INFINITY);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec) {
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              mx2 = __hmax2_nan(mx2, p2[e]);
              mn2 = __hmin2_nan(mn2, p2[e]);
            }
          }
        }
        mx = nan_max(__low2float(mx2), __high2float(mx2));
        mn = nan_min(__low2float(mn2), __high2float(mn2));
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec) {
            float f[N];
            unpack<T, N>(v[k], f);
#pragma unroll
            for (int e = 0; e < N; ++e) {
              mx = nan_max(mx, f[e]);
              mn = nan_min(mn, f[e]);
            }
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      }
      if (lane == 0) {
        s_mx[warp] = mx;
        s_mn[warp] = mn;
      }
      __syncthreads();
      mx = s_mx[0];
      mn = s_mn[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        mx = nan_max(mx, s_mx[w]);
        mn = nan_min(mn, s_mn[w]);
      }
      __syncthreads();
      int_qparams<T>(mn, mx, a.qr, a.sym, s, z);
      mx_all = mx;
      mn_all = mn;
    } else {
      s = E::to_f(s_in[g]);
      z = (a.sym || z_in == nullptr) ? 0.f : E::to_f(z_in[g]);
    }
    // static mode has no min/max: keep the exact division there
    const QuantCtx c = make_quant_ctx(s, z, is_static ? INFINITY : nan_max(fabsf(mx_all), fabsf(mn_all)));
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      if (!c.exact && a.fake_out && !a.codes_out) {
        // bf16 dequantised output only: packed bf16x2 arithmetic (see group_vec_bf16_fake_kernel)
        const __nv_bfloat162 s2 = __float2bfloat162_rn(s), z2 = __float2bfloat162_rn(z);
        const __nv_bfloat162 qmin2 = __float2bfloat162_rn(a.qr.qmin), qmax2 = __float2bfloat162_rn(a.qr.qmax);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec)
            __stcs(reinterpret_cast<uint4*>(a.fake_out) + g * nvec + i, bf16_qdq_vec(v[k], c, s2, z2, qmin2, qmax2));
        }
        if (threadIdx.x == 0) {
          if (a.scales_out) reinterpret_cast<T*>(a.scales_out)[g] = E::from_f(s);
          if (a.zeros_out) reinterpret_cast<T*>(a.zeros_out)[g] = E::from_f(z);
        }
        continue;
      }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) {
        float f[N], q[N], d[N];
        unpack<T, N>(v[k], f);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          q[e] = int_quant_fast<T>(f[e], c, a.qr);
          d[e] = int_dequant_fast<T>(q[e], c);
        }
        const int64_t vidx = g * nvec + i;
        if (a.fake_out) __stcs(reinterpret_cast<uint4*>(a.fake_out) + vidx, pack<T, N>(d));
        if (a.codes_out) store_codes<N>(a, vidx * N, q);
      }
    }
    if (threadIdx.x == 0) {
      if (a.scales_out) reinterpret_cast<T*>(a.scales_out)[g] = E::from_f(s);
      if (a.zeros_out) reinterpret_cast<T*>(a.zeros_out)[g] = E::from_f(z);
    }
  }
}

// ---- kernel C: any group length / alignment; scalar, two passes --------------------------------
template <typename T>
__global__ void __launch_bounds__(256) generic_kernel(QuantArgs a) {
  using E = Elem<T>;
  __shared__ float s_mx[8], s_mn[8];
  const T* s_in = reinterpret_cast<const T*>(a.scales_in);
  const T* z_in = reinterpret_cast<const T*>(a.zeros_in);
  const bool is_static = a.scales_in != nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t g = blockIdx.x; g < a.n_groups_total; g += gridDim.x) {
    const T* in = reinterpret_cast<const T*>(a.in) + g * a.group;
    float s, z;
    if (!is_static) {
      float mx = -INFINITY, mn = INFINITY;
      for (int64_t i = threadIdx.x; i < a.group; i += 256) {
        const float f = E::to_f(in[i]);
        mx = nan_max(mx, f);
        mn = nan_min(mn, f);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      }
      if (lane == 0) {
        s_mx[warp] = mx;
        s_mn[warp] = mn;
      }
      __syncthreads();
      mx = s_mx[0];
      mn = s_mn[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        mx = nan_max(mx, s_mx[w]);
        mn = nan_min(mn, s_mn[w]);
      }
      __syncthreads();
      int_qparams<T>(mn, mx, a.qr, a.sym, s, z);
    } else {
      s = E::to_f(s_in[g]);
      z = (a.sym || z_in == nullptr) ? 0.f : E::to_f(z_in[g]);
    }
    const int qmin = (int)a.qr.qmin;
    // PACK4 pairs never straddle threads: each thread handles element pairs
    for (int64_t i = 2 * (int64_t)threadIdx.x; i < a.group; i += 512) {
      float q2[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (i + e >= a.group) { q2[e] = a.qr.qmin; continue; }
        const float f = E::to_f(in[i + e]);
        const float q = int_quant<T>(f, s, z, a.qr);
        q2[e] = q;
        const int64_t idx = g * a.group + i + e;
        if (a.fake_out) reinterpret_cast<T*>(a.fake_out)[idx] = E::from_f(int_dequant<T>(q, s, z));
        if (a.code_fmt == LC_CODES_I32) reinterpret_cast<int32_t*>(a.codes_out)[idx] = code_to_int(q);
        if (a.code_fmt == LC_CODES_I8) reinterpret_cast<uint8_t*>(a.codes_out)[idx] = (uint8_t)(code_to_int(q) & 0xff);
      }
      if (a.code_fmt == LC_CODES_PACK4) {
        // group and cols are even here (checked on the host)
        reinterpret_cast<uint8_t*>(a.codes_out)[(g * a.group + i) >> 1] =
            (uint8_t)(((code_to_int(q2[0]) - qmin) & 0xf) | (((code_to_int(q2[1]) - qmin) & 0xf) << 4));
      }
    }
    if (threadIdx.x == 0) {
      if (a.scales_out) reinterpret_cast<T*>(a.scales_out)[g] = E::from_f(s);
      if (a.zeros_out) reinterpret_cast<T*>(a.zeros_out)[g] = E::from_f(z);
    }
  }
}

template <typename T, int L, int V>
void launch_group_vec(const QuantArgs& a, cudaStream_t st) {
  const int64_t threads_needed = a.n_groups_total * L;
  int64_t blocks = (threads_needed + 255) / 256;
  const int64_t cap = (int64_t)kNumSMsB200 * 4 * 8;  // a few waves of resident CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    // dynamic fake quant of a bf16 tensor (the RTN / AWQ case): packed-arithmetic kernel
    if (a.fake_out && !a.codes_out && !a.scales_in) {
      group_vec_bf16_fake_kernel<L, V><<<(unsigned)blocks, 256, 0, st>>>(a);
      return;
    }
  }
  group_vec_kernel<T, L, V><<<(unsigned)blocks, 256, 0, st>>>(a);
}

template <typename T>
int dispatch(const QuantArgs& a, cudaStream_t st) {
  constexpr int N = Elem<T>::kPerVec;
  const bool ptr_ok = aligned16(a.in) && (!a.fake_out || aligned16(a.fake_out)) &&
                      (!a.codes_out || aligned16(a.codes_out));
  const bool vec_ok = ptr_ok && (a.group % N == 0);
  const int64_t nvec = a.group / N;  // 16-byte vectors per group
  if (a.col_scale && !(vec_ok && aligned16(a.col_scale) && nvec >= 1 && nvec <= 128 && (nvec & (nvec - 1)) == 0))
    return LC_ERR_SHAPE;  // the column-scaled variant exists for vectorisable groups of up to 2 KB only
  if (vec_ok && nvec <= 128 && (nvec & (nvec - 1)) == 0) {
    switch ((int)nvec) {
      case 128: launch_group_vec<T, 32, 4>(a, st); break;
      case 64: launch_group_vec<T, 16, 4>(a, st); break;
      case 32: launch_group_vec<T, 8, 4>(a, st); break;
      case 16: launch_group_vec<T, 4, 4>(a, st); break;
      case 8: launch_group_vec<T, 2, 4>(a, st); break;
      case 4: launch_group_vec<T, 1, 4>(a, st); break;
      case 2: launch_group_vec<T, 2, 1>(a, st); break;
      default: launch_group_vec<T, 1, 1>(a, st); break;
    }
  } else if (vec_ok && nvec <= 256 * 16) {
    int64_t blocks = a.n_groups_total;
    const int64_t cap = (int64_t)kNumSMsB200 * 8 * 8;
    if (blocks > cap) blocks = cap;
    if (nvec <= 256) row_vec_kernel<T, 1><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 512) row_vec_kernel<T, 2><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 1024) row_vec_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(a);
    else if (nvec <= 2048) row_vec_kernel<T, 8><<<(unsigned)blocks, 256, 0, st>>>(a);
    else row_vec_kernel<T, 16><<<(unsigned)blocks, 256, 0, st>>>(a);
  } else {
    int64_t blocks = a.n_groups_total;
    const int64_t cap = (int64_t)kNumSMsB200 * 8 * 8;
    if (blocks > cap) blocks = cap;
    generic_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(a);
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

static int rtn_quant_impl(const void* in, const void* col_scale, int dtype, int64_t rows, int64_t cols, int64_t group,
                          int bits, int sym, const void* scales_in, const void* zeros_in, void* fake_out,
                          void* codes_out, int code_fmt, void* scales_out, void* zeros_out, lc_stream_t stream) {
  using namespace lc;
  if (rows < 0 || cols < 0 || group < 0) return LC_ERR_ARG;
  if (bits < 2 || bits > 8) return LC_ERR_ARG;
  if (dtype != LC_F32 && dtype != LC_BF16 && dtype != LC_F16) return LC_ERR_ARG;
  if (code_fmt < LC_CODES_NONE || code_fmt > LC_CODES_PACK4) return LC_ERR_ARG;
  if ((code_fmt != LC_CODES_NONE) != (codes_out != nullptr)) return LC_ERR_ARG;
  if (code_fmt == LC_CODES_PACK4 && bits != 4) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (in == nullptr) return LC_ERR_ARG;
  // IntegerQuantizer.reshape_tensor (quant.py:611-631): a last dim shorter than the group is
  // left un-grouped; a non-divisible one is an error.
  if (group == 0 || group > cols) group = cols;
  if (cols % group != 0) return LC_ERR_SHAPE;
  if (code_fmt == LC_CODES_PACK4 && (group % 2 != 0)) return LC_ERR_SHAPE;
  if (scales_in == nullptr && zeros_in != nullptr) return LC_ERR_ARG;

  QuantArgs a;
  a.col_scale = col_scale;
  a.in = in;
  a.scales_in = scales_in;
  a.zeros_in = zeros_in;
  a.fake_out = fake_out;
  a.codes_out = codes_out;
  a.scales_out = scales_out;
  a.zeros_out = zeros_out;
  a.rows = rows;
  a.cols = cols;
  a.group = group;
  a.n_groups_total = rows * (cols / group);
  a.bits = bits;
  a.sym = sym ? 1 : 0;
  a.code_fmt = code_fmt;
  a.qr = int_qrange(bits, a.sym);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return dispatch<float>(a, st);
    case LC_BF16: return dispatch<__nv_bfloat16>(a, st);
    default: return dispatch<__half>(a, st);
  }
}

extern "C" LC_API int lc_rtn_int_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group, int bits,
                                       int sym, const void* scales_in, const void* zeros_in, void* fake_out,
                                       void* codes_out, int code_fmt, void* scales_out, void* zeros_out,
                                       lc_stream_t stream) {
  return rtn_quant_impl(in, nullptr, dtype, rows, cols, group, bits, sym, scales_in, zeros_in, fake_out, codes_out,
                        code_fmt, scales_out, zeros_out, stream);
}

extern "C" LC_API int lc_awq_scale_quant(const void* w, const void* col_scale, int dtype, int64_t rows, int64_t cols,
                                         int64_t group, int bits, int sym, void* fake_out, lc_stream_t stream) {
  if (!col_scale || !fake_out) return LC_ERR_ARG;
  return rtn_quant_impl(w, col_scale, dtype, rows, cols, group, bits, sym, nullptr, nullptr, fake_out, nullptr,
                        LC_CODES_NONE, nullptr, nullptr, stream);
}
