// Two-level integer fake quantisation of a weight (Weight48IntegerQuantizer.fake_quant_weight_dynamic,
// llmc/compression/quantization/quant.py:1230-1367): quantise every row to 8 bits (per_channel, an
// int_range such as [-120, 120]), quantise those integer codes to 4 bits per group of 128 with the
// group's scale and zero point clamped to what 8 bits hold, then dequantise back through both levels.
// The reference is a chain of about thirty tensor ops with two full-size intermediates; here a CTA owns
// a row: one read and one write of the weight (HBM-bound, 2 * sizeof(dtype) bytes per element).
//
// Arithmetic is the reference's, op for op, in the weight's dtype (computed in fp32, rounded to the
// dtype after every op), so the result is bit-identical.  The divisions w / s use the reciprocal-and-
// correct scheme of the one-level kernels (exact, see div_rint): at both levels the dividend and the
// scale are values of the dtype (the level-2 dividends are integers of at most 8 bits).
#include <type_traits>

#include "bf16x2.cuh"
#include "lc_common.cuh"

namespace lc {
namespace {

struct LevelCfg {
  float qmin, qmax;
  int sym;
  float s_lo, s_hi, z_lo, z_hi;     // clamps of the scale and the zero point (quant.py:1318-1323)
};

struct W48Args {
  const void* in;
  void* out;
  int64_t rows, cols;
  int group;
  LevelCfg l8, l4;
};

// Weight48IntegerQuantizer.get_qparams (quant.py:1304-1323), every op rounded to T.  Unlike the
// one-level get_qparams the zero point is not clamped to [qmin, qmax] but to [z_lo, z_hi].
template <typename T>
__device__ __forceinline__ void w48_qparams(float mn, float mx, const LevelCfg& c, float& s, float& z) {
  using E = Elem<T>;
  if (c.sym) {
    float a = nan_max(fabsf(mx), fabsf(mn));
    a = E::rnd(nan_max(a, 1e-5f));
    s = E::rnd(__fdiv_rn(a, c.qmax));
    z = 0.f;
  } else {
    float d = E::rnd(__fsub_rn(mx, mn));
    d = E::rnd(nan_max(d, 1e-5f));
    s = E::rnd(__fdiv_rn(d, __fsub_rn(c.qmax, c.qmin)));
    float t = E::rnd(__fdiv_rn(mn, s));
    t = rintf(t);
    z = E::rnd(__fsub_rn(c.qmin, t));
  }
  s = E::rnd(clampf(s, c.s_lo, c.s_hi));     // the clamp bounds need not be values of T
  z = E::rnd(clampf(z, c.z_lo, c.z_hi));
}

template <typename T, int N>
__device__ __forceinline__ void unpack_vec(const uint4& v, float (&f)[N]) {
  const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = Elem<T>::to_f(p[i]);
}
template <typename T, int N>
__device__ __forceinline__ uint4 pack_vec(const float (&f)[N]) {
  uint4 v;
  T* p = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < N; ++i) p[i] = Elem<T>::from_f(f[i]);
  return v;
}

// One CTA per row, V 16-byte vectors per thread in registers; LG = lanes that share a 4-bit group.
template <typename T, int V>
__global__ void __launch_bounds__(256) w48_kernel(W48Args a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec;
  __shared__ float s_mx[8], s_mn[8];
  const int64_t nvec = a.cols / N;
  const int lg = a.group / N;       // power of two, <= 32
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float abs8 = nan_max(fabsf(a.l8.qmin), fabsf(a.l8.qmax));
  const bool z4_small = fabsf(a.l4.z_lo) <= 128.f && fabsf(a.l4.z_hi) <= 128.f;

  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(a.in) + row * nvec;
    uint4* out = reinterpret_cast<uint4*>(a.out) + row * nvec;
    uint4 v[V];
    float mx = -INFINITY, mn = INFINITY;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) {
        v[k] = __ldcs(in + i);
        float f[N];
        unpack_vec<T, N>(v[k], f);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          mx = nan_max(mx, f[e]);
          mn = nan_min(mn, f[e]);
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
    float s8, z8;
    w48_qparams<T>(mn, mx, a.l8, s8, z8);
    const QuantCtx c8 = make_quant_ctx(s8, z8, nan_max(fabsf(mx), fabsf(mn)));
    const QRange qr8{a.l8.qmin, a.l8.qmax};
    const QRange qr4{a.l4.qmin, a.l4.qmax};

    // bf16 rows without NaN / inf / degenerate scale: packed bf16x2 arithmetic (see bf16x2.cuh)
    bool packed = false;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) packed = !c8.exact;
    QuantCtx2 c8p;
    __nv_bfloat162 z8p, s8p;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      c8p = make_ctx2(c8, qr8);
      z8p = c8p.z;
      s8p = c8p.s;
    }

#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      const bool live = i < nvec;
      float q8[N];
      uint32_t q8w[4] = {0u, 0u, 0u, 0u};
      float gmx = -INFINITY, gmn = INFINITY;
      if (live) {
        if (packed) {
          if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
            __nv_bfloat162 mx2 = bf2_of(0xff80ff80u), mn2 = bf2_of(0x7f807f80u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 q = quant2(bf_lo(w[j]), bf_hi(w[j]), c8, c8p);   // step 1
              q8w[j] = u32_of(q);
              mx2 = __hmax2_nan(mx2, q);
              mn2 = __hmin2_nan(mn2, q);
            }
            gmx = nan_max(bf_lo(u32_of(mx2)), bf_hi(u32_of(mx2)));
            gmn = nan_min(bf_lo(u32_of(mn2)), bf_hi(u32_of(mn2)));
          }
        } else {
          float f[N];
          unpack_vec<T, N>(v[k], f);
#pragma unroll
          for (int e = 0; e < N; ++e) {
            q8[e] = int_quant_fast<T>(f[e], c8, qr8);       // step 1: the 8-bit codes, as values of T
            gmx = nan_max(gmx, q8[e]);
            gmn = nan_min(gmn, q8[e]);
          }
        }
      }
      // the lg lanes that hold one group are adjacent and aligned (nvec is a multiple of lg)
      for (int o = lg >> 1; o > 0; o >>= 1) {
        gmx = nan_max(gmx, __shfl_xor_sync(0xffffffffu, gmx, o));
        gmn = nan_min(gmn, __shfl_xor_sync(0xffffffffu, gmn, o));
      }
      if (live) {
        float s4, z4;
        w48_qparams<T>(gmn, gmx, a.l4, s4, z4);
        const QuantCtx c4 = make_quant_ctx(s4, z4, abs8);
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          if (packed && !c4.exact) {
            const QuantCtx2 c4p = make_ctx2(c4, qr4);
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 q4 = quant2(bf_lo(q8w[j]), bf_hi(q8w[j]), c4, c4p);      // step 2
              const __nv_bfloat162 d8 = dequant2(q4, c4p);                                  // step 3
              const __nv_bfloat162 t8 = z8 == 0.f ? d8 : __hsub2(d8, z8p);                  // step 4
              o[j] = u32_of(__hmul2(t8, s8p));
            }
            __stcs(out + i, make_uint4(o[0], o[1], o[2], o[3]));
            continue;
          }
          if (packed) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              q8[2 * j] = bf_lo(q8w[j]);
              q8[2 * j + 1] = bf_hi(q8w[j]);
            }
          }
        }
        float d[N];
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const float q4 = int_quant_fast<T>(q8[e], c4, qr4);                       // step 2
          // step 3: q4 - z4 is an integer; below 256 in magnitude it is exact in every T
          const float t4 = z4_small ? __fsub_rn(q4, z4) : E::rnd(__fsub_rn(q4, z4));
          const float d8 = E::rnd(__fmul_rn(t4, s4));
          // step 4: subtracting a zero zero-point changes nothing; the store rounds the product to T
          const float t8 = z8 == 0.f ? d8 : E::rnd(__fsub_rn(d8, z8));
          d[e] = __fmul_rn(t8, s8);
        }
        __stcs(out + i, pack_vec<T, N>(d));
      }
    }
  }
}

template <typename T>
int w48_dispatch(const W48Args& a, cudaStream_t st) {
  constexpr int N = Elem<T>::kPerVec;
  if (a.cols % N != 0 || a.group % N != 0) return LC_ERR_SHAPE;
  const int lg = a.group / N;
  if (lg < 1 || lg > 32 || (lg & (lg - 1)) != 0) return LC_ERR_SHAPE;
  if (!aligned16(a.in) || !aligned16(a.out)) return LC_ERR_ALIGN;
  const int64_t nvec = a.cols / N;
  if (nvec > 256 * 16) return LC_ERR_SHAPE;
  int64_t blocks = a.rows;
  const int64_t cap = (int64_t)kNumSMsB200 * 8 * 8;
  if (blocks > cap) blocks = cap;
  if (nvec <= 256) w48_kernel<T, 1><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 512) w48_kernel<T, 2><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 1024) w48_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 2048) w48_kernel<T, 8><<<(unsigned)blocks, 256, 0, st>>>(a);
  else w48_kernel<T, 16><<<(unsigned)blocks, 256, 0, st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_rtn_w48_fake_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group,
                                            const lc_w48_level* bit8, const lc_w48_level* bit4, void* out,
                                            lc_stream_t stream) {
  using namespace lc;
  if (!bit8 || !bit4 || rows < 0 || cols < 0) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (!in || !out) return LC_ERR_ARG;
  if (group <= 0 || cols % group != 0) return LC_ERR_SHAPE;     // reshape_tensor raises (quant.py:1289-1302)
  W48Args a;
  a.in = in;
  a.out = out;
  a.rows = rows;
  a.cols = cols;
  a.group = (int)group;
  const lc_w48_level* src[2] = {bit8, bit4};
  LevelCfg* dst[2] = {&a.l8, &a.l4};
  for (int i = 0; i < 2; ++i) {
    if (!(src[i]->qmin < src[i]->qmax) || fabsf(src[i]->qmin) > 128.f || fabsf(src[i]->qmax) > 255.f) return LC_ERR_ARG;
    dst[i]->qmin = src[i]->qmin;
    dst[i]->qmax = src[i]->qmax;
    dst[i]->sym = src[i]->symmetric ? 1 : 0;
    dst[i]->s_lo = src[i]->scales_min;
    dst[i]->s_hi = src[i]->scales_max;
    dst[i]->z_lo = src[i]->zeros_min;
    dst[i]->z_hi = src[i]->zeros_max;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return w48_dispatch<float>(a, st);
    case LC_BF16: return w48_dispatch<__nv_bfloat16>(a, st);
    case LC_F16: return w48_dispatch<__half>(a, st);
    default: return LC_ERR_ARG;
  }
}
