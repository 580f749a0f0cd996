// Element-wise pieces of the calibration block forward (the caller side of the Hessian hooks),
// fused so that each is one pass over HBM instead of the 5-7 separate tensor ops a decoder block's
// stock module code launches.  Each kernel rounds to the tensor dtype after every op of the chain
// it replaces, so the results are bit-identical to that chain:
//
//   rope:     q_embed = (q * cos) + (rotate_half(q) * sin), rotate_half(x) = cat(-x[D/2:], x[:D/2])
//   silu_mul: out = silu(gate) * up, silu(x) = x / (1 + exp(-x)) evaluated in fp32
//   rmsnorm:  out = weight * (x.float() * rsqrt(mean(x.float()^2, -1) + eps)).to(dtype)
//
// Both are HBM-bound: 16-byte vectors, one read of every input, one write of the output.
#include "lc_common.cuh"

namespace lc {
namespace {

template <typename T> struct Vec16;   // 16 bytes of T
template <> struct Vec16<float> { float v[4]; };
template <> struct Vec16<__nv_bfloat16> { __nv_bfloat16 v[8]; };
template <> struct Vec16<__half> { __half v[8]; };

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

// One thread per 16-byte vector of the first half of a head and its partner in the second half.
// x, out: [tokens][heads][D]; cs, sn: [table_tokens][D], token t reading row t % table_tokens (one
// table shared by all sequences of a batch when table_tokens is the sequence length).
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, const T* __restrict__ cs,
                                                   const T* __restrict__ sn, T* __restrict__ out, int64_t tokens,
                                                   int heads, int D, int64_t table_tokens) {
  using E = Elem<T>;
  constexpr int V = E::kPerVec;
  const int half_vecs = D / 2 / V;
  const int64_t total = tokens * heads * half_vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int hv = (int)(idx % half_vecs);
    const int64_t th = idx / half_vecs;          // token * heads + head
    const int64_t tok = (th / heads) % table_tokens;
    const T* xp = x + th * D + hv * V;
    const T* cp = cs + tok * D + hv * V;
    const T* sp = sn + tok * D + hv * V;
    const Vec16<T> x1 = ld16(xp), x2 = ld16(xp + D / 2);
    const Vec16<T> c1 = ld16(cp), c2 = ld16(cp + D / 2);
    const Vec16<T> s1 = ld16(sp), s2 = ld16(sp + D / 2);
    Vec16<T> o1, o2;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float a1 = E::to_f(x1.v[j]), a2 = E::to_f(x2.v[j]);
      // first half: x1 * cos + (-x2) * sin; second half: x2 * cos + x1 * sin
      const float p1 = E::rnd(__fmul_rn(a1, E::to_f(c1.v[j])));
      const float r1 = E::rnd(__fmul_rn(-a2, E::to_f(s1.v[j])));
      const float p2 = E::rnd(__fmul_rn(a2, E::to_f(c2.v[j])));
      const float r2 = E::rnd(__fmul_rn(a1, E::to_f(s2.v[j])));
      o1.v[j] = E::from_f(__fadd_rn(p1, r1));
      o2.v[j] = E::from_f(__fadd_rn(p2, r2));
    }
    T* op = out + th * D + hv * V;
    st16(op, o1);
    st16(op + D / 2, o2);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                       T* __restrict__ out, int64_t n_vec) {
  using E = Elem<T>;
  constexpr int V = E::kPerVec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_vec;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const Vec16<T> g = ld16(gate + idx * V), u = ld16(up + idx * V);
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = E::to_f(g.v[j]);
      const float s = E::rnd(__fdiv_rn(x, __fadd_rn(1.f, expf(-x))));
      o.v[j] = E::from_f(__fmul_rn(s, E::to_f(u.v[j])));
    }
    st16(out + idx * V, o);
  }
}

// RMS norm of one row per warp.  The sum of squares is associated exactly like the row reduction it
// replaces (torch's mean over the last dimension of a contiguous fp32 tensor with 128 <= C < 8192):
// lane l owns the 4-element vectors l, l + 32, l + 64, ... and keeps one running sum per vector
// element, the four sums are folded left to right, and the 32 lane totals are combined by a
// butterfly tree with offsets 16, 8, 4, 2, 1; squares and sums are separate fp32 roundings (no FMA).  `factor` is the
// caller's 1/C as the replaced op computes it (rows / (rows * C) in fp32).
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ weight,
                                                      T* __restrict__ out, int64_t rows, int C, float factor,
                                                      float eps) {
  using E = Elem<T>;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * C;
  T* orow = out + row * C;
  const int n_vec = C >> 7;   // vectors per lane
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  constexpr int kBatch = 8;   // loads in flight per lane
  for (int j0 = 0; j0 < n_vec; j0 += kBatch) {
    float v[kBatch][4];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (j0 + b < n_vec) {
        const T* p = xr + (((j0 + b) << 5) + lane) * 4;
        if constexpr (sizeof(T) == 4) {
          const float4 t = *reinterpret_cast<const float4*>(p);
          v[b][0] = t.x, v[b][1] = t.y, v[b][2] = t.z, v[b][3] = t.w;
        } else {
          const uint2 t = *reinterpret_cast<const uint2*>(p);
          const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
          for (int i = 0; i < 4; ++i) v[b][i] = E::to_f(e[i]);
        }
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (j0 + b < n_vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(v[b][i], v[b][i]));
      }
    }
  }
  float t = __fadd_rn(__fadd_rn(__fadd_rn(acc[0], acc[1]), acc[2]), acc[3]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
  const float r = rsqrtf(__fadd_rn(__fmul_rn(t, factor), eps));

  for (int j = 0; j < n_vec; ++j) {
    const int c = ((j << 5) + lane) * 4;
    if constexpr (sizeof(T) == 4) {
      const float4 a = *reinterpret_cast<const float4*>(xr + c);
      const float4 w = *reinterpret_cast<const float4*>(weight + c);
      float4 o;
      o.x = __fmul_rn(w.x, __fmul_rn(a.x, r));
      o.y = __fmul_rn(w.y, __fmul_rn(a.y, r));
      o.z = __fmul_rn(w.z, __fmul_rn(a.z, r));
      o.w = __fmul_rn(w.w, __fmul_rn(a.w, r));
      *reinterpret_cast<float4*>(orow + c) = o;
    } else {
      const uint2 a = *reinterpret_cast<const uint2*>(xr + c);
      const uint2 w = *reinterpret_cast<const uint2*>(weight + c);
      const T* ae = reinterpret_cast<const T*>(&a);
      const T* we = reinterpret_cast<const T*>(&w);
      uint2 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        oe[i] = E::from_f(__fmul_rn(E::to_f(we[i]), E::rnd(__fmul_rn(E::to_f(ae[i]), r))));
      *reinterpret_cast<uint2*>(orow + c) = o;
    }
  }
}

unsigned grid_for(int64_t work_items, int threads) {
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)kNumSMsB200 * 16;
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

template <typename T>
int rope_launch(const void* x, const void* cs, const void* sn, void* out, int64_t tokens, int heads, int D,
                int64_t table_tokens, cudaStream_t st) {
  const int64_t total = tokens * heads * (D / 2 / Elem<T>::kPerVec);
  rope_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(cs),
                                                       static_cast<const T*>(sn), static_cast<T*>(out), tokens, heads,
                                                       D, table_tokens);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_rope_apply(const void* x, const void* cos_tab, const void* sin_tab, int dtype,
                                    int64_t tokens, int heads, int head_dim, int64_t table_tokens, void* out,
                                    lc_stream_t stream) {
  using namespace lc;
  if (!x || !cos_tab || !sin_tab || !out) return LC_ERR_ARG;
  if (tokens <= 0 || heads <= 0 || head_dim <= 0 || table_tokens <= 0 || tokens % table_tokens != 0) return LC_ERR_ARG;
  const int per_vec = dtype == LC_F32 ? 4 : 8;
  if (head_dim % (2 * per_vec) != 0) return LC_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(cos_tab) || !aligned16(sin_tab) || !aligned16(out)) return LC_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return rope_launch<float>(x, cos_tab, sin_tab, out, tokens, heads, head_dim, table_tokens, st);
    case LC_BF16:
      return rope_launch<__nv_bfloat16>(x, cos_tab, sin_tab, out, tokens, heads, head_dim, table_tokens, st);
    case LC_F16: return rope_launch<__half>(x, cos_tab, sin_tab, out, tokens, heads, head_dim, table_tokens, st);
    default: return LC_ERR_ARG;
  }
}

extern "C" LC_API int lc_silu_mul(const void* gate, const void* up, int dtype, int64_t n, void* out,
                                  lc_stream_t stream) {
  using namespace lc;
  if (!gate || !up || !out || n <= 0) return LC_ERR_ARG;
  const int per_vec = dtype == LC_F32 ? 4 : 8;
  if (n % per_vec != 0) return LC_ERR_SHAPE;
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return LC_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_vec = n / per_vec;
  const unsigned grid = grid_for(n_vec, 256);
  switch (dtype) {
    case LC_F32:
      silu_mul_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(gate), static_cast<const float*>(up),
                                                   static_cast<float*>(out), n_vec);
      break;
    case LC_BF16:
      silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate),
                                                           static_cast<const __nv_bfloat16*>(up),
                                                           static_cast<__nv_bfloat16*>(out), n_vec);
      break;
    case LC_F16:
      silu_mul_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                                    static_cast<__half*>(out), n_vec);
      break;
    default: return LC_ERR_ARG;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_rmsnorm(const void* x, const void* weight, int dtype, int64_t rows, int64_t cols,
                                 float mean_factor, float eps, void* out, lc_stream_t stream) {
  using namespace lc;
  if (!x || !weight || !out || rows <= 0 || cols <= 0) return LC_ERR_ARG;
  if (cols % 128 != 0 || cols >= 8192) return LC_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out)) return LC_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows + 7) / 8);
  switch (dtype) {
    case LC_F32:
      rmsnorm_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(weight),
                                                  static_cast<float*>(out), rows, (int)cols, mean_factor, eps);
      break;
    case LC_BF16:
      rmsnorm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                          static_cast<const __nv_bfloat16*>(weight),
                                                          static_cast<__nv_bfloat16*>(out), rows, (int)cols,
                                                          mean_factor, eps);
      break;
    case LC_F16:
      rmsnorm_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(weight),
                                                   static_cast<__half*>(out), rows, (int)cols, mean_factor, eps);
      break;
    default: return LC_ERR_ARG;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}
