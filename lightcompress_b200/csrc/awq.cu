// Family 4: AWQ scale + clip search helpers.
//
//   act_mean     x_bar[c] = mean_t |x[t][c]|                       (one pass over x, deterministic)
//   div_cols     x / s[col], rounded to the tensor dtype            (scaling_input)
//   loss         mean((a - b)^2) with the subtraction rounded to T  (calculate_loss)
//   clip_search  per (row, group): 10-point clip grid with the reference's per-op rounding, keeps
//                the best range and clamps the weights -- no (rows x tokens x groups x 128)
//                intermediate ever leaves the SM.
//
// The decisions of the clip search are dominated by rounding noise, so the arithmetic follows the
// reference op by op for 16-bit tensors: every product x*w is rounded to T (one HMUL2 per two
// products), the 128-term sum is accumulated in fp32 and rounded to T once, the difference, its
// square and the mean over tokens are each rounded to T, and comparisons are strict.
#include "lc_common.cuh"

namespace lc {
namespace {

// ---- act_mean -----------------------------------------------------------------------------------
// Stage 1: grid (column slabs of 256, token splits); block (32, 8): thread = one 8-column vector,
// 8 row phases.  Stage 2 adds the splits in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) abs_sum_kernel(const T* x, int64_t tokens, int64_t cols, float* partial) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * N;
  const int64_t per = (tokens + gridDim.y - 1) / gridDim.y;
  const int64_t t0 = blockIdx.y * per, t1 = min(tokens, t0 + per);
  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.f;
  if (c0 < cols) {
    for (int64_t t = t0 + threadIdx.y; t < t1; t += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + t * cols + c0);
      const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += fabsf(Elem<T>::to_f(p[i]));
    }
  }
  __shared__ float red[8][32][N + 1];
#pragma unroll
  for (int i = 0; i < N; ++i) red[threadIdx.y][threadIdx.x][i] = acc[i];
  __syncthreads();
  if (threadIdx.y == 0 && c0 < cols) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) s += red[r][threadIdx.x][i];
      partial[(int64_t)blockIdx.y * cols + c0 + i] = s;
    }
  }
}

template <typename T>
__global__ void abs_mean_finish_kernel(const float* partial, int splits, int64_t tokens, int64_t cols, T* out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += partial[(int64_t)k * cols + c];
  out[c] = Elem<T>::from_f(__fdiv_rn(s, (float)tokens));
}

// ---- div_cols -----------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float div_rnd(float w, float s, float r) { return Elem<T>::rnd(__fdiv_rn(w, s)); }
template <>
__device__ __forceinline__ float div_rnd<__nv_bfloat16>(float w, float s, float r) {
  // same bf16 value as the IEEE quotient (see div_rint<__nv_bfloat16>); non-finite / extreme
  // operands fall back to the IEEE division
  const float q0 = __fmul_rn(w, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-q0, s, w), r, q0);
  if (!(fabsf(q1) < 1e37f) || !(s > 1e-30f && s < 1e30f)) return Elem<__nv_bfloat16>::rnd(ieee_div(w, s));
  return Elem<__nv_bfloat16>::rnd(q1);
}

template <typename T>
__global__ void __launch_bounds__(256) div_cols_kernel(const T* x, const T* s, int64_t rows, int64_t cols, T* out) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * N;
  if (c0 >= cols) return;
  float sv[N], rv[N];
  {
    const uint4 v = *reinterpret_cast<const uint4*>(s + c0);
    const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      sv[i] = Elem<T>::to_f(p[i]);
      rv[i] = __frcp_rn(sv[i]);
    }
  }
  // four rows per iteration: four 16-byte loads in flight per thread
  constexpr int U = 4;
  const int64_t stride = (int64_t)gridDim.y * 8;
  for (int64_t r0 = (int64_t)blockIdx.y * 8 + threadIdx.y; r0 < rows; r0 += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < rows) v[u] = __ldcs(reinterpret_cast<const uint4*>(x + r * cols + c0));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * stride;
      if (r >= rows) break;
      const T* p = reinterpret_cast<const T*>(&v[u]);
      uint4 o;
      T* q = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int i = 0; i < N; ++i) q[i] = Elem<T>::from_f(div_rnd<T>(Elem<T>::to_f(p[i]), sv[i], rv[i]));
      __stcs(reinterpret_cast<uint4*>(out + r * cols + c0), o);
    }
  }
}

// ---- loss ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sq_diff_partial_kernel(const T* a, const T* b, int64_t n, double* partial) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t nvec = n / N;
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * 256) {
    const uint4 va = __ldcs(reinterpret_cast<const uint4*>(a) + i);
    const uint4 vb = __ldcs(reinterpret_cast<const uint4*>(b) + i);
    const T* pa = reinterpret_cast<const T*>(&va);
    const T* pb = reinterpret_cast<const T*>(&vb);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float d = Elem<T>::rnd(__fsub_rn(Elem<T>::to_f(pa[k]), Elem<T>::to_f(pb[k])));
      acc = fmaf(d, d, acc);
    }
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * N + threadIdx.x; i < n; i += 256) {
      const float d = Elem<T>::rnd(__fsub_rn(Elem<T>::to_f(a[i]), Elem<T>::to_f(b[i])));
      acc = fmaf(d, d, acc);
    }
  }
  __shared__ double red[8];
  double s = acc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

__global__ void sq_diff_finish_kernel(const double* partial, int blocks, int64_t n, float* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < blocks; ++i) t += partial[i];
    out[0] = (float)(t / (double)n);
  }
}

// ---- clip search ----------------------------------------------------------------------------------
constexpr int kClipGroup = 128;
constexpr int kClipMaxTok = 512;
constexpr int kClipWarps = 16;
constexpr int kXStride = kClipGroup + 8;  // elements per staged token row: 272 bytes, conflict-free 128-bit reads

template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  __device__ static __forceinline__ void mul_unpack(uint32_t x, uint32_t w, float& lo, float& hi) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&x),
                                     *reinterpret_cast<const __nv_bfloat162*>(&w));
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
    lo = __uint_as_float(u << 16);
    hi = __uint_as_float(u & 0xffff0000u);
  }
};
template <> struct Pair<__half> {
  using type = __half2;
  __device__ static __forceinline__ void mul_unpack(uint32_t x, uint32_t w, float& lo, float& hi) {
    const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&x), *reinterpret_cast<const __half2*>(&w));
    const float2 f = __half22float2(p);
    lo = f.x;
    hi = f.y;
  }
};

struct ClipArgs {
  const void* W;
  const void* X;
  void* W_out;
  void* best_max;
  void* best_min;
  int64_t rows, cols, x_row_stride;  // x_row_stride: elements between sampled token rows
  int n_tok, n_groups, n_iter, n_grid, bits, sym, clip_sym, rows_per_cta;
  int ffma_sums;       // 1: sums on the CUDA cores (the kernel without MMAs), for comparison
  QRange qr;
};

// dot products of the lane's tokens with the 128 weights staged in `wv` (T-rounded products,
// fp32 accumulation in four partial sums, one rounding to T)
template <typename T, int TOK_PER_LANE>
__device__ __forceinline__ void group_dots(const T* xs, const T* wv, int lane, int n_tok, float (&out)[TOK_PER_LANE]) {
#pragma unroll
  for (int k = 0; k < TOK_PER_LANE; ++k) {
    const int t = lane + 32 * k;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (t < n_tok) {
      const uint4* xr = reinterpret_cast<const uint4*>(xs + (size_t)t * kXStride);
      const uint4* wr = reinterpret_cast<const uint4*>(wv);
#pragma unroll 4
      for (int j = 0; j < kClipGroup / 8; ++j) {
        const uint4 xv = xr[j], wq = wr[j];
        float l, h;
        Pair<T>::mul_unpack(xv.x, wq.x, l, h); a0 += l; a1 += h;
        Pair<T>::mul_unpack(xv.y, wq.y, l, h); a2 += l; a3 += h;
        Pair<T>::mul_unpack(xv.z, wq.z, l, h); a0 += l; a1 += h;
        Pair<T>::mul_unpack(xv.w, wq.w, l, h); a2 += l; a3 += h;
      }
    }
    out[k] = Elem<T>::rnd((a0 + a1) + (a2 + a3));
  }
}

template <typename T>
__global__ void __launch_bounds__(kClipWarps * 32, 1) clip_search_kernel(ClipArgs a) {
  using E = Elem<T>;
  constexpr int TPL = kClipMaxTok / 32;  // tokens per lane
  extern __shared__ __align__(16) unsigned char smem[];
  T* xs = reinterpret_cast<T*>(smem);                                  // [n_tok][kXStride]
  T* wbuf = xs + (size_t)kClipMaxTok * kXStride;                       // [warps][128]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.x;
  const T* X = reinterpret_cast<const T*>(a.X);
  const T* W = reinterpret_cast<const T*>(a.W);

  // stage the group's slice of the sampled tokens: n_tok rows of 128 elements
  for (int idx = threadIdx.x; idx < a.n_tok * (kClipGroup / 8); idx += blockDim.x) {
    const int t = idx / (kClipGroup / 8), j = idx % (kClipGroup / 8);
    const uint4 v = *reinterpret_cast<const uint4*>(X + (int64_t)t * a.x_row_stride + (int64_t)g * kClipGroup + j * 8);
    *reinterpret_cast<uint4*>(xs + (size_t)t * kXStride + j * 8) = v;
  }
  __syncthreads();

  T* wv = wbuf + warp * kClipGroup;
  const float n_tok_f = (float)a.n_tok;
  const int64_t r_begin = (int64_t)blockIdx.y * a.rows_per_cta;
  const int64_t r_end = min(a.rows, r_begin + a.rows_per_cta);
  for (int64_t r = r_begin + warp; r < r_end; r += kClipWarps) {
    // lane holds w[4*lane .. 4*lane+3]
    const uint2 raw = *reinterpret_cast<const uint2*>(W + r * a.cols + (int64_t)g * kClipGroup + 4 * lane);
    const T* wp = reinterpret_cast<const T*>(&raw);
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = E::to_f(wp[i]);
    float mx = a.clip_sym ? fabsf(w[0]) : w[0], mn = w[0];
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      mx = nan_max(mx, a.clip_sym ? fabsf(w[i]) : w[i]);
      mn = nan_min(mn, w[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    const float org_max = mx, org_min = mn;

    // org_out = (x * w).sum(-1)
    __syncwarp();
    *reinterpret_cast<uint2*>(wv + 4 * lane) = raw;
    __syncwarp();
    float org_out[TPL];
    group_dots<T, TPL>(xs, wv, lane, a.n_tok, org_out);

    float best_max = org_max, best_min = org_min;
    float min_err = E::rnd(1e9f);
    for (int it = 0; it < a.n_iter; ++it) {
      const float ratio = (float)(1.0 - (double)it / (double)a.n_grid);
      const float max_val = E::rnd(__fmul_rn(org_max, ratio));
      const float min_val = a.clip_sym ? -max_val : E::rnd(__fmul_rn(org_min, ratio));
      // cur_w = clamp(w, min_val, max_val); q_w = fake_quant_weight_dynamic(cur_w)
      float cw[4];
      float cmx, cmn;
#pragma unroll
      for (int i = 0; i < 4; ++i) cw[i] = clampf(w[i], min_val, max_val);
      cmx = cw[0];
      cmn = cw[0];
#pragma unroll
      for (int i = 1; i < 4; ++i) {
        cmx = nan_max(cmx, cw[i]);
        cmn = nan_min(cmn, cw[i]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        cmx = nan_max(cmx, __shfl_xor_sync(0xffffffffu, cmx, o));
        cmn = nan_min(cmn, __shfl_xor_sync(0xffffffffu, cmn, o));
      }
      float s, z;
      int_qparams<T>(cmn, cmx, a.qr, a.sym, s, z);
      T qw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qw[i] = E::from_f(int_dequant<T>(int_quant<T>(cw[i], s, z, a.qr), s, z));
      __syncwarp();
      *reinterpret_cast<uint2*>(wv + 4 * lane) = *reinterpret_cast<const uint2*>(qw);
      __syncwarp();
      float cur[TPL];
      group_dots<T, TPL>(xs, wv, lane, a.n_tok, cur);
      // err = (cur_out - org_out).pow(2).mean(tokens)
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < TPL; ++k) {
        if (lane + 32 * k < a.n_tok) {
          const float d = E::rnd(__fsub_rn(cur[k], org_out[k]));
          acc += E::rnd(__fmul_rn(d, d));
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const float err = E::rnd(__fdiv_rn(acc, n_tok_f));
      if (err < min_err) {
        min_err = err;
        best_max = max_val;
        best_min = min_val;
      }
    }
    if (lane == 0) {
      reinterpret_cast<T*>(a.best_max)[r * a.n_groups + g] = E::from_f(best_max);
      reinterpret_cast<T*>(a.best_min)[r * a.n_groups + g] = E::from_f(best_min);
    }
    if (a.W_out) {
      const float lo = a.clip_sym ? -best_max : best_min;
      T cwv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) cwv[i] = E::from_f(clampf(w[i], lo, best_max));
      *reinterpret_cast<uint2*>(reinterpret_cast<T*>(a.W_out) + r * a.cols + (int64_t)g * kClipGroup + 4 * lane) =
          *reinterpret_cast<const uint2*>(cwv);
    }
  }
}


// ---- clip search, summation on the tensor cores -------------------------------------------------------
// The reference's errors are sums of products that were each rounded to the tensor dtype
// ((input_feat * q_w).sum(-1), auto_clip.py:150-171), so the products cannot come from a GEMM.  The
// SUMS can: a lane forms the rounded products with packed multiplies directly in the register layout
// of an MMA A operand (16 tokens x 16 columns; the lane's x values come from ldmatrix, its four column
// weights from shared memory) and the MMA multiplies them by a matrix of ones, which adds them up in
// fp32 -- one instruction per 256 products instead of an unpack and an add per product.  The original
// weights and all clip candidates of a row are prepared first (kMmaCands vectors of 128 values, stored
// in the operand's column order), so an x fragment is loaded once per row and used by every candidate.
constexpr int kMmaCands = 11;      // the unclipped row + up to 10 grid points (max_shrink 0.5 of a 20-point grid)

template <typename T> struct MmaOps;
template <> struct MmaOps<__nv_bfloat16> {
  static constexpr uint32_t kOnes = 0x3F803F80u;
  __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&p);
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __forceinline__ float sum2(uint32_t a) {
    return __uint_as_float(a << 16) + __uint_as_float(a & 0xffff0000u);
  }
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(kOnes), "r"(kOnes));
  }
};
template <> struct MmaOps<__half> {
  static constexpr uint32_t kOnes = 0x3C003C00u;
  __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&p);
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static __forceinline__ float sum2(uint32_t a) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&a));
    return f.x + f.y;
  }
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(kOnes), "r"(kOnes));
  }
};

template <typename T>
__global__ void __launch_bounds__(kClipWarps * 32, 1) clip_search_mma_kernel(ClipArgs a) {
  using E = Elem<T>;
  using M = MmaOps<T>;
  extern __shared__ __align__(16) unsigned char smem[];
  T* xs = reinterpret_cast<T*>(smem);                                              // [n_tok][kXStride]
  uint32_t* wq_all = reinterpret_cast<uint32_t*>(xs + (size_t)kClipMaxTok * kXStride);   // [warps][cands][64]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.x;
  const T* X = reinterpret_cast<const T*>(a.X);
  const T* W = reinterpret_cast<const T*>(a.W);

  for (int idx = threadIdx.x; idx < a.n_tok * (kClipGroup / 8); idx += blockDim.x) {
    const int t = idx / (kClipGroup / 8), j = idx % (kClipGroup / 8);
    const uint4 v = *reinterpret_cast<const uint4*>(X + (int64_t)t * a.x_row_stride + (int64_t)g * kClipGroup + j * 8);
    *reinterpret_cast<uint4*>(xs + (size_t)t * kXStride + j * 8) = v;
  }
  __syncthreads();

  uint32_t* wq = wq_all + warp * (kMmaCands * 64);
  // The lane owns columns 4 * lane .. + 3 of the group: k tile lane / 4, and inside it the column pairs
  // (2c, 2c + 1) of c = 2 * (lane & 1) and 2 * (lane & 1) + 1, first half of the tile for (lane & 3) < 2,
  // second half otherwise.  Operand order of a k tile: [c][half] pairs, 8 words.
  const int st_kt = lane >> 2, st_half = (lane & 3) >> 1, st_c = 2 * (lane & 1);
  const int st0 = st_kt * 8 + st_c * 2 + st_half, st1 = st0 + 2;
  const int c = lane & 3;
  const float n_tok_f = (float)a.n_tok;
  const int n_cand = a.n_iter + 1;
  const uint32_t xs_base = (uint32_t)__cvta_generic_to_shared(xs);
  // ldmatrix row address of this lane: matrix lane / 8 = (token half, column half), row lane % 8
  const uint32_t ld_off = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * kXStride + (lane >> 4) * 8) * (uint32_t)sizeof(T);

  const int64_t r_begin = (int64_t)blockIdx.y * a.rows_per_cta;
  const int64_t r_end = min(a.rows, r_begin + a.rows_per_cta);
  for (int64_t r = r_begin + warp; r < r_end; r += kClipWarps) {
    const uint2 raw = *reinterpret_cast<const uint2*>(W + r * a.cols + (int64_t)g * kClipGroup + 4 * lane);
    const T* wp = reinterpret_cast<const T*>(&raw);
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = E::to_f(wp[i]);
    float mx = a.clip_sym ? fabsf(w[0]) : w[0], mn = w[0];
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      mx = nan_max(mx, a.clip_sym ? fabsf(w[i]) : w[i]);
      mn = nan_min(mn, w[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    const float org_max = mx, org_min = mn;

    // ---- the row and its clip candidates, in operand order ----
    __syncwarp();
    wq[st0] = raw.x;
    wq[st1] = raw.y;
    for (int it = 0; it < a.n_iter; ++it) {
      const float ratio = (float)(1.0 - (double)it / (double)a.n_grid);
      const float max_val = E::rnd(__fmul_rn(org_max, ratio));
      const float min_val = a.clip_sym ? -max_val : E::rnd(__fmul_rn(org_min, ratio));
      float cw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) cw[i] = clampf(w[i], min_val, max_val);
      float cmx = cw[0], cmn = cw[0];
#pragma unroll
      for (int i = 1; i < 4; ++i) {
        cmx = nan_max(cmx, cw[i]);
        cmn = nan_min(cmn, cw[i]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        cmx = nan_max(cmx, __shfl_xor_sync(0xffffffffu, cmx, o));
        cmn = nan_min(cmn, __shfl_xor_sync(0xffffffffu, cmn, o));
      }
      float s, z;
      int_qparams<T>(cmn, cmx, a.qr, a.sym, s, z);
      T qw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qw[i] = E::from_f(int_dequant<T>(int_quant<T>(cw[i], s, z, a.qr), s, z));
      const uint2 packed = *reinterpret_cast<const uint2*>(qw);
      wq[(it + 1) * 64 + st0] = packed.x;
      wq[(it + 1) * 64 + st1] = packed.y;
    }
    __syncwarp();

    // ---- sums of rounded products: tokens in tiles of 16, columns in tiles of 16 ----
    float errsum[kMmaCands];
#pragma unroll
    for (int q = 0; q < kMmaCands; ++q) errsum[q] = 0.f;
#pragma unroll 1
    for (int tt = 0; tt < a.n_tok; tt += 16) {
      float acc[kMmaCands][4];
#pragma unroll
      for (int q = 0; q < kMmaCands; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
      // x fragment of the next column tile in flight while the eleven candidates of this one are multiplied;
      // a candidate's four weights are loaded for all candidates before the first product, so that the loads,
      // the packed multiplies and the eleven independent accumulator chains overlap
      uint32_t xf[2][4];
      {
        const uint32_t addr = xs_base + (uint32_t)(tt * kXStride) * (uint32_t)sizeof(T) + ld_off;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(xf[0][0]), "=r"(xf[0][1]), "=r"(xf[0][2]), "=r"(xf[0][3])
                     : "r"(addr));
      }
#pragma unroll
      for (int kt = 0; kt < kClipGroup / 16; ++kt) {
        const int cur = kt & 1;
        if (kt + 1 < kClipGroup / 16) {
          const uint32_t addr = xs_base + (uint32_t)(tt * kXStride + (kt + 1) * 16) * (uint32_t)sizeof(T) + ld_off;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                       : "=r"(xf[cur ^ 1][0]), "=r"(xf[cur ^ 1][1]), "=r"(xf[cur ^ 1][2]), "=r"(xf[cur ^ 1][3])
                       : "r"(addr));
        }
        uint2 qv[kMmaCands];
#pragma unroll
        for (int q = 0; q < kMmaCands; ++q) qv[q] = *reinterpret_cast<const uint2*>(&wq[q * 64 + kt * 8 + c * 2]);
#pragma unroll
        for (int q = 0; q < kMmaCands; ++q) {
          if (q < n_cand)
            M::mma(acc[q], M::mul2(xf[cur][0], qv[q].x), M::mul2(xf[cur][1], qv[q].x), M::mul2(xf[cur][2], qv[q].y),
                   M::mul2(xf[cur][3], qv[q].y));
        }
      }
      // rows grp and grp + 8 of the tile; the four lanes of a quad hold the same sums: lane c == 0 counts
      // (packed: both tokens of the lane at once; the difference of two T values and the square of a T value
      // round once to T either way)
      if (c == 0) {
        const uint32_t org2 = M::pack(acc[0][0], acc[0][2]);
#pragma unroll
        for (int q = 1; q < kMmaCands; ++q) {
          if (q < n_cand) {
            const uint32_t d2 = M::sub2(M::pack(acc[q][0], acc[q][2]), org2);
            errsum[q] += M::sum2(M::mul2(d2, d2));
          }
        }
      }
    }
    float best_max = org_max, best_min = org_min;
    float min_err = E::rnd(1e9f);
#pragma unroll
    for (int q = 1; q < kMmaCands; ++q) {
      if (q < n_cand) {
        float accq = errsum[q];
#pragma unroll
        for (int o = 16; o >= 4; o >>= 1) accq += __shfl_xor_sync(0xffffffffu, accq, o);
        accq = __shfl_sync(0xffffffffu, accq, 0);
        const float err = E::rnd(__fdiv_rn(accq, n_tok_f));
        if (err < min_err) {
          const float ratio = (float)(1.0 - (double)(q - 1) / (double)a.n_grid);
          min_err = err;
          best_max = E::rnd(__fmul_rn(org_max, ratio));
          best_min = a.clip_sym ? -best_max : E::rnd(__fmul_rn(org_min, ratio));
        }
      }
    }
    if (lane == 0) {
      reinterpret_cast<T*>(a.best_max)[r * a.n_groups + g] = E::from_f(best_max);
      reinterpret_cast<T*>(a.best_min)[r * a.n_groups + g] = E::from_f(best_min);
    }
    if (a.W_out) {
      const float lo = a.clip_sym ? -best_max : best_min;
      T cwv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) cwv[i] = E::from_f(clampf(w[i], lo, best_max));
      *reinterpret_cast<uint2*>(reinterpret_cast<T*>(a.W_out) + r * a.cols + (int64_t)g * kClipGroup + 4 * lane) =
          *reinterpret_cast<const uint2*>(cwv);
    }
  }
}

template <typename T>
int clip_launch(const ClipArgs& a0, cudaStream_t st) {
  ClipArgs a = a0;
  const size_t smem = ((size_t)kClipMaxTok * kXStride + (size_t)kClipWarps * kClipGroup) * sizeof(T);
  const size_t smem_mma = (size_t)kClipMaxTok * kXStride * sizeof(T) + (size_t)kClipWarps * kMmaCands * 64 * sizeof(uint32_t);
  const bool use_mma = a.n_tok % 16 == 0 && a.n_iter + 1 <= kMmaCands && !a.ffma_sums;
  LC_CHECK_CUDA(cudaFuncSetAttribute(clip_search_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LC_CHECK_CUDA(cudaFuncSetAttribute(clip_search_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem_mma));
  // one CTA per (group, row chunk), one CTA per SM at a time: the number of row chunks is the one between
  // one and four waves of CTAs that fills its last wave best (each CTA stages its x slice once)
  int best_splits = 1;
  double best_eff = -1.0;
  const int max_splits = (int)((a.rows + kClipWarps - 1) / kClipWarps);
  for (int sp = 1; sp <= max_splits && (int64_t)sp * a.n_groups <= 4 * kNumSMsB200 + a.n_groups; ++sp) {
    int64_t rp = (a.rows + sp - 1) / sp;
    rp = (rp + kClipWarps - 1) / kClipWarps * kClipWarps;
    const int64_t ctas = (int64_t)a.n_groups * ((a.rows + rp - 1) / rp);
    if (ctas < kNumSMsB200 && sp < max_splits) continue;
    const int64_t waves = (ctas + kNumSMsB200 - 1) / kNumSMsB200;
    // time ~ waves x rows per CTA; efficiency = work / (SMs x time)
    const double eff = (double)a.rows * a.n_groups / ((double)kNumSMsB200 * (double)waves * (double)rp);
    if (eff > best_eff + 1e-9) best_eff = eff, best_splits = sp;
  }
  int64_t rpc = (a.rows + best_splits - 1) / best_splits;
  rpc = (rpc + kClipWarps - 1) / kClipWarps * kClipWarps;
  a.rows_per_cta = (int)rpc;
  dim3 grid((unsigned)a.n_groups, (unsigned)((a.rows + rpc - 1) / rpc));
  if (use_mma) clip_search_mma_kernel<T><<<grid, kClipWarps * 32, smem_mma, st>>>(a);
  else clip_search_kernel<T><<<grid, kClipWarps * 32, smem, st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_awq_act_mean(const void* x, int dtype, int64_t tokens, int64_t cols, void* out,
                                      float* scratch, int64_t scratch_floats, lc_stream_t stream) {
  using namespace lc;
  if (!x || !out || !scratch || tokens <= 0 || cols <= 0) return LC_ERR_ARG;
  if (dtype != LC_BF16 && dtype != LC_F16 && dtype != LC_F32) return LC_ERR_ARG;
  const int N = dtype == LC_F32 ? 4 : 8;
  if (cols % N != 0 || !aligned16(x)) return LC_ERR_ALIGN;
  int splits = (int)((tokens + 255) / 256);
  if (splits > 64) splits = 64;
  if (scratch_floats < (int64_t)splits * cols) return LC_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((cols / N + 31) / 32), (unsigned)splits), block(32, 8);
  const unsigned fb = (unsigned)((cols + 255) / 256);
  switch (dtype) {
    case LC_BF16:
      abs_sum_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, tokens, cols, scratch);
      abs_mean_finish_kernel<__nv_bfloat16><<<fb, 256, 0, st>>>(scratch, splits, tokens, cols, (__nv_bfloat16*)out);
      break;
    case LC_F16:
      abs_sum_kernel<__half><<<grid, block, 0, st>>>((const __half*)x, tokens, cols, scratch);
      abs_mean_finish_kernel<__half><<<fb, 256, 0, st>>>(scratch, splits, tokens, cols, (__half*)out);
      break;
    default:
      abs_sum_kernel<float><<<grid, block, 0, st>>>((const float*)x, tokens, cols, scratch);
      abs_mean_finish_kernel<float><<<fb, 256, 0, st>>>(scratch, splits, tokens, cols, (float*)out);
      break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_awq_div_cols(const void* x, const void* col_scale, int dtype, int64_t rows, int64_t cols,
                                      void* out, lc_stream_t stream) {
  using namespace lc;
  if (!x || !col_scale || !out || rows <= 0 || cols <= 0) return LC_ERR_ARG;
  if (dtype != LC_BF16 && dtype != LC_F16 && dtype != LC_F32) return LC_ERR_ARG;
  const int N = dtype == LC_F32 ? 4 : 8;
  if (cols % N != 0 || !aligned16(x) || !aligned16(out) || !aligned16(col_scale)) return LC_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t gy = (rows + 7) / 8;
  const int64_t cap = 8 * kNumSMsB200;
  if (gy > cap) gy = cap;
  dim3 grid((unsigned)((cols / N + 31) / 32), (unsigned)gy), block(32, 8);
  switch (dtype) {
    case LC_BF16:
      div_cols_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)col_scale,
                                                              rows, cols, (__nv_bfloat16*)out);
      break;
    case LC_F16:
      div_cols_kernel<__half><<<grid, block, 0, st>>>((const __half*)x, (const __half*)col_scale, rows, cols,
                                                      (__half*)out);
      break;
    default:
      div_cols_kernel<float><<<grid, block, 0, st>>>((const float*)x, (const float*)col_scale, rows, cols, (float*)out);
      break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_awq_loss(const void* a, const void* b, int dtype, int64_t n, float* loss_out, double* scratch,
                                  int64_t scratch_doubles, lc_stream_t stream) {
  using namespace lc;
  if (!a || !b || !loss_out || !scratch || n <= 0) return LC_ERR_ARG;
  if (dtype != LC_BF16 && dtype != LC_F16 && dtype != LC_F32) return LC_ERR_ARG;
  if (!aligned16(a) || !aligned16(b)) return LC_ERR_ALIGN;
  int blocks = 4 * kNumSMsB200;
  if (scratch_doubles < blocks) return LC_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_BF16:
      sq_diff_partial_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, n,
                                                                    scratch);
      break;
    case LC_F16:
      sq_diff_partial_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)a, (const __half*)b, n, scratch);
      break;
    default: sq_diff_partial_kernel<float><<<blocks, 256, 0, st>>>((const float*)a, (const float*)b, n, scratch); break;
  }
  LC_LAUNCH_CHECK();
  sq_diff_finish_kernel<<<1, 32, 0, st>>>(scratch, blocks, n, loss_out);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

static int clip_search_impl(const void* W, const void* X, int dtype, int64_t rows, int64_t cols, int64_t x_tokens,
                            int64_t x_token_step, int64_t group, int bits, int sym, int clip_sym, int n_grid,
                            double max_shrink, void* best_max, void* best_min, void* W_out, int ffma_sums,
                            lc_stream_t stream) {
  using namespace lc;
  if (!W || !X || !best_max || !best_min || rows <= 0 || cols <= 0 || x_tokens <= 0 || x_token_step <= 0) return LC_ERR_ARG;
  if (bits < 2 || bits > 8 || n_grid <= 0 || max_shrink < 0.0 || max_shrink > 1.0) return LC_ERR_ARG;
  if (dtype != LC_BF16 && dtype != LC_F16) return LC_ERR_ARG;      // 16-bit tensors only
  if (group != kClipGroup || cols % kClipGroup != 0) return LC_ERR_SHAPE;
  const int64_t n_tok = (x_tokens + x_token_step - 1) / x_token_step;  // x[0::step]
  if (n_tok > kClipMaxTok) return LC_ERR_SHAPE;
  if (!aligned16(W) || !aligned16(X) || (W_out && !aligned16(W_out))) return LC_ERR_ALIGN;
  ClipArgs a;
  a.W = W;
  a.X = X;
  a.W_out = W_out;
  a.best_max = best_max;
  a.best_min = best_min;
  a.rows = rows;
  a.cols = cols;
  a.x_row_stride = x_token_step * cols;
  a.n_tok = (int)n_tok;
  a.n_groups = (int)(cols / kClipGroup);
  a.n_grid = n_grid;
  a.n_iter = (int)(max_shrink * n_grid);
  a.bits = bits;
  a.sym = sym ? 1 : 0;
  a.clip_sym = clip_sym ? 1 : 0;
  a.rows_per_cta = 0;
  a.ffma_sums = ffma_sums;
  a.qr = int_qrange(bits, a.sym);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == LC_BF16 ? clip_launch<__nv_bfloat16>(a, st) : clip_launch<__half>(a, st);
}

extern "C" LC_API int lc_awq_clip_search(const void* W, const void* X, int dtype, int64_t rows, int64_t cols,
                                         int64_t x_tokens, int64_t x_token_step, int64_t group, int bits, int sym,
                                         int clip_sym, int n_grid, double max_shrink, void* best_max, void* best_min,
                                         void* W_out, lc_stream_t stream) {
  return clip_search_impl(W, X, dtype, rows, cols, x_tokens, x_token_step, group, bits, sym, clip_sym, n_grid, max_shrink,
                          best_max, best_min, W_out, 0, stream);
}

extern "C" LC_API int lc_awq_clip_search_cuda_cores(const void* W, const void* X, int dtype, int64_t rows, int64_t cols,
                                                    int64_t x_tokens, int64_t x_token_step, int64_t group, int bits,
                                                    int sym, int clip_sym, int n_grid, double max_shrink,
                                                    void* best_max, void* best_min, void* W_out, lc_stream_t stream) {
  return clip_search_impl(W, X, dtype, rows, cols, x_tokens, x_token_step, group, bits, sym, clip_sym, n_grid, max_shrink,
                          best_max, best_min, W_out, 1, stream);
}
