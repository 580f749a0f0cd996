// SpQR: the GPTQ block loop with groups of 16 columns, leave-one-out outlier detection per group and
// unquantised outliers (llmc/compression/quantization/spqr.py:184-285).
//
// Like GPTQ every row is a chain of dependent column steps that share only the inverse-Hessian factor U,
// so a thread owns one row.  A warp holds its 32 rows x 128 columns of the block in shared memory (row
// pitch 129 floats: a lane walking along its row never meets another lane's bank); the block's 128 x 128
// piece of U arrives by asynchronous 16-byte copies and is read warp-uniformly.  Per group of 16 columns:
//   1. the lane takes the group's 16 values into registers and decides which of them are outliers: for
//      every element, how much the group's weighted quantisation error falls when that element is left
//      out of the min-max statistics (16 leave-one-out quantisations of 15 values, spqr.py:185-203);
//   2. the group's scale and zero point come from the values with the outliers replaced by the mean of the
//      others, and pass through the second-level quantisation of the statistics (spqr.py:325-346);
//   3. the 16 column steps run in registers: quantise, error, outlier test on the error, spread the error
//      over the later columns of the group;
//   4. the group's 16 errors are then applied, in column order, to the later columns of the block in
//      shared memory.  Each element sees the same subtractions in the same order as in the reference's
//      column-by-column update, so the block is bit-identical to it.
// Steps 2-4 use the reference's fp32 operations one for one (IEEE division, no fused multiply-add).  Step 1
// only feeds comparisons against a threshold and multiplies by reciprocals.
#include "lc_common.cuh"
#include "tf32x3_gemm.cuh"

namespace lc {

int gptq_trail_launch(float* W, const float* err_t, const float* U, int64_t rows, int64_t cols, int64_t col0,
                      int k, int64_t col1, cudaStream_t st, int64_t col_end);

namespace {

constexpr int kBlk = 128;
constexpr int kG = 16;                 // group size (the reference's spqr_w_only.yml)
constexpr int kThreads = 64;           // rows per CTA
constexpr int kPitch = kBlk + 1;
constexpr size_t kSmemBytes = (size_t)(kBlk * kBlk + kBlk + kThreads * kPitch) * sizeof(float);

struct SpqrArgs {
  float* W;
  const float* U;
  float* err_t;        // [128][rows]
  float* panel_hi;     // optional [panel depth][rows]
  float* panel_lo;
  int panel_k0;
  float* scales;       // rows x n_groups (groups of 16 columns)
  float* zeros;
  uint8_t* mask;       // rows x cols, 1 = outlier (kept unquantised)
  float* loss_rows;
  const float* thr;    // device scalar: the outlier threshold, +inf = no outliers
  int64_t rows, cols, col0, n_groups;
  int simplified;
  float qmax;
};

// statistics quantizers on a (rows, 1) tensor (spqr.py:328-339): every value is a group by itself, range
// 0, scale c = clamp(0, 1e-5) / 7, zero point -(v / c); v / c + zero = 0, code 0, and back: (v / c) * c
__device__ __forceinline__ float second_level(float v) {
  const float c = __fdiv_rn(1e-5f, 7.f);
  const float zz = __fsub_rn(0.f, __fdiv_rn(v, c));
  float q = rintf(__fadd_rn(__fdiv_rn(v, fmaxf(c, 1e-9f)), zz));
  q = fminf(fmaxf(q, 0.f), 7.f);
  return __fmul_rn(__fsub_rn(q, zz), c);
}

// weighted squared error of quantising the 16 values with the min-max statistics of all but `skip`
// (skip < 0: of all), summed over all but `skip`
template <int kSkip>
__device__ __forceinline__ float group_error(const float (&x)[kG], const float (&hdinv)[kG], float mn, float mx,
                                             float qmax) {
  const float s = __fdiv_rn(fmaxf(__fsub_rn(mx, mn), 1e-5f), qmax);
  const float z = __fsub_rn(0.f, __fdiv_rn(mn, s));
  const float rs = __frcp_rn(fmaxf(s, 1e-9f));
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < kG; ++k) {
    if (k == kSkip) continue;
    float q = rintf(__fmaf_rn(x[k], rs, z));
    q = fminf(fmaxf(q, 0.f), qmax);
    const float d = __fmul_rn(__fsub_rn(__fmul_rn(__fsub_rn(q, z), s), x[k]), hdinv[k]);
    acc = __fmaf_rn(d, d, acc);
  }
  return acc;
}

template <int kJ>
struct LooLoop {
  static __device__ __forceinline__ void run(const float (&x)[kG], const float (&hdinv)[kG], float mn1, int imn,
                                             float mn2, float mx1, int imx, float mx2, float qmax, float base,
                                             float thr, unsigned& outl) {
    const float mn = (kJ == imn) ? mn2 : mn1, mx = (kJ == imx) ? mx2 : mx1;
    const float e = base - group_error<kJ>(x, hdinv, mn, mx, qmax);
    if (e > thr) outl |= 1u << kJ;
    LooLoop<kJ + 1>::run(x, hdinv, mn1, imn, mn2, mx1, imx, mx2, qmax, base, thr, outl);
  }
};
template <>
struct LooLoop<kG> {
  static __device__ __forceinline__ void run(const float (&)[kG], const float (&)[kG], float, int, float, float, int,
                                             float, float, float, float, unsigned&) {}
};

__global__ void __launch_bounds__(kThreads) spqr_block_kernel(SpqrArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* u1 = sm;                                   // [128][128] of U, rows col0 .., columns col0 ..
  float* dinv = sm + kBlk * kBlk;                   // 1 / U_ii
  float* tile = dinv + kBlk + threadIdx.x * kPitch; // this thread's row of the block
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // U block: 4096 16-byte asynchronous copies, all in flight at once
  {
    const float* ub = a.U + a.col0 * a.cols + a.col0;
    const unsigned sbase = (unsigned)__cvta_generic_to_shared(u1);
    for (int idx = threadIdx.x; idx < kBlk * kBlk / 4; idx += kThreads) {
      const int i = idx >> 5, j4 = (idx & 31) << 2;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sbase + (unsigned)((i * kBlk + j4) * 4)),
                   "l"(ub + (int64_t)i * a.cols + j4));
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  // W: a warp reads its 32 rows, row by row (coalesced), and parks them at the row pitch
  const int64_t r0w = (int64_t)blockIdx.x * kThreads + warp * 32;
  {
    float* wt = dinv + kBlk + (warp * 32) * kPitch;
    for (int rr = 0; rr < 32; ++rr) {
      const int64_t r = r0w + rr;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < a.rows) v = *reinterpret_cast<const float4*>(a.W + r * a.cols + a.col0 + 4 * lane);
      float* p = wt + rr * kPitch + 4 * lane;
      p[0] = v.x, p[1] = v.y, p[2] = v.z, p[3] = v.w;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();
  for (int i = threadIdx.x; i < kBlk; i += kThreads) dinv[i] = __frcp_rn(u1[i * kBlk + i]);
  __syncthreads();

  const int64_t r = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const bool live = r < a.rows;
  const float thr = a.thr[0];
  const bool detect = thr < INFINITY;
  const float qmax = a.qmax;
  float loss = 0.f;

#pragma unroll 1
  for (int g = 0; g < kBlk / kG; ++g) {
    const int c0 = g * kG;
    float x[kG], hdinv[kG];
#pragma unroll
    for (int k = 0; k < kG; ++k) {
      x[k] = tile[c0 + k];
      hdinv[k] = dinv[c0 + k];
    }
    // ---- group statistics ----
    float mn1 = x[0], mx1 = x[0];
    int imn = 0, imx = 0;
#pragma unroll
    for (int k = 1; k < kG; ++k) {
      if (x[k] < mn1) mn1 = x[k], imn = k;
      if (x[k] > mx1) mx1 = x[k], imx = k;
    }
    float y_mn = mn1, y_mx = mx1;
    if (detect && !a.simplified) {
      float mn2 = INFINITY, mx2 = -INFINITY;
#pragma unroll
      for (int k = 0; k < kG; ++k) {
        if (k != imn) mn2 = fminf(mn2, x[k]);
        if (k != imx) mx2 = fmaxf(mx2, x[k]);
      }
      const float base = group_error<-1>(x, hdinv, mn1, mx1, qmax);
      unsigned outl = 0;
      LooLoop<0>::run(x, hdinv, mn1, imn, mn2, mx1, imx, mx2, qmax, base, thr, outl);
      if (outl) {
        // statistics of the group with the outliers replaced by the mean of the others (spqr.py:222-227)
        float sum = 0.f, cnt = 0.f;
#pragma unroll
        for (int k = 0; k < kG; ++k) {
          const float keep = (outl >> k & 1u) ? 0.f : 1.f;
          sum = __fadd_rn(sum, __fmul_rn(x[k], keep));
          cnt += keep;
        }
        const float mean = __fdiv_rn(sum, fmaxf(cnt, 1.f));
        y_mn = INFINITY, y_mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < kG; ++k) {
          const float m = (outl >> k & 1u) ? 1.f : 0.f;
          const float y = __fadd_rn(__fmul_rn(x[k], 1.f - m), __fmul_rn(mean, m));
          y_mn = fminf(y_mn, y), y_mx = fmaxf(y_mx, y);
        }
      }
    }
    float s = __fdiv_rn(fmaxf(__fsub_rn(y_mx, y_mn), 1e-5f), qmax);
    float z = __fsub_rn(0.f, __fdiv_rn(y_mn, s));
    s = second_level(s);
    z = second_level(z);
    if (live) {
      const int64_t gi = r * a.n_groups + (a.col0 + c0) / kG;
      a.scales[gi] = s;
      a.zeros[gi] = z;
    }
    const float sc = fmaxf(s, 1e-9f);
    // ---- the 16 column steps ----
    float e[kG];
    unsigned mbits = 0;
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      const float w = x[j];
      float q = rintf(__fadd_rn(__fdiv_rn(w, sc), z));
      q = fminf(fmaxf(q, 0.f), qmax);
      const float dq = __fmul_rn(__fsub_rn(q, z), s);
      const float d = u1[(c0 + j) * kBlk + c0 + j];
      float err = __fdiv_rn(__fsub_rn(w, dq), d);
      if (detect && __fmul_rn(err, err) > thr) {
        mbits |= 1u << j;
        err = __fdiv_rn(__fsub_rn(w, w), d);        // the outlier keeps its value: no error to spread
      }
      e[j] = err;
      loss = __fmaf_rn(err, err, loss);
#pragma unroll
      for (int k = j + 1; k < kG; ++k) x[k] = __fsub_rn(x[k], __fmul_rn(err, u1[(c0 + j) * kBlk + c0 + k]));
    }
    // kept values, mask and errors of the group
#pragma unroll
    for (int k = 0; k < kG; ++k) tile[c0 + k] = x[k];
    if (live) {
#pragma unroll
      for (int k = 0; k < kG; ++k) {
        a.err_t[(int64_t)(c0 + k) * a.rows + r] = e[k];
        if (a.panel_hi) {
          const float hi = __uint_as_float(__float_as_uint(e[k]) & 0xffffe000u);
          a.panel_hi[(int64_t)(a.panel_k0 + c0 + k) * a.rows + r] = e[k];
          a.panel_lo[(int64_t)(a.panel_k0 + c0 + k) * a.rows + r] = e[k] - hi;
        }
      }
      if (a.mask) {
        uint32_t* mp = reinterpret_cast<uint32_t*>(a.mask + r * a.cols + a.col0 + c0);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t wv = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) wv |= (mbits >> (4 * q4 + b) & 1u) << (8 * b);
          mp[q4] = wv;
        }
      }
    }
    // ---- the group's errors on the later columns of the block, column order ----
#pragma unroll 1
    for (int c = c0 + kG; c < kBlk; c += 4) {
      float v0 = tile[c], v1 = tile[c + 1], v2 = tile[c + 2], v3 = tile[c + 3];
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        const float4 u = *reinterpret_cast<const float4*>(&u1[(c0 + j) * kBlk + c]);
        v0 = __fsub_rn(v0, __fmul_rn(e[j], u.x));
        v1 = __fsub_rn(v1, __fmul_rn(e[j], u.y));
        v2 = __fsub_rn(v2, __fmul_rn(e[j], u.z));
        v3 = __fsub_rn(v3, __fmul_rn(e[j], u.w));
      }
      tile[c] = v0, tile[c + 1] = v1, tile[c + 2] = v2, tile[c + 3] = v3;
    }
  }
  if (live && a.loss_rows) a.loss_rows[r] += loss;
  __syncwarp();
  // kept values back, row by row
  {
    const float* wt = dinv + kBlk + (warp * 32) * kPitch;
    for (int rr = 0; rr < 32; ++rr) {
      const int64_t rw = r0w + rr;
      if (rw >= a.rows) break;
      const float* p = wt + rr * kPitch + 4 * lane;
      *reinterpret_cast<float4*>(a.W + rw * a.cols + a.col0 + 4 * lane) = make_float4(p[0], p[1], p[2], p[3]);
    }
  }
}

int spqr_block_launch(const SpqrArgs& a, cudaStream_t st) {
  if (cudaFuncSetAttribute(spqr_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
      cudaSuccess)
    return LC_ERR_CUDA;
  spqr_block_kernel<<<(unsigned)((a.rows + kThreads - 1) / kThreads), kThreads, kSmemBytes, st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

// SpQR.w_qdq (spqr.py:367-390): outliers keep their value, the rest is the static fake quantisation with
// the statistics of the group its column has in the permuted order
template <typename T>
__global__ void __launch_bounds__(256) spqr_dequant_kernel(const float* W, const float* scales, const float* zeros,
                                                           const uint8_t* mask, const int64_t* invperm, int64_t rows,
                                                           int64_t cols, int64_t n_groups, float qmax, T* out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t g = (invperm ? invperm[c] : c) / kG;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    const float w = W[r * cols + c];
    float v = w;
    if (!mask[r * cols + c]) {
      const float s = scales[r * n_groups + g], z = zeros[r * n_groups + g];
      float q = rintf(__fadd_rn(__fdiv_rn(w, fmaxf(s, 1e-9f)), z));
      q = fminf(fmaxf(q, 0.f), qmax);
      v = __fmul_rn(__fsub_rn(q, z), s);
    }
    out[r * cols + c] = Elem<T>::from_f(v);
  }
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_spqr_weight_transform(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols,
                                               int bits, const float* threshold, int simplified, float* scratch_err,
                                               float* panel_hi, float* panel_lo, float* scales, float* zeros,
                                               uint8_t* mask_u8, float* loss_rows, int32_t* status,
                                               lc_stream_t stream) {
  using namespace lc;
  constexpr int kPanel = 1024, kSub = 256;
  if (!W || !U || !threshold || !scratch_err || !scales || !zeros) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (cols % 128 != 0) return LC_ERR_SHAPE;
  if (!aligned16(W) || !aligned16(U) || (mask_u8 && (reinterpret_cast<uintptr_t>(mask_u8) & 3u))) return LC_ERR_ALIGN;
  const bool tc = U_lo != nullptr;
  if (tc && (!panel_hi || !panel_lo || rows % 4 != 0)) return LC_ERR_ARG;
  if (tc && (!aligned16(U_lo) || !aligned16(panel_hi) || !aligned16(panel_lo))) return LC_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (loss_rows) LC_CHECK_CUDA(cudaMemsetAsync(loss_rows, 0, rows * sizeof(float), st));
  SpqrArgs a;
  a.W = W, a.U = U, a.err_t = scratch_err, a.scales = scales, a.zeros = zeros, a.mask = mask_u8;
  a.loss_rows = loss_rows, a.thr = threshold, a.rows = rows, a.cols = cols, a.n_groups = cols / kG;
  a.simplified = simplified ? 1 : 0, a.qmax = (float)((1 << bits) - 1);
  a.panel_hi = tc ? panel_hi : nullptr, a.panel_lo = tc ? panel_lo : nullptr, a.panel_k0 = 0;
  int rc;
  if (!tc) {
    // the reference's schedule: everything to the right after every block (fp32 FFMA, K = 128)
    for (int64_t i1 = 0; i1 < cols; i1 += kBlk) {
      a.col0 = i1;
      if ((rc = spqr_block_launch(a, st)) != LC_OK) return rc;
      if ((rc = gptq_trail_launch(W, scratch_err, U, rows, cols, i1, kBlk, i1 + kBlk, st, -1)) != LC_OK) return rc;
    }
    return LC_OK;
  }
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  // three-level trailing update as in the GPTQ loop: eager inside a 256-column sub-panel, K = 256 for the
  // rest of the 1024-column panel, K = 1024 for everything right of the panel (tensor cores, tf32 x 3)
  GemmMat E, Um;
  if ((rc = gemm_mat_init(&E, panel_hi, panel_lo, kPanel, rows, rows)) != LC_OK) return rc;
  if ((rc = gemm_mat_init(&Um, U, U_lo, cols, cols, cols)) != LC_OK) return rc;
  for (int64_t p1 = 0; p1 < cols; p1 += kPanel) {
    const int64_t p2 = (p1 + kPanel < cols) ? p1 + kPanel : cols;
    for (int64_t s1 = p1; s1 < p2; s1 += kSub) {
      const int64_t s2 = (s1 + kSub < p2) ? s1 + kSub : p2;
      for (int64_t i1 = s1; i1 < s2; i1 += kBlk) {
        a.col0 = i1, a.panel_k0 = (int)(i1 - p1);
        if ((rc = spqr_block_launch(a, st)) != LC_OK) return rc;
        if ((rc = gptq_trail_launch(W, scratch_err, U, rows, cols, i1, kBlk, i1 + kBlk, st, s2)) != LC_OK) return rc;
      }
      if (s2 < p2 && (rc = tf32x3_gemm_launch(W + s2, cols, E, s1 - p1, 0, Um, s1, s2, rows, p2 - s2, s2 - s1, 1, -1.f,
                                              0, status, st)) != LC_OK)
        return rc;
    }
    if (p2 < cols && (rc = tf32x3_gemm_launch(W + p2, cols, E, 0, 0, Um, p1, p2, rows, cols - p2, p2 - p1, 1, -1.f, 0,
                                              status, st)) != LC_OK)
      return rc;
  }
  return LC_OK;
}

extern "C" LC_API int lc_spqr_dequant(const float* W, const float* scales, const float* zeros, const uint8_t* mask_u8,
                                      const int64_t* invperm, int64_t rows, int64_t cols, int bits, void* out,
                                      int out_dtype, lc_stream_t stream) {
  using namespace lc;
  if (!W || !scales || !zeros || !mask_u8 || !out || rows <= 0 || cols <= 0 || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (cols % 16 != 0) return LC_ERR_SHAPE;
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_F16) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 g((unsigned)((cols + 255) / 256), (unsigned)(rows < 1024 ? rows : 1024));
  const float qmax = (float)((1 << bits) - 1);
  const int64_t ng = cols / 16;
  switch (out_dtype) {
    case LC_F32:
      spqr_dequant_kernel<float><<<g, 256, 0, st>>>(W, scales, zeros, mask_u8, invperm, rows, cols, ng, qmax, (float*)out);
      break;
    case LC_BF16:
      spqr_dequant_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(W, scales, zeros, mask_u8, invperm, rows, cols, ng, qmax,
                                                            (__nv_bfloat16*)out);
      break;
    default:
      spqr_dequant_kernel<__half><<<g, 256, 0, st>>>(W, scales, zeros, mask_u8, invperm, rows, cols, ng, qmax,
                                                     (__half*)out);
      break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}
