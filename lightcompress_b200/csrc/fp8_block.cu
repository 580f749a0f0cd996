// Family 1 (float): FP8 e4m3 block-wise weights, one fp32 scale per 128 x 128 block -- the layout of
// block-quantised FP8 checkpoints.  Follows FloatQuantizer with granularity 'per_block'
// (llmc/compression/quantization/quant.py: reshape_tensor :637-641 pads to whole blocks with zeros,
// get_minmax_range :138-140 takes the block's |x| extremes in fp32, get_qparams :544-551, quant /
// dequant :1060-1075, real_quant_weight_dynamic :1194-1220) and the two helpers built on it,
// weight_cast_to_fp8 / weight_cast_to_bf16 (quant.py:20-45; the reference's Triton versions of the same
// two, kernel.py:56-131, run when Triton is usable).  With fp32 scales every op of the chain is an fp32
// op on the promoted tensor: u = x / s, e4m3 round-to-nearest-even, q * s, one rounding to the output
// dtype at the end.
//
// One CTA per block: 256 threads hold the block's 16384 elements in registers between the abs-max
// reduction and the quantise pass, so HBM is read once.  HBM-bound.
#include <cuda_fp8.h>

#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int kBlk = 128;

constexpr float kRcp448 = 0.002232142956927419f;      // 1 / 448 rounded to fp32

// fp32 `/` as the reference's Triton kernels compile it: the full-range approximate division (within 2 ulp of
// the quotient).  It matters where x / s falls within an ulp of the midpoint of two e4m3 values.
__device__ __forceinline__ float div_full(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

struct BlockQuantArgs {
  const void* in;
  void* fake_out;
  uint8_t* codes_out;
  float* scales_out;   // (ceil(rows/128), ceil(cols/128))
  int64_t rows, cols;
  int n_col_blocks;
  int triton_scale;    // 1: s = max|x| * fl(1/448) without a floor, as the reference's Triton kernel computes it
};

__device__ __forceinline__ float e4m3_value(uint8_t c) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(__half(hr));
}

// Thread t of 256 owns, for pass p = 0..PASSES-1, the 16-byte vector (row p * RPP + t / VPR, vector t % VPR)
// of the block, VPR = vectors per 128-element row, RPP = rows per pass.
template <typename T>
__global__ void __launch_bounds__(256) fp8_block_quant_kernel(BlockQuantArgs a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec, VPR = kBlk / N, RPP = 256 / VPR, PASSES = kBlk / RPP;
  __shared__ float red[8];
  const int bi = blockIdx.x / a.n_col_blocks, bj = blockIdx.x % a.n_col_blocks;
  const int vr = threadIdx.x / VPR, vc = threadIdx.x % VPR;
  const int64_t col = (int64_t)bj * kBlk + vc * N;
  const bool vec_ok = (a.cols % N == 0);   // rows stay 16-byte aligned
  float x[PASSES][N];
  float am = 0.f;
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int64_t row = (int64_t)bi * kBlk + p * RPP + vr;
#pragma unroll
    for (int e = 0; e < N; ++e) x[p][e] = 0.f;   // the reference pads ragged blocks with zeros
    if (row < a.rows) {
      const T* src = static_cast<const T*>(a.in) + row * a.cols + col;
      if (vec_ok && col + N <= a.cols) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src));
        const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int e = 0; e < N; ++e) x[p][e] = E::to_f(pv[e]);
      } else {
#pragma unroll
        for (int e = 0; e < N; ++e)
          if (col + e < a.cols) x[p][e] = E::to_f(src[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < N; ++e) am = nan_max(am, fabsf(x[p][e]));
  }
  // block abs-max
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = nan_max(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (lane == 0) red[warp] = am;
    __syncthreads();
    am = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) am = nan_max(am, red[w]);
  }
  // scales = clamp(absmax, 1e-5) / 448 in fp32 (never zero after the clamp)
  const float s = a.triton_scale ? __fmul_rn(am, kRcp448) : __fdiv_rn(nan_max(am, 1e-5f), 448.f);
  if (threadIdx.x == 0 && a.scales_out) a.scales_out[(int64_t)bi * a.n_col_blocks + bj] = s;

#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int64_t row = (int64_t)bi * kBlk + p * RPP + vr;
    if (row >= a.rows) continue;
    T fk[N];
    uint8_t cd[N];
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float u = a.triton_scale ? div_full(x[p][e], s) : __fadd_rn(__fdiv_rn(x[p][e], s), 0.f);
      const __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(u, __NV_SATFINITE, __NV_E4M3);
      cd[e] = (uint8_t)c;
      fk[e] = E::from_f(__fmul_rn(__fsub_rn(e4m3_value((uint8_t)c), 0.f), s));
    }
    const int64_t off = row * a.cols + col;
    if (vec_ok && col + N <= a.cols) {
      if (a.fake_out) __stcs(reinterpret_cast<uint4*>(static_cast<T*>(a.fake_out) + off), *reinterpret_cast<const uint4*>(fk));
      if (a.codes_out) {
        if constexpr (N == 8)
          *reinterpret_cast<uint2*>(a.codes_out + off) = *reinterpret_cast<const uint2*>(cd);
        else
          *reinterpret_cast<uint32_t*>(a.codes_out + off) = *reinterpret_cast<const uint32_t*>(cd);
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) {
        if (col + e < a.cols) {
          if (a.fake_out) static_cast<T*>(a.fake_out)[off + e] = fk[e];
          if (a.codes_out) a.codes_out[off + e] = cd[e];
        }
      }
    }
  }
}

// out = T(float(code) * scale_of_block): weight_cast_to_bf16
template <typename T>
__global__ void __launch_bounds__(256) fp8_block_dequant_kernel(const uint8_t* __restrict__ codes,
                                                                const float* __restrict__ scales, int64_t rows,
                                                                int64_t cols, int n_col_blocks, T* __restrict__ out) {
  const int64_t total = rows * cols;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total;
       i += (int64_t)gridDim.x * blockDim.x * 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t k = i + e;
      if (k < total) {
        const int64_t r = k / cols, c = k % cols;
        const float s = scales[(r / kBlk) * n_col_blocks + c / kBlk];
        out[k] = Elem<T>::from_f(__fmul_rn(__fsub_rn(e4m3_value(codes[k]), 0.f), s));
      }
    }
  }
}

// act_quant of the block-wise FP8 linear (kernel.py:7-53): per group of 128 values, s = max|x| / 448 in
// fp32 (no floor: an all-zero group gives s = 0 and NaN codes, like the reference), y = e4m3(x / s).
// The Triton kernel's `/ 448.0` is a multiplication by the fp32 reciprocal (its scales on a B200 equal
// max|x| * fl(1/448) in every case tried and the exactly rounded quotient in 41 % of them), and its
// x / s is the full-range approximate division (div_full above).
// One warp per group, four elements per lane.
template <typename T>
__global__ void __launch_bounds__(256) fp8_act_quant_kernel(const T* __restrict__ x, int64_t n_groups,
                                                            uint8_t* __restrict__ y, float* __restrict__ s_out) {
  using E = Elem<T>;
  constexpr int U = 4;   // groups per warp in flight
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t g0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * U; g0 < n_groups; g0 += warps * U) {
    float v[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t g = g0 + u;
      if (g < n_groups) {
        const T* src = x + g * kBlk + lane * 4;
        if constexpr (sizeof(T) == 4) {
          const float4 t = __ldcs(reinterpret_cast<const float4*>(src));
          v[u][0] = t.x, v[u][1] = t.y, v[u][2] = t.z, v[u][3] = t.w;
        } else {
          const uint2 t = __ldcs(reinterpret_cast<const uint2*>(src));
          const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
          for (int i = 0; i < 4; ++i) v[u][i] = E::to_f(e[i]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t g = g0 + u;
      if (g >= n_groups) break;
      float am = nan_max(nan_max(fabsf(v[u][0]), fabsf(v[u][1])), nan_max(fabsf(v[u][2]), fabsf(v[u][3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) am = nan_max(am, __shfl_xor_sync(0xffffffffu, am, o));
      const float s = __fmul_rn(am, kRcp448);
      uint8_t c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        c[i] = (uint8_t)__nv_cvt_float_to_fp8(div_full(v[u][i], s), __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint32_t*>(y + g * kBlk + lane * 4) = *reinterpret_cast<const uint32_t*>(c);
      if (lane == 0) s_out[g] = s;
    }
  }
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_fp8_e4m3_act_quant(const void* x, int dtype, int64_t n, int64_t group, void* y, float* scales,
                                            lc_stream_t stream) {
  using namespace lc;
  if (!x || !y || !scales || n <= 0 || group != kBlk) return LC_ERR_ARG;
  if (n % kBlk != 0) return LC_ERR_SHAPE;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 3u)) return LC_ERR_ALIGN;
  const int64_t n_groups = n / kBlk;
  int64_t blocks = (n_groups + 31) / 32;
  const int64_t cap = (int64_t)kNumSMsB200 * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* yo = static_cast<uint8_t*>(y);
  switch (dtype) {
    case LC_F32: fp8_act_quant_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)x, n_groups, yo, scales); break;
    case LC_BF16:
      fp8_act_quant_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)x, n_groups, yo, scales);
      break;
    case LC_F16: fp8_act_quant_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half*)x, n_groups, yo, scales); break;
    default: return LC_ERR_ARG;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

static int block_quant_impl(const void* in, int dtype, int64_t rows, int64_t cols, int64_t block, void* fake_out,
                            void* codes_out, float* scales_out, int triton_scale, lc_stream_t stream) {
  using namespace lc;
  if (rows < 0 || cols < 0 || block != kBlk) return LC_ERR_ARG;
  if (dtype != LC_F32 && dtype != LC_BF16 && dtype != LC_F16) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (!in) return LC_ERR_ARG;
  const int N = dtype == LC_F32 ? 4 : 8;
  if (cols % N == 0 && (!aligned16(in) || (fake_out && !aligned16(fake_out)))) return LC_ERR_ALIGN;
  if (cols % N == 0 && codes_out && (reinterpret_cast<uintptr_t>(codes_out) & 7u)) return LC_ERR_ALIGN;
  BlockQuantArgs a;
  a.in = in;
  a.fake_out = fake_out;
  a.codes_out = static_cast<uint8_t*>(codes_out);
  a.scales_out = scales_out;
  a.rows = rows;
  a.cols = cols;
  a.n_col_blocks = (int)((cols + kBlk - 1) / kBlk);
  a.triton_scale = triton_scale;
  const int64_t n_blocks = ((rows + kBlk - 1) / kBlk) * a.n_col_blocks;
  if (n_blocks > 0x7fffffff) return LC_ERR_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: fp8_block_quant_kernel<float><<<(unsigned)n_blocks, 256, 0, st>>>(a); break;
    case LC_BF16: fp8_block_quant_kernel<__nv_bfloat16><<<(unsigned)n_blocks, 256, 0, st>>>(a); break;
    default: fp8_block_quant_kernel<__half><<<(unsigned)n_blocks, 256, 0, st>>>(a); break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_fp8_e4m3_block_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t block,
                                              void* fake_out, void* codes_out, float* scales_out, lc_stream_t stream) {
  return block_quant_impl(in, dtype, rows, cols, block, fake_out, codes_out, scales_out, 0, stream);
}

extern "C" LC_API int lc_fp8_e4m3_block_quant_triton(const void* in, int dtype, int64_t rows, int64_t cols,
                                                     int64_t block, void* fake_out, void* codes_out, float* scales_out,
                                                     lc_stream_t stream) {
  return block_quant_impl(in, dtype, rows, cols, block, fake_out, codes_out, scales_out, 1, stream);
}

extern "C" LC_API int lc_fp8_e4m3_block_dequant(const void* codes, const float* scales, int64_t rows, int64_t cols,
                                                int64_t block, void* out, int out_dtype, lc_stream_t stream) {
  using namespace lc;
  if (rows < 0 || cols < 0 || block != kBlk) return LC_ERR_ARG;
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_F16) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (!codes || !scales || !out) return LC_ERR_ARG;
  const int ncb = (int)((cols + kBlk - 1) / kBlk);
  const int64_t work = (rows * cols + 3) / 4;
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = (int64_t)kNumSMsB200 * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* c = static_cast<const uint8_t*>(codes);
  switch (out_dtype) {
    case LC_F32: fp8_block_dequant_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(c, scales, rows, cols, ncb, (float*)out); break;
    case LC_BF16:
      fp8_block_dequant_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(c, scales, rows, cols, ncb,
                                                                              (__nv_bfloat16*)out);
      break;
    default: fp8_block_dequant_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(c, scales, rows, cols, ncb, (__half*)out); break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}
