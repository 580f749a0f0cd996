// Family 3: the data-movement steps around the GPTQ solver -- diagonal extraction for the
// act-order sort, the permute + dampen gather that feeds the Cholesky factorisation, and the
// final un-permute of the kept weights.
#include "lc_common.cuh"

namespace lc {
namespace {

__global__ void diag_kernel(const float* H, int64_t cols, float* out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cols) out[i] = H[i * cols + i];
}

// damp = percdamp * mean_i( dead_i ? 1 : hscale * H_ii ); one CTA, fixed summation order.
// late_dead (SpQR, spqr.py:143-149): the mean is taken over |hscale * H_ii| before the dead columns are set
__global__ void __launch_bounds__(1024) damp_kernel(const float* H, int64_t cols, float hscale, float percdamp,
                                                    float* damp_out, int late_dead) {
  __shared__ double red[32];
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float h = H[i * cols + i];
    if (late_dead) acc += (double)fabsf(hscale * h);
    else acc += (h == 0.f) ? 1.0 : (double)(hscale * h);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    damp_out[0] = percdamp * (float)(t / (double)cols);
  }
}

__global__ void __launch_bounds__(256) permute_h_kernel(const float* H, const int64_t* perm, int64_t cols,
                                                        float hscale, const float* damp, float* Hp, int flags) {
  const int reverse = flags & 1, upper = flags & 2;
  const int64_t i = blockIdx.y;
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= cols) return;
  // reverse: write Hp with both index orders reversed (row i, col j hold entry cols-1-i, cols-1-j)
  const int64_t si = reverse ? cols - 1 - i : i;
  const int64_t sj = reverse ? cols - 1 - j : j;
  const int64_t pi = perm ? perm[si] : si;
  const int64_t pj = perm ? perm[sj] : sj;
  // upper: H holds its upper triangle only (lc_hessian_accum_upper)
  float v = hscale * (upper && pi > pj ? H[pj * cols + pi] : H[pi * cols + pj]);
  if (i == j) {
    // a dead column's diagonal: 1 + damp (gptq.py:139-150 sets it before dampening), or exactly 1 with
    // LC_H_LATE_DEAD (spqr.py:143-149 sets it after)
    if (v == 0.f) v = (flags & 4) ? 1.f : 1.f + damp[0];
    else v += damp[0];
  }
  Hp[i * cols + j] = v;
}

template <typename T>
__global__ void __launch_bounds__(256) permute_w_kernel(const T* W, const float* H, const int64_t* perm,
                                                        int64_t rows, int64_t cols, float* Wp) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= cols) return;
  const int64_t pj = perm ? perm[j] : j;
  const bool dead = H[pj * cols + pj] == 0.f;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    Wp[r * cols + j] = dead ? 0.f : Elem<T>::to_f(W[r * cols + pj]);
  }
}

// The same two gathers with a row at a time through shared memory, so that global memory is read and written
// in whole rows (a thread per column gathers 2 or 4 bytes from a different sector for every element).
// Shared memory: cols int32 (source column, -1 = dead) + one row.
template <typename T>
__global__ void __launch_bounds__(256) permute_w_rows_kernel(const T* __restrict__ W, const float* __restrict__ H,
                                                             const int64_t* __restrict__ perm, int64_t rows,
                                                             int64_t cols, float* __restrict__ Wp) {
  extern __shared__ __align__(16) unsigned char prep_sm[];
  int32_t* sperm = reinterpret_cast<int32_t*>(prep_sm);
  T* srow = reinterpret_cast<T*>(sperm + cols);
  for (int64_t j = threadIdx.x; j < cols; j += 256) {
    const int64_t pj = perm ? perm[j] : j;
    sperm[j] = (H[pj * cols + pj] == 0.f) ? -1 : (int32_t)pj;
  }
  __syncthreads();
  constexpr int N = 16 / (int)sizeof(T);
  const bool vec = cols % N == 0 && (reinterpret_cast<uintptr_t>(W) & 15u) == 0;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* wr = W + r * cols;
    if (vec) {
      for (int64_t v = threadIdx.x; v < cols / N; v += 256)
        reinterpret_cast<uint4*>(srow)[v] = reinterpret_cast<const uint4*>(wr)[v];
    } else {
      for (int64_t j = threadIdx.x; j < cols; j += 256) srow[j] = wr[j];
    }
    __syncthreads();
    float* out = Wp + r * cols;
    for (int64_t j = threadIdx.x; j < cols; j += 256) {
      const int32_t p = sperm[j];
      out[j] = p < 0 ? 0.f : Elem<T>::to_f(srow[p]);
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256) unpermute_rows_kernel(const float* __restrict__ Wp,
                                                             const int64_t* __restrict__ perm, int64_t rows,
                                                             int64_t cols, T* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char prep_sm[];
  int32_t* sperm = reinterpret_cast<int32_t*>(prep_sm);
  float* srow = reinterpret_cast<float*>(sperm + cols);
  for (int64_t j = threadIdx.x; j < cols; j += 256) sperm[j] = (int32_t)(perm ? perm[j] : j);
  __syncthreads();
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* wr = Wp + r * cols;
    for (int64_t j = threadIdx.x; j < cols; j += 256) srow[sperm[j]] = wr[j];
    __syncthreads();
    T* o = out + r * cols;
    for (int64_t c = threadIdx.x; c < cols; c += 256) o[c] = Elem<T>::from_f(srow[c]);
    __syncthreads();
  }
}

constexpr int64_t kPrepMaxSmem = 200 * 1024;

template <typename T>
__global__ void __launch_bounds__(256) unpermute_kernel(const float* Wp, const int64_t* perm, int64_t rows,
                                                        int64_t cols, T* out) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= cols) return;
  const int64_t pj = perm ? perm[j] : j;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    out[r * cols + pj] = Elem<T>::from_f(Wp[r * cols + j]);
  }
}

// Deploy-time weight of a GPTQ-quantised linear straight from the solver's codes:
// out[r][c] = T((q - z) * s) with q = codes[r][j] + qmin, j = invperm[c] the column's place in the
// permuted order, and s, z the parameters of row r, group j / 128.  One thread per output column
// (coalesced writes; the gathered reads are one byte and mostly hit L2).
template <typename T>
__global__ void __launch_bounds__(256) dequant_unpermute_kernel(const uint8_t* __restrict__ codes,
                                                                const float* __restrict__ scales,
                                                                const float* __restrict__ zeros,
                                                                const int64_t* __restrict__ invperm, int64_t rows,
                                                                int64_t cols, int64_t n_groups, float qmin,
                                                                T* __restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t j = invperm ? invperm[c] : c;
  const int64_t g = j >> 7;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    const float q = __fadd_rn((float)codes[r * cols + j], qmin);
    const float z = zeros ? zeros[r * n_groups + g] : 0.f;
    out[r * cols + c] = Elem<T>::from_f(__fmul_rn(__fsub_rn(q, z), scales[r * n_groups + g]));
  }
}

// out[i][j] = in[n-1-i][n-1-j]
__global__ void __launch_bounds__(256) flip2_kernel(const float* in, int64_t n, float* out) {
  const int64_t i = blockIdx.y;
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j < n) out[i * n + j] = in[(n - 1 - i) * n + (n - 1 - j)];
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_gptq_flip(const float* in, int64_t n, float* out, lc_stream_t stream) {
  if (!in || !out || n <= 0 || in == out) return LC_ERR_ARG;
  dim3 g((unsigned)((n + 255) / 256), (unsigned)n);
  lc::flip2_kernel<<<g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, n, out);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_diag(const float* H, int64_t cols, float* diag_out, lc_stream_t stream) {
  if (!H || !diag_out || cols <= 0) return LC_ERR_ARG;
  lc::diag_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(H, cols,
                                                                                                     diag_out);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_permute_damp(const void* W, int w_dtype, const float* H, const int64_t* perm, int64_t rows,
                                    int64_t cols, float hscale, float percdamp, int reverse_h, float* Wp,
                                    float* Hp, float* scratch, lc_stream_t stream) {
  using namespace lc;
  if (!H || cols <= 0 || (W != nullptr) != (Wp != nullptr) || (Hp && !scratch) || (!W && !Hp)) return LC_ERR_ARG;
  if (W && rows <= 0) return LC_ERR_ARG;
  if (w_dtype != LC_F32 && w_dtype != LC_BF16 && w_dtype != LC_F16) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (Hp) {
    damp_kernel<<<1, 1024, 0, st>>>(H, cols, hscale, percdamp, scratch, (reverse_h & 4) ? 1 : 0);
    LC_LAUNCH_CHECK();
    dim3 gh((unsigned)((cols + 255) / 256), (unsigned)cols);
    permute_h_kernel<<<gh, 256, 0, st>>>(H, perm, cols, hscale, scratch, Hp, reverse_h);
    LC_LAUNCH_CHECK();
  }
  if (!W) return LC_OK;
  {
    // a row at a time through shared memory when a row and the column table fit
    const int64_t esz = w_dtype == LC_F32 ? 4 : 2;
    const int64_t smem = cols * (4 + esz);
    if (smem <= kPrepMaxSmem) {
      const unsigned grid = (unsigned)(rows < 8 * kNumSMsB200 ? rows : 8 * kNumSMsB200);
      switch (w_dtype) {
        case LC_F32:
          LC_CHECK_CUDA(cudaFuncSetAttribute(permute_w_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kPrepMaxSmem));
          permute_w_rows_kernel<float><<<grid, 256, (size_t)smem, st>>>((const float*)W, H, perm, rows, cols, Wp);
          break;
        case LC_BF16:
          LC_CHECK_CUDA(cudaFuncSetAttribute(permute_w_rows_kernel<__nv_bfloat16>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrepMaxSmem));
          permute_w_rows_kernel<__nv_bfloat16><<<grid, 256, (size_t)smem, st>>>((const __nv_bfloat16*)W, H, perm, rows,
                                                                                  cols, Wp);
          break;
        default:
          LC_CHECK_CUDA(cudaFuncSetAttribute(permute_w_rows_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kPrepMaxSmem));
          permute_w_rows_kernel<__half><<<grid, 256, (size_t)smem, st>>>((const __half*)W, H, perm, rows, cols, Wp);
          break;
      }
      LC_LAUNCH_CHECK();
      return LC_OK;
    }
  }
  dim3 gw((unsigned)((cols + 255) / 256), (unsigned)(rows < 1024 ? rows : 1024));
  switch (w_dtype) {
    case LC_F32: permute_w_kernel<float><<<gw, 256, 0, st>>>((const float*)W, H, perm, rows, cols, Wp); break;
    case LC_BF16:
      permute_w_kernel<__nv_bfloat16><<<gw, 256, 0, st>>>((const __nv_bfloat16*)W, H, perm, rows, cols, Wp);
      break;
    default: permute_w_kernel<__half><<<gw, 256, 0, st>>>((const __half*)W, H, perm, rows, cols, Wp); break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_unpermute(const float* Wp, const int64_t* perm, int64_t rows, int64_t cols, void* out,
                                 int out_dtype, lc_stream_t stream) {
  using namespace lc;
  if (!Wp || !out || rows <= 0 || cols <= 0) return LC_ERR_ARG;
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_F16) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cols * 8 <= kPrepMaxSmem) {
    const size_t smem = (size_t)cols * 8;
    const unsigned grid = (unsigned)(rows < 8 * kNumSMsB200 ? rows : 8 * kNumSMsB200);
    switch (out_dtype) {
      case LC_F32:
        LC_CHECK_CUDA(cudaFuncSetAttribute(unpermute_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)kPrepMaxSmem));
        unpermute_rows_kernel<float><<<grid, 256, smem, st>>>(Wp, perm, rows, cols, (float*)out);
        break;
      case LC_BF16:
        LC_CHECK_CUDA(cudaFuncSetAttribute(unpermute_rows_kernel<__nv_bfloat16>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrepMaxSmem));
        unpermute_rows_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(Wp, perm, rows, cols, (__nv_bfloat16*)out);
        break;
      default:
        LC_CHECK_CUDA(cudaFuncSetAttribute(unpermute_rows_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)kPrepMaxSmem));
        unpermute_rows_kernel<__half><<<grid, 256, smem, st>>>(Wp, perm, rows, cols, (__half*)out);
        break;
    }
    LC_LAUNCH_CHECK();
    return LC_OK;
  }
  dim3 g((unsigned)((cols + 255) / 256), (unsigned)(rows < 1024 ? rows : 1024));
  switch (out_dtype) {
    case LC_F32: unpermute_kernel<float><<<g, 256, 0, st>>>(Wp, perm, rows, cols, (float*)out); break;
    case LC_BF16: unpermute_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(Wp, perm, rows, cols, (__nv_bfloat16*)out); break;
    default: unpermute_kernel<__half><<<g, 256, 0, st>>>(Wp, perm, rows, cols, (__half*)out); break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_dequant_unpermute(const uint8_t* codes, const float* scales, const float* zeros,
                                                const int64_t* invperm, int64_t rows, int64_t cols, int bits, int sym,
                                                void* out, int out_dtype, lc_stream_t stream) {
  using namespace lc;
  if (!codes || !scales || !out || rows <= 0 || cols <= 0 || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_F16) return LC_ERR_ARG;
  const int64_t n_groups = (cols + 127) / 128;
  const float qmin = int_qrange(bits, sym ? 1 : 0).qmin;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 g((unsigned)((cols + 255) / 256), (unsigned)(rows < 1024 ? rows : 1024));
  switch (out_dtype) {
    case LC_F32:
      dequant_unpermute_kernel<float><<<g, 256, 0, st>>>(codes, scales, zeros, invperm, rows, cols, n_groups, qmin,
                                                         (float*)out);
      break;
    case LC_BF16:
      dequant_unpermute_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(codes, scales, zeros, invperm, rows, cols, n_groups,
                                                                 qmin, (__nv_bfloat16*)out);
      break;
    default:
      dequant_unpermute_kernel<__half><<<g, 256, 0, st>>>(codes, scales, zeros, invperm, rows, cols, n_groups, qmin,
                                                          (__half*)out);
      break;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}
