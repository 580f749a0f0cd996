// Histograms of a batch of calibration activations, for calib_algo 'static_hist'
// (BaseQuantizer.get_static_hist_range, llmc/compression/quantization/quant.py:461-521, which calls
// torch.histc(tensor.float(), bins, min, max) once per calibration tensor).  One launch reads every tensor
// of the batch once; each tensor has its own range.
//
// Binning follows torch.histc on CUDA for fp32 input: values outside [min, max] are not counted,
//     bin = (int)((x - min) * bins / (max - min))       (fp32, left to right)
// and a value that lands on `bins` (x == max) belongs to the last bin.  NaN is not counted.
//
// HBM-bound: numel * sizeof(dtype) bytes read per tensor; 4 * bins bytes written per tensor.
// Counts are accumulated as integers in shared memory, then added to the fp32 result, so a bin is exact
// up to 2^24 elements per CTA contribution (torch accumulates its float bins with atomic adds as well).
#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int kMaxTensors = 64;
constexpr int kThreads = 256;
constexpr int kVecPerThread = 8;
constexpr int kMaxBins = 4096;

struct HistArgs {
  const void* ptr[kMaxTensors];
  int64_t numel[kMaxTensors];
  int cta_begin[kMaxTensors + 1];
  int count;
  int bins;
  const float* mins;     // per tensor
  const float* maxs;
  float* hist;           // [count][bins], zeroed by the caller side of this file
};

template <typename T>
__global__ void __launch_bounds__(kThreads) hist_kernel(const __grid_constant__ HistArgs a) {
  using E = Elem<T>;
  constexpr int N = 16 / (int)sizeof(T);
  extern __shared__ int s_bins[];
  int t = 0;
  while (t + 1 < a.count && (int)blockIdx.x >= a.cta_begin[t + 1]) ++t;
  for (int i = threadIdx.x; i < a.bins; i += kThreads) s_bins[i] = 0;
  __syncthreads();
  const int64_t n = a.numel[t];
  const T* src = static_cast<const T*>(a.ptr[t]);
  const float lo = a.mins[t], hi = a.maxs[t];
  const float width = hi - lo, nb = (float)a.bins;
  const int64_t chunk = (int64_t)kThreads * kVecPerThread * N;
  // several chunks per CTA (grid-stride over the tensor's CTAs) keep the shared-memory flush rare
  const int ctas = a.cta_begin[t + 1] - a.cta_begin[t];
  const bool vec_ok = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  auto put = [&](float f) {
    if (f >= lo && f <= hi) {
      int b = (int)(__fdiv_rn(__fmul_rn(__fsub_rn(f, lo), nb), width));
      if (b == a.bins) b -= 1;
      if (b >= 0 && b < a.bins) atomicAdd(&s_bins[b], 1);
    }
  };
  for (int64_t e0 = (int64_t)((int)blockIdx.x - a.cta_begin[t]) * chunk; e0 < n; e0 += (int64_t)ctas * chunk) {
    if (vec_ok && e0 + chunk <= n) {
      uint4 v[kVecPerThread];
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k)
        v[k] = __ldcs(reinterpret_cast<const uint4*>(src + e0) + threadIdx.x + k * kThreads);
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k) {
        const T* e = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
        for (int i = 0; i < N; ++i) put(E::to_f(e[i]));
      }
    } else {
      const int64_t end = (e0 + chunk < n) ? e0 + chunk : n;
      for (int64_t i = e0 + threadIdx.x; i < end; i += kThreads) put(E::to_f(src[i]));
    }
  }
  __syncthreads();
  float* out = a.hist + (int64_t)t * a.bins;
  for (int i = threadIdx.x; i < a.bins; i += kThreads)
    if (s_bins[i]) atomicAdd(out + i, (float)s_bins[i]);
}

template <typename T>
int hist_launch(const void* const* tensors, const int64_t* numels, int count, int bins, const float* mins,
                const float* maxs, float* hist, cudaStream_t st) {
  constexpr int N = 16 / (int)sizeof(T);
  const int64_t chunk = (int64_t)kThreads * kVecPerThread * N;
  LC_CHECK_CUDA(cudaMemsetAsync(hist, 0, (size_t)count * bins * sizeof(float), st));
  for (int first = 0; first < count; first += kMaxTensors) {
    const int nb = count - first < kMaxTensors ? count - first : kMaxTensors;
    HistArgs a;
    a.count = nb;
    a.bins = bins;
    a.mins = mins + first;
    a.maxs = maxs + first;
    a.hist = hist + (int64_t)first * bins;
    int cta = 0;
    for (int i = 0; i < nb; ++i) {
      a.ptr[i] = tensors[first + i];
      a.numel[i] = numels[first + i];
      a.cta_begin[i] = cta;
      // at most 4 CTAs per SM per tensor: beyond that a CTA loops over several chunks
      int64_t want = (numels[first + i] + chunk - 1) / chunk;
      const int64_t cap = 4 * kNumSMsB200;
      if (want > cap) want = cap;
      cta += (int)(want > 0 ? want : 1);
    }
    a.cta_begin[nb] = cta;
    hist_kernel<T><<<cta, kThreads, bins * sizeof(int), st>>>(a);
    LC_LAUNCH_CHECK();
  }
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_act_hist_per_tensor(const void* const* tensors, const int64_t* numels, int count, int dtype,
                                             const float* mins, const float* maxs, int bins, float* hist,
                                             lc_stream_t stream) {
  using namespace lc;
  if (!tensors || !numels || !mins || !maxs || !hist || count <= 0) return LC_ERR_ARG;
  if (bins <= 0 || bins > kMaxBins) return LC_ERR_ARG;
  for (int i = 0; i < count; ++i) {
    if (numels[i] <= 0 || !tensors[i]) return LC_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(tensors[i]) % dtype_size(dtype)) return LC_ERR_ALIGN;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return hist_launch<float>(tensors, numels, count, bins, mins, maxs, hist, st);
    case LC_BF16: return hist_launch<__nv_bfloat16>(tensors, numels, count, bins, mins, maxs, hist, st);
    case LC_F16: return hist_launch<__half>(tensors, numels, count, bins, mins, maxs, hist, st);
    default: return LC_ERR_ARG;
  }
}
