// Per-tensor ranges of a batch of calibration activations, for static activation quantisation
// (BaseQuantizer.get_minmax_range with granularity 'per_tensor', get_minmax_stats,
// get_static_minmax_range and get_static_moving_minmax_range,
// llmc/compression/quantization/quant.py:134-145, :223-262, :523-542).  The reference runs two
// full-tensor reductions per calibration tensor (torch.max, torch.min) and, for the moving average,
// three scalar kernels per tensor and bound; here one launch reads every tensor of the batch once
// and a second, single-warp launch folds the per-tensor values.
//
// HBM-bound: numel * sizeof(dtype) bytes read per tensor, nothing written but two floats.
//
// Min and max are exact in any order (no rounding), NaN propagates like torch.max / torch.min:
// the partial results are combined with integer atomics on an order-preserving key in which a NaN
// sorts above +inf for the maximum and below -inf for the minimum.
#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int kMaxTensors = 64;       // tensors per launch (kernel-parameter space)
constexpr int kThreads = 256;
constexpr int kVecPerThread = 8;      // 16-byte vectors per thread: 32 KB per CTA

struct RangeArgs {
  const void* ptr[kMaxTensors];
  int64_t numel[kMaxTensors];
  int cta_begin[kMaxTensors + 1];     // first CTA of each tensor
  int count;
  int32_t* key_min;                   // aliases the float outputs until range_decode_kernel ran
  int32_t* key_max;
};

// order-preserving map from fp32 bit patterns to signed integers
__device__ __forceinline__ int32_t order_key(float f) {
  const int32_t b = __float_as_int(f);
  return b >= 0 ? b : (b ^ 0x7fffffff);
}
__device__ __forceinline__ float key_value(int32_t k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }

__global__ void range_init_kernel(int32_t* key_min, int32_t* key_max, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) {
    key_min[i] = order_key(INFINITY);
    key_max[i] = order_key(-INFINITY);
  }
}

__global__ void range_decode_kernel(int32_t* key_min, int32_t* key_max, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) {
    reinterpret_cast<float*>(key_min)[i] = key_value(key_min[i]);
    reinterpret_cast<float*>(key_max)[i] = key_value(key_max[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) range_kernel(const __grid_constant__ RangeArgs a) {
  using E = Elem<T>;
  constexpr int N = 16 / (int)sizeof(T);
  // which tensor this CTA reads: cta_begin is short, a linear scan by every thread is cheap
  int t = 0;
  while (t + 1 < a.count && (int)blockIdx.x >= a.cta_begin[t + 1]) ++t;
  const int64_t n = a.numel[t];
  const T* src = static_cast<const T*>(a.ptr[t]);
  const int64_t chunk = (int64_t)kThreads * kVecPerThread * N;
  const int64_t e0 = (int64_t)((int)blockIdx.x - a.cta_begin[t]) * chunk;
  float mx = -INFINITY, mn = INFINITY;
  bool nan = false;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  if (vec_ok && e0 + chunk <= n) {
    uint4 v[kVecPerThread];
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k)
      v[k] = __ldcs(reinterpret_cast<const uint4*>(src + e0) + threadIdx.x + k * kThreads);
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const T* e = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float f = E::to_f(e[i]);
        nan |= (f != f);
        mx = fmaxf(mx, f);      // fmaxf / fminf drop NaN operands; the flag carries them
        mn = fminf(mn, f);
      }
    }
  } else {
    const int64_t end = (e0 + chunk < n) ? e0 + chunk : n;
    for (int64_t i = e0 + threadIdx.x; i < end; i += kThreads) {
      const float f = E::to_f(src[i]);
      nan |= (f != f);
      mx = fmaxf(mx, f);
      mn = fminf(mn, f);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  nan = __any_sync(0xffffffffu, nan);
  __shared__ float s_mx[kThreads / 32], s_mn[kThreads / 32];
  __shared__ int s_nan[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_mx[warp] = mx;
    s_mn[warp] = mn;
    s_nan[warp] = nan;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) {
      mx = fmaxf(mx, s_mx[w]);
      mn = fminf(mn, s_mn[w]);
      nan |= (s_nan[w] != 0);
    }
    if (nan) {
      atomicMax(a.key_max + t, order_key(__int_as_float(0x7fc00000)));
      atomicMin(a.key_min + t, order_key(__int_as_float(0xffc00000)));
    } else {
      atomicMax(a.key_max + t, order_key(mx));
      atomicMin(a.key_min + t, order_key(mn));
    }
  }
}

// m <- m + alpha * (v - m) over the tensors in order, every op rounded to T like the reference's
// 0-dim tensor arithmetic (the Python scalar alpha enters the product as an fp32 value).
template <typename T>
__global__ void moving_range_kernel(const float* mins, const float* maxs, int count, float alpha, float* out) {
  using E = Elem<T>;
  if (threadIdx.x >= 2) return;
  const float* v = threadIdx.x == 0 ? mins : maxs;
  float m = v[0];
  for (int i = 1; i < count; ++i) {
    const float d = E::rnd(__fsub_rn(v[i], m));
    const float s = E::rnd(__fmul_rn(d, alpha));
    m = E::rnd(__fadd_rn(m, s));
  }
  out[threadIdx.x] = m;
}

template <typename T>
int range_launch(const void* const* tensors, const int64_t* numels, int count, float* min_out, float* max_out,
                 cudaStream_t st) {
  constexpr int N = 16 / (int)sizeof(T);
  const int64_t chunk = (int64_t)kThreads * kVecPerThread * N;
  int32_t* kmin = reinterpret_cast<int32_t*>(min_out);
  int32_t* kmax = reinterpret_cast<int32_t*>(max_out);
  range_init_kernel<<<(count + 255) / 256, 256, 0, st>>>(kmin, kmax, count);
  LC_LAUNCH_CHECK();
  for (int t0 = 0; t0 < count; t0 += kMaxTensors) {
    RangeArgs a;
    a.count = (count - t0 < kMaxTensors) ? count - t0 : kMaxTensors;
    a.key_min = kmin + t0;
    a.key_max = kmax + t0;
    int64_t ctas = 0;
    for (int i = 0; i < a.count; ++i) {
      a.ptr[i] = tensors[t0 + i];
      a.numel[i] = numels[t0 + i];
      a.cta_begin[i] = (int)ctas;
      ctas += (numels[t0 + i] + chunk - 1) / chunk;
      if (ctas > 0x7fffffff) return LC_ERR_SHAPE;
    }
    a.cta_begin[a.count] = (int)ctas;
    if (ctas == 0) continue;
    range_kernel<T><<<(unsigned)ctas, kThreads, 0, st>>>(a);
    LC_LAUNCH_CHECK();
  }
  range_decode_kernel<<<(count + 255) / 256, 256, 0, st>>>(kmin, kmax, count);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_act_range_per_tensor(const void* const* tensors, const int64_t* numels, int count, int dtype,
                                              float* min_out, float* max_out, lc_stream_t stream) {
  using namespace lc;
  if (!tensors || !numels || !min_out || !max_out || count <= 0) return LC_ERR_ARG;
  for (int i = 0; i < count; ++i) {
    if (numels[i] <= 0 || !tensors[i]) return LC_ERR_ARG;       // torch.max of an empty tensor raises too
    if (reinterpret_cast<uintptr_t>(tensors[i]) % dtype_size(dtype)) return LC_ERR_ALIGN;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return range_launch<float>(tensors, numels, count, min_out, max_out, st);
    case LC_BF16: return range_launch<__nv_bfloat16>(tensors, numels, count, min_out, max_out, st);
    case LC_F16: return range_launch<__half>(tensors, numels, count, min_out, max_out, st);
    default: return LC_ERR_ARG;
  }
}

extern "C" LC_API int lc_act_range_moving(const float* mins, const float* maxs, int count, int dtype, double alpha,
                                          float* out2, lc_stream_t stream) {
  using namespace lc;
  if (!mins || !maxs || !out2 || count <= 0) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float a = (float)alpha;
  switch (dtype) {
    case LC_F32: moving_range_kernel<float><<<1, 32, 0, st>>>(mins, maxs, count, a, out2); break;
    case LC_BF16: moving_range_kernel<__nv_bfloat16><<<1, 32, 0, st>>>(mins, maxs, count, a, out2); break;
    case LC_F16: moving_range_kernel<__half><<<1, 32, 0, st>>>(mins, maxs, count, a, out2); break;
    default: return LC_ERR_ARG;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}
