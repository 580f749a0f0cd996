// MSE range search of the integer quantizer (calib_algo 'mse'): for every group the clipping range
// [min, max] is shrunk over a grid of steps and the range with the smallest sum |qdq(x) - x|^norm
// wins (IntegerQuantizer.get_tensor_range -> BaseQuantizer.get_mse_range,
// llmc/compression/quantization/quant.py:147-205, with get_qparams :544-558 and quant_dequant
// :698-716 inside the loop).  The reference launches about a dozen full-tensor ops per grid step
// (80 steps by default); here a warp owns a group, keeps it in registers and walks the whole grid.
//
// Arithmetic follows the reference op for op in fp32 (it converts the tensor with .float() first):
// p = 1 - i / grid as a double rounded to fp32, the range of step i derived from the BEST range so
// far (the reference updates its min / max tensors in place through the views it shrinks from, so
// accepted shrinks compound), IEEE divisions, round-half-even, powf for the error norm, the group
// sum associated like torch's row reduction (four running sums per lane over 16-byte vectors lane,
// lane + 32, ...; folded left to right; butterfly with offsets 16..1), strict `<` for the update.
// Compute-bound (powf): about 290 instructions per element-step.
#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int kMaxVec = 16;   // 16-byte vectors per lane: groups of up to 2048 elements stay in registers

struct MseArgs {
  const void* in;
  float* min_out;
  float* max_out;
  int64_t n_groups;
  int group;        // multiple of 128
  int sym;
  int steps;        // int(maxshrink * grid)
  double grid;
  float norm;
  QRange qr;
};

template <typename T>
__device__ __forceinline__ void load_vec4(const T* p, float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = Elem<T>::to_f(e[i]);
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(256) mse_range_kernel(MseArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= a.n_groups) return;
  const T* src = static_cast<const T*>(a.in) + g * a.group;
  float x[NV][4];
  float mx = -INFINITY, mn = INFINITY;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    load_vec4(src + ((j << 5) + lane) * 4, x[j]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      mx = nan_max(mx, x[j][i]);
      mn = nan_min(mn, x[j][i]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }

  float best = INFINITY, best_min = mn, best_max = mx;
  const float qspan = __fsub_rn(a.qr.qmax, a.qr.qmin);
  for (int i = 0; i < a.steps; ++i) {
    const float p = (float)(1.0 - (double)i / a.grid);
    const float xmin = __fmul_rn(p, best_min), xmax = __fmul_rn(p, best_max);
    float s, z;
    if (a.sym) {
      const float am = nan_max(nan_max(fabsf(xmax), fabsf(xmin)), 1e-5f);
      s = __fdiv_rn(am, a.qr.qmax);
      z = 0.f;
    } else {
      const float d = nan_max(__fsub_rn(xmax, xmin), 1e-5f);
      s = __fdiv_rn(d, qspan);
      z = clampf(__fsub_rn(a.qr.qmin, rintf(__fdiv_rn(xmin, s))), a.qr.qmin, a.qr.qmax);
    }
    const QuantCtx qc = make_quant_ctx(s, z, nan_max(fabsf(mx), fabsf(mn)));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NV; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float q = int_quant_fast<float>(x[j][e], qc, a.qr);
        const float dq = int_dequant_fast<float>(q, qc);
        const float d = fabsf(__fsub_rn(dq, x[j][e]));
        acc[e] = __fadd_rn(acc[e], powf(d, a.norm));
      }
    }
    float err = __fadd_rn(__fadd_rn(__fadd_rn(acc[0], acc[1]), acc[2]), acc[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) err = __fadd_rn(err, __shfl_xor_sync(0xffffffffu, err, o));
    if (err < best) {
      best = err;
      best_min = xmin;
      best_max = xmax;
    }
  }
  if (lane == 0) {
    a.min_out[g] = best_min;
    a.max_out[g] = best_max;
  }
}

template <typename T>
int launch(const MseArgs& a, cudaStream_t st) {
  const unsigned grid = (unsigned)((a.n_groups + 7) / 8);
  switch (a.group / 128) {
    case 1: mse_range_kernel<T, 1><<<grid, 256, 0, st>>>(a); break;
    case 2: mse_range_kernel<T, 2><<<grid, 256, 0, st>>>(a); break;
    case 4: mse_range_kernel<T, 4><<<grid, 256, 0, st>>>(a); break;
    case 8: mse_range_kernel<T, 8><<<grid, 256, 0, st>>>(a); break;
    case 16: mse_range_kernel<T, kMaxVec><<<grid, 256, 0, st>>>(a); break;
    default: return LC_ERR_SHAPE;
  }
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_rtn_mse_range(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group, int bits,
                                       int sym, double maxshrink, int mse_grid, float norm, float* min_out,
                                       float* max_out, lc_stream_t stream) {
  using namespace lc;
  if (!in || !min_out || !max_out || rows <= 0 || cols <= 0) return LC_ERR_ARG;
  if (bits < 2 || bits > 8 || mse_grid < 1 || !(maxshrink > 0.0) || maxshrink > 1.0) return LC_ERR_ARG;
  const int64_t g = group ? group : cols;
  if (cols % g != 0) return LC_ERR_SHAPE;
  // 128, 256, 512, 1024 or 2048 elements per group
  if (g % 128 != 0 || g > 2048 || ((g / 128) & (g / 128 - 1)) != 0) return LC_ERR_SHAPE;
  if (!aligned16(in)) return LC_ERR_ALIGN;
  MseArgs a;
  a.in = in;
  a.min_out = min_out;
  a.max_out = max_out;
  a.n_groups = rows * (cols / g);
  a.group = (int)g;
  a.sym = sym ? 1 : 0;
  a.steps = (int)(maxshrink * mse_grid);
  a.grid = (double)mse_grid;
  a.norm = norm;
  a.qr = int_qrange(bits, a.sym);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return launch<float>(a, st);
    case LC_BF16: return launch<__nv_bfloat16>(a, st);
    case LC_F16: return launch<__half>(a, st);
    default: return LC_ERR_ARG;
  }
}
