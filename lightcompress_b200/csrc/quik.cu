// QUIK (llmc/compression/quantization/quik.py): mixed-precision fake quant that leaves the outlier
// feature columns in floating point, plus the per-channel activation statistic that picks them.
//
//  * col_absmax_kernel: running per-channel max |x| over calibration tokens (get_tensor_scale,
//    quik.py:35-42: view(-1, hidden).abs(), max over dim 0, max with the running value).  The
//    reference copies every per-call result to the host; here the running vector stays on the device
//    in fp32 (max is exact in any order) and is read once at the end.  HBM-bound: one read of x.
//  * row_masked_kernel: IntegerQuantizer.fake_quant_weight_dynamic / fake_quant_act_dynamic with
//    args['int_indices'] / args['fp_indices'] (quant.py:753-782, :832-868) for per_channel / per_token
//    granularity: the reference gathers the integer columns, quantises each row over them, and
//    scatters both parts into a zeroed tensor (five full-size passes).  A row's min / max do not
//    depend on the order of its columns, so a per-column byte mask (1 = keep floating point) gives
//    the same result in one read and one write; columns in neither index list come out zero, as in
//    the reference.  Arithmetic as in the one-level kernels (bit-identical to the op chain).
#include <type_traits>

#include "bf16x2.cuh"
#include "lc_common.cuh"

namespace lc {
namespace {

// ---- per-channel |x| max --------------------------------------------------------------------------
// grid (column slabs of 32 vectors, token splits); block (32, 8): thread = one 16-byte vector of
// columns, 8 row phases.  The splits meet in the running vector through integer atomics (|x| >= 0, so
// the fp32 bit pattern orders like the value; a NaN pattern sorts above +inf and therefore sticks,
// like torch.max).
template <typename T>
__global__ void __launch_bounds__(256) col_absmax_kernel(const T* x, int64_t tokens, int64_t cols, int* running) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * N;
  const int64_t per = (tokens + gridDim.y - 1) / gridDim.y;
  const int64_t t0 = blockIdx.y * per, t1 = min(tokens, t0 + per);
  int acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0;
  if (c0 < cols) {
    for (int64_t t = t0 + threadIdx.y; t < t1; t += 8) {
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(x + t * cols + c0));
      const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = max(acc[i], __float_as_int(fabsf(Elem<T>::to_f(p[i]))));
    }
  }
  __shared__ int red[8][32][N + 1];
#pragma unroll
  for (int i = 0; i < N; ++i) red[threadIdx.y][threadIdx.x][i] = acc[i];
  __syncthreads();
  if (threadIdx.y == 0 && c0 < cols) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      int m = 0;
#pragma unroll
      for (int r = 0; r < 8; ++r) m = max(m, red[r][threadIdx.x][i]);
      atomicMax(running + c0 + i, m);
    }
  }
}

// ---- masked row quantisation ----------------------------------------------------------------------
struct MaskedArgs {
  const void* in;
  void* out;
  const uint8_t* mask;      // cols bytes: 0 = quantise, 1 = keep, 2 = zero (column in neither index list)
  int64_t rows, cols;
  QRange qr;
  int sym;
};

template <typename T, int V>
__global__ void __launch_bounds__(256) row_masked_kernel(MaskedArgs a) {
  using E = Elem<T>;
  constexpr int N = E::kPerVec;
  __shared__ float s_mx[8], s_mn[8];
  const int64_t nvec = a.cols / N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the mask is the same for every row: keep this thread's slices in registers
  uint64_t mk[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int64_t i = threadIdx.x + (int64_t)k * 256;
    mk[k] = 0;
    if (i < nvec) {
      if constexpr (N == 8) mk[k] = *reinterpret_cast<const uint64_t*>(a.mask + i * 8);
      else mk[k] = *reinterpret_cast<const uint32_t*>(a.mask + i * 4);
    }
  }
  // bf16: 16-bit select masks per pair of elements (quantise / keep), for the packed-arithmetic path
  constexpr bool kPacked = std::is_same<T, __nv_bfloat16>::value && V <= 4;
  uint32_t sel[kPacked ? V : 1][4], keep[kPacked ? V : 1][4];
  if constexpr (kPacked) {
#pragma unroll
    for (int k = 0; k < V; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned b0 = (unsigned)((mk[k] >> (16 * j)) & 0xff), b1 = (unsigned)((mk[k] >> (16 * j + 8)) & 0xff);
        sel[k][j] = (b0 == 0 ? 0xffffu : 0u) | (b1 == 0 ? 0xffff0000u : 0u);
        keep[k][j] = (b0 == 1 ? 0xffffu : 0u) | (b1 == 1 ? 0xffff0000u : 0u);
      }
    }
  }
  // short rows: the next row's vectors are requested before this row is processed, so that a CTA
  // does not sit idle for a DRAM round trip per row
  constexpr bool kPrefetch = V <= 4;
  uint4 v[V], nx[kPrefetch ? V : 1];
  if (kPrefetch && (int64_t)blockIdx.x < a.rows) {
    const uint4* in0 = reinterpret_cast<const uint4*>(a.in) + (int64_t)blockIdx.x * nvec;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) v[k] = __ldcs(in0 + i);
    }
  }
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(a.in) + row * nvec;
    uint4* out = reinterpret_cast<uint4*>(a.out) + row * nvec;
    if constexpr (kPrefetch) {
      const int64_t next = row + gridDim.x;
      if (next < a.rows) {
        const uint4* inn = reinterpret_cast<const uint4*>(a.in) + next * nvec;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec) nx[k] = __ldcs(inn + i);
        }
      }
    }
    float mx = -INFINITY, mn = INFINITY;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) {
        if constexpr (!kPrefetch) v[k] = __ldcs(in + i);
        if constexpr (kPacked) {
          // elements that are not quantised are replaced by -inf / +inf before the packed max / min
          const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
          __nv_bfloat162 mx2 = bf2_of(0xff80ff80u), mn2 = bf2_of(0x7f807f80u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            mx2 = __hmax2_nan(mx2, bf2_of((w[j] & sel[k][j]) | (0xff80ff80u & ~sel[k][j])));
            mn2 = __hmin2_nan(mn2, bf2_of((w[j] & sel[k][j]) | (0x7f807f80u & ~sel[k][j])));
          }
          mx = nan_max(mx, nan_max(bf_lo(u32_of(mx2)), bf_hi(u32_of(mx2))));
          mn = nan_min(mn, nan_min(bf_lo(u32_of(mn2)), bf_hi(u32_of(mn2))));
        } else {
          float f[N];
          const T* p = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
          for (int e = 0; e < N; ++e) {
            f[e] = E::to_f(p[e]);
            if (((mk[k] >> (8 * e)) & 0xff) == 0) {
              mx = nan_max(mx, f[e]);
              mn = nan_min(mn, f[e]);
            }
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
    float s, z;
    int_qparams<T>(mn, mx, a.qr, a.sym, s, z);
    const QuantCtx c = make_quant_ctx(s, z, nan_max(fabsf(mx), fabsf(mn)));
    if constexpr (kPacked) {
      if (!c.exact) {
        const QuantCtx2 c2 = make_ctx2(c, a.qr);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int64_t i = threadIdx.x + (int64_t)k * 256;
          if (i < nvec) {
            const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t d = u32_of(dequant2(quant2(bf_lo(w[j]), bf_hi(w[j]), c, c2), c2));
              o[j] = (d & sel[k][j]) | (w[j] & keep[k][j]);      // neither bit set: zero
            }
            __stcs(out + i, make_uint4(o[0], o[1], o[2], o[3]));
          }
        }
        if constexpr (kPrefetch) {
#pragma unroll
          for (int k = 0; k < V; ++k) v[k] = nx[k];
        }
        continue;
      }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int64_t i = threadIdx.x + (int64_t)k * 256;
      if (i < nvec) {
        uint4 o = v[k];
        T* po = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const unsigned m = (unsigned)((mk[k] >> (8 * e)) & 0xff);
          if (m == 0) {
            const float q = int_quant_fast<T>(E::to_f(po[e]), c, a.qr);
            po[e] = E::from_f(int_dequant_fast<T>(q, c));
          } else if (m != 1) {
            po[e] = E::from_f(0.f);
          }
        }
        __stcs(out + i, o);
      }
    }
    if constexpr (kPrefetch) {
#pragma unroll
      for (int k = 0; k < V; ++k) v[k] = nx[k];
    }
  }
}

template <typename T>
int masked_dispatch(const MaskedArgs& a, cudaStream_t st) {
  constexpr int N = Elem<T>::kPerVec;
  if (a.cols % N != 0) return LC_ERR_SHAPE;
  if (!aligned16(a.in) || !aligned16(a.out) || (reinterpret_cast<uintptr_t>(a.mask) & 7u)) return LC_ERR_ALIGN;
  const int64_t nvec = a.cols / N;
  if (nvec > 256 * 16) return LC_ERR_SHAPE;
  int64_t blocks = a.rows;
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  if (blocks > cap) blocks = cap;
  if (nvec <= 256) row_masked_kernel<T, 1><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 512) row_masked_kernel<T, 2><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 1024) row_masked_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(a);
  else if (nvec <= 2048) row_masked_kernel<T, 8><<<(unsigned)blocks, 256, 0, st>>>(a);
  else row_masked_kernel<T, 16><<<(unsigned)blocks, 256, 0, st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

template <typename T>
int absmax_launch(const void* x, int64_t tokens, int64_t cols, float* running, cudaStream_t st) {
  constexpr int N = Elem<T>::kPerVec;
  if (cols % N != 0) return LC_ERR_SHAPE;
  if (!aligned16(x)) return LC_ERR_ALIGN;
  const int64_t slabs = (cols / N + 31) / 32;
  int64_t splits = (tokens + 63) / 64;
  const int64_t want = (int64_t)kNumSMsB200 * 8 / (slabs > 0 ? slabs : 1);
  if (splits > want) splits = want;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  dim3 grid((unsigned)slabs, (unsigned)splits), block(32, 8);
  col_absmax_kernel<T><<<grid, block, 0, st>>>(static_cast<const T*>(x), tokens, cols, reinterpret_cast<int*>(running));
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_quik_col_absmax(const void* x, int dtype, int64_t tokens, int64_t cols, float* running,
                                         lc_stream_t stream) {
  using namespace lc;
  if (!running || tokens < 0 || cols <= 0) return LC_ERR_ARG;
  if (tokens == 0) return LC_OK;
  if (!x) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return absmax_launch<float>(x, tokens, cols, running, st);
    case LC_BF16: return absmax_launch<__nv_bfloat16>(x, tokens, cols, running, st);
    case LC_F16: return absmax_launch<__half>(x, tokens, cols, running, st);
    default: return LC_ERR_ARG;
  }
}

extern "C" LC_API int lc_rtn_int_fake_quant_masked(const void* in, int dtype, int64_t rows, int64_t cols, int bits,
                                                   int sym, const uint8_t* col_mask, void* out, lc_stream_t stream) {
  using namespace lc;
  if (rows < 0 || cols < 0 || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (rows == 0 || cols == 0) return LC_OK;
  if (!in || !out || !col_mask) return LC_ERR_ARG;
  MaskedArgs a;
  a.in = in;
  a.out = out;
  a.mask = col_mask;
  a.rows = rows;
  a.cols = cols;
  a.sym = sym ? 1 : 0;
  a.qr = int_qrange(bits, a.sym);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LC_F32: return masked_dispatch<float>(a, st);
    case LC_BF16: return masked_dispatch<__nv_bfloat16>(a, st);
    case LC_F16: return masked_dispatch<__half>(a, st);
    default: return LC_ERR_ARG;
  }
}
