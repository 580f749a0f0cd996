// Family 3: trailing update of the GPTQ solver,  W[:, col1:] -= Err * U[col0:col0+k, col1:].
//
// fp32 in, fp32 out, K <= 128, so the update is bound by the read-modify-write of W
// (32 flop per byte); an fp32 FFMA tile kernel keeps the reference's fp32 products.
// Err is stored k-major ([128][rows]) by the block kernel so that both operand tiles are
// contiguous along the dimension the threads walk.
//
// CTA tile 128 (rows) x 128 (cols), 256 threads, 8x8 accumulators per thread, K in chunks of
// 16 staged through shared memory with register prefetch of the next chunk.
#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int TM = 128, TN = 128, TK = 16;

struct TrailArgs {
  float* W;
  const float* err_t;  // [128][rows]
  const float* U;
  int64_t rows, cols, col0, col1, col_end;  // updates columns [col1, col_end)
  int k;
};

template <bool VEC>
__global__ void __launch_bounds__(256) gptq_trail_kernel(TrailArgs a) {
  __shared__ __align__(16) float As[2][TK][TM];
  __shared__ __align__(16) float Bs[2][TK][TN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM;
  const int64_t n0 = a.col1 + (int64_t)blockIdx.x * TN;

  // global -> smem assignment: each thread moves 2 float4 of A and 2 of B per chunk
  // A chunk: TK rows (k) x TM floats (m): 16 x 32 float4 = 512 float4
  float4 pa[2], pb[2];
  auto load_chunk = [&](int kc) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int v = tid + t * 256;
      const int kk = v >> 5, c4 = (v & 31) * 4;
      const int kg = kc * TK + kk;
      float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vb = va;
      if (kg < a.k) {
        const float* pa_g = a.err_t + (int64_t)kg * a.rows + m0 + c4;
        const float* pb_g = a.U + (a.col0 + kg) * a.cols + n0 + c4;
        if (VEC) {
          if (m0 + c4 < a.rows) va = *reinterpret_cast<const float4*>(pa_g);
          if (n0 + c4 < a.col_end) vb = *reinterpret_cast<const float4*>(pb_g);
        } else {
          if (m0 + c4 + 0 < a.rows) va.x = pa_g[0];
          if (m0 + c4 + 1 < a.rows) va.y = pa_g[1];
          if (m0 + c4 + 2 < a.rows) va.z = pa_g[2];
          if (m0 + c4 + 3 < a.rows) va.w = pa_g[3];
          if (n0 + c4 + 0 < a.col_end) vb.x = pb_g[0];
          if (n0 + c4 + 1 < a.col_end) vb.y = pb_g[1];
          if (n0 + c4 + 2 < a.col_end) vb.z = pb_g[2];
          if (n0 + c4 + 3 < a.col_end) vb.w = pb_g[3];
        }
      }
      pa[t] = va;
      pb[t] = vb;
    }
  };
  auto store_chunk = [&](int buf) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int v = tid + t * 256;
      const int kk = v >> 5, c4 = (v & 31) * 4;
      *reinterpret_cast<float4*>(&As[buf][kk][c4]) = pa[t];
      *reinterpret_cast<float4*>(&Bs[buf][kk][c4]) = pb[t];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int nchunks = (a.k + TK - 1) / TK;
  load_chunk(0);
  store_chunk(0);
  __syncthreads();
  for (int kc = 0; kc < nchunks; ++kc) {
    const int buf = kc & 1;
    if (kc + 1 < nchunks) load_chunk(kc + 1);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kc + 1 < nchunks) {
      store_chunk(buf ^ 1);
      __syncthreads();
    }
  }

  // W -= acc
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= a.rows) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t n = n0 + (h == 0 ? tx * 4 : 64 + tx * 4);
      float* p = a.W + m * a.cols + n;
      if (VEC) {
        if (n < a.col_end) {
          float4 c = *reinterpret_cast<float4*>(p);
          c.x -= acc[i][h * 4 + 0];
          c.y -= acc[i][h * 4 + 1];
          c.z -= acc[i][h * 4 + 2];
          c.w -= acc[i][h * 4 + 3];
          *reinterpret_cast<float4*>(p) = c;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < a.col_end) p[j] -= acc[i][h * 4 + j];
      }
    }
  }
}

}  // namespace

int gptq_trail_launch(float* W, const float* err_t, const float* U, int64_t rows, int64_t cols, int64_t col0,
                      int k, int64_t col1, cudaStream_t st, int64_t col_end) {
  if (col_end < 0 || col_end > cols) col_end = cols;
  if (col1 >= col_end) return LC_OK;
  TrailArgs a{W, err_t, U, rows, cols, col0, col1, col_end, k};
  dim3 grid((unsigned)((col_end - col1 + TN - 1) / TN), (unsigned)((rows + TM - 1) / TM));
  const bool vec = (cols % 4 == 0) && (rows % 4 == 0) && (col1 % 4 == 0) && (col_end % 4 == 0) && aligned16(W) &&
                   aligned16(err_t) && aligned16(U);
  if (vec) gptq_trail_kernel<true><<<grid, 256, 0, st>>>(a);
  else gptq_trail_kernel<false><<<grid, 256, 0, st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

int gptq_block_launch(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0, int count,
                      int bits, int sym, float* err_t, float* scales, float* zeros, int64_t n_groups,
                      uint8_t* codes, float* loss_rows, cudaStream_t st, float* panel_hi, float* panel_lo,
                      int panel_k0, const int32_t* col_group);

}  // namespace lc

extern "C" LC_API int lc_gptq_trailing_update(float* W, const float* err, const float* U, int64_t rows, int64_t cols,
                                       int64_t col0, int k, int64_t col1, lc_stream_t stream) {
  if (!W || !err || !U) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || k < 1 || k > 128 || col0 < 0 || col0 + k > cols || col1 < col0 + k) return LC_ERR_ARG;
  return lc::gptq_trail_launch(W, err, U, rows, cols, col0, k, col1, reinterpret_cast<cudaStream_t>(stream), -1);
}

// ---- allocation-free variant -------------------------------------------------------------------
// Some callers can hand over their weight and factor buffers but cannot obtain scratch memory at
// call time: a serving or export process whose device memory is entirely owned by a pool or an
// arena it must not grow, or code running where cudaMalloc / the torch caching allocator is off
// limits (inside a region that forbids allocation, or a plugin host that gives the plugin no
// allocator).  For them the Err scratch of the block loop lives in a fixed device array that is
// part of this library's image.  Every GPU that loads the library carries these 8 MiB until the
// process exits.
constexpr int64_t kNoAllocMaxRows = 16384;  // rows of W the fixed scratch can serve
static __device__ __align__(256) float g_noalloc_err[128 * kNoAllocMaxRows];

namespace lc {
namespace {
constexpr int kMaxDevices = 64;
// Device address of g_noalloc_err per device ordinal.  In host code the array's name is only a
// handle: the address a kernel can use must be asked for, once per device, with that device current.
float* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_scratch(float** out) {
  int dev = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return LC_ERR_ARG;
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_err) != cudaSuccess || p == nullptr) return LC_ERR_CUDA;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return LC_OK;
}
}  // namespace
}  // namespace lc

extern "C" LC_API int lc_gptq_weight_transform_noalloc(float* W, const float* U, int64_t rows, int64_t cols,
                                                       int bits, int sym, float* scales, float* zeros,
                                                       uint8_t* codes_u8, float* loss_rows, lc_stream_t stream) {
  if (rows > kNoAllocMaxRows) return LC_ERR_WORKSPACE;  // the built-in scratch holds 128 x 16384 floats
  float* scratch = nullptr;
  const int rc = lc::noalloc_scratch(&scratch);
  if (rc != LC_OK) return rc;
  return lc_gptq_weight_transform(W, U, rows, cols, bits, sym, scratch, scales, zeros, codes_u8, loss_rows, stream);
}

// The block loop of GPTQ.weight_transform with the FFMA trailing update.  n_quant < cols: owq;
// col_group != NULL: static groups (scales / zeros are input tables).
static int transform_ffma(float* W, const float* U, int64_t rows, int64_t cols, int64_t n_quant, int bits, int sym,
                          float* scratch_err, float* scales, float* zeros, const int32_t* col_group,
                          uint8_t* codes_u8, float* loss_rows, lc_stream_t stream) {
  if (!W || !U || !scratch_err || !scales || (!zeros && !(col_group && sym))) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || n_quant <= 0 || n_quant > cols || bits < 2 || bits > 8) return LC_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_groups = (cols + 127) / 128;
  if (loss_rows) LC_CHECK_CUDA(cudaMemsetAsync(loss_rows, 0, rows * sizeof(float), st));
  for (int64_t i1 = 0; i1 < n_quant; i1 += 128) {
    const int count = (int)((n_quant - i1 < 128) ? (n_quant - i1) : 128);
    int rc = lc::gptq_block_launch(W, U, rows, cols, i1, count, bits, sym, scratch_err, scales, zeros, n_groups,
                                   codes_u8, loss_rows, st, nullptr, nullptr, 0, col_group);
    if (rc != LC_OK) return rc;
    rc = lc::gptq_trail_launch(W, scratch_err, U, rows, cols, i1, count, i1 + count, st, -1);
    if (rc != LC_OK) return rc;
  }
  return LC_OK;
}

extern "C" LC_API int lc_gptq_weight_transform_owq(float* W, const float* U, int64_t rows, int64_t cols, int64_t n_quant,
                                                   int bits, int sym, float* scratch_err, float* scales, float* zeros,
                                                   uint8_t* codes_u8, float* loss_rows, lc_stream_t stream) {
  return transform_ffma(W, U, rows, cols, n_quant, bits, sym, scratch_err, scales, zeros, nullptr, codes_u8, loss_rows,
                        stream);
}

extern "C" LC_API int lc_gptq_weight_transform_static(float* W, const float* U, int64_t rows, int64_t cols, int bits,
                                                      int sym, float* scratch_err, const float* scales,
                                                      const float* zeros, const int32_t* col_group, uint8_t* codes_u8,
                                                      float* loss_rows, lc_stream_t stream) {
  if (!col_group) return LC_ERR_ARG;
  return transform_ffma(W, U, rows, cols, cols, bits, sym, scratch_err, const_cast<float*>(scales),
                        const_cast<float*>(zeros), col_group, codes_u8, loss_rows, stream);
}

extern "C" LC_API int lc_gptq_weight_transform(float* W, const float* U, int64_t rows, int64_t cols, int bits, int sym,
                                        float* scratch_err, float* scales, float* zeros, uint8_t* codes_u8,
                                        float* loss_rows, lc_stream_t stream) {
  return lc_gptq_weight_transform_owq(W, U, rows, cols, cols, bits, sym, scratch_err, scales, zeros, codes_u8, loss_rows,
                                      stream);
}
