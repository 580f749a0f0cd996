// Family 3: the GPTQ trailing update on the tensor cores, with three-level (lazy) batching.
//
// The reference updates all columns to the right after every 128-column block
// (W[:, i2:] -= Err1 @ Hinv[i1:i2, i2:], gptq.py:244): K = 128, 32 flop per byte of W traffic.  Here
// the eager update after a block only covers the rest of its 256-column sub-panel (fp32 FFMA kernel,
// at most 128 columns); the rest of the 1024-column panel is updated once per sub-panel (K = 256) and
// everything to the right of the panel once per panel,
//     W[:, p2:] -= E^T (rows x 1024) * U[p1:p2, p2:],
// a K = 1024 GEMM; both on tcgen05 with kind::tf32 and the three-term split (tf32x3_gemm.cu).  The sums are
// the reference's, associated differently.  The block kernel stores E k-major together with its low
// part; lc_gptq_split_tf32 makes the low part of U.
#include "lc_common.cuh"
#include "tf32x3_gemm.cuh"

namespace lc {
namespace {

__global__ void __launch_bounds__(256) split_tf32_kernel(const float* x, int64_t n, float* lo) {
  const int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    float4 o;
    o.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
    o.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
    o.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
    o.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
    *reinterpret_cast<float4*>(lo + i) = o;
  } else {
    for (int64_t k = i; k < n; ++k) lo[k] = x[k] - __uint_as_float(__float_as_uint(x[k]) & 0xffffe000u);
  }
}

int panel_update_launch(float* W, const float* e_hi, const float* e_lo, const float* U, const float* U_lo,
                        int64_t rows, int64_t cols, int p1, int p2, int32_t* status, cudaStream_t st) {
  if (p2 >= cols) return LC_OK;
  const int64_t off = (int64_t)p1 * cols + p2;
  return tf32x3_gemm_tn(W + p2, cols, e_hi, e_lo, rows, U + off, U_lo + off, cols, rows, cols - p2, p2 - p1, 1, -1.f,
                        0, status, st);
}

}  // namespace

int gptq_trail_launch(float* W, const float* err_t, const float* U, int64_t rows, int64_t cols, int64_t col0,
                      int k, int64_t col1, cudaStream_t st, int64_t col_end);
int gptq_block_launch(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0, int count,
                      int bits, int sym, float* err_t, float* scales, float* zeros, int64_t n_groups,
                      uint8_t* codes, float* loss_rows, cudaStream_t st, float* panel_hi, float* panel_lo,
                      int panel_k0, const int32_t* col_group);

}  // namespace lc

extern "C" LC_API int lc_gptq_split_tf32(const float* x, int64_t n, float* lo, lc_stream_t stream) {
  if (!x || !lo || n <= 0) return LC_ERR_ARG;
  if (!lc::aligned16(x) || !lc::aligned16(lo)) return LC_ERR_ALIGN;
  lc::split_tf32_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, n, lo);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_panel_update(float* W, const float* e_hi, const float* e_lo, const float* U,
                                           const float* U_lo, int64_t rows, int64_t cols, int64_t p1, int64_t p2,
                                           int32_t* status, lc_stream_t stream) {
  using namespace lc;
  if (!W || !e_hi || !e_lo || !U || !U_lo) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || p1 < 0 || p2 <= p1 || p2 > cols || (p2 - p1) % 16 != 0) return LC_ERR_ARG;
  if (cols % 4 != 0 || rows % 4 != 0 || p2 % 4 != 0) return LC_ERR_SHAPE;
  if (!aligned16(W) || !aligned16(e_hi) || !aligned16(e_lo) || !aligned16(U) || !aligned16(U_lo)) return LC_ERR_ALIGN;
  return panel_update_launch(W, e_hi, e_lo, U, U_lo, rows, cols, (int)p1, (int)p2, status,
                             reinterpret_cast<cudaStream_t>(stream));
}

// The block loop with the three-level trailing update.  n_quant < cols: owq; col_group != NULL: static
// groups (scales / zeros are input tables).
static int transform_tc(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols, int64_t n_quant,
                        int bits, int sym, float* scratch_err, float* panel_hi, float* panel_lo, float* scales,
                        float* zeros, const int32_t* col_group, uint8_t* codes_u8, float* loss_rows,
                        int32_t* status, lc_stream_t stream) {
  using namespace lc;
  constexpr int kPanel = 1024, kSub = 256;
  if (!W || !U || !U_lo || !scratch_err || !panel_hi || !panel_lo || !scales || (!zeros && !(col_group && sym)))
    return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || n_quant <= 0 || n_quant > cols || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (cols % 128 != 0 || rows % 4 != 0) return LC_ERR_SHAPE;      // TMA pitch / whole blocks; use the FFMA entry point otherwise
  if (!aligned16(W) || !aligned16(U) || !aligned16(U_lo) || !aligned16(panel_hi) || !aligned16(panel_lo)) return LC_ERR_ALIGN;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_groups = cols / 128;
  if (loss_rows) LC_CHECK_CUDA(cudaMemsetAsync(loss_rows, 0, rows * sizeof(float), st));
  // operands of every update: E (k-major panel buffer) and U, prepared once
  GemmMat E, Um;
  {
    int rc;
    if ((rc = gemm_mat_init(&E, panel_hi, panel_lo, kPanel, rows, rows)) != LC_OK) return rc;
    if ((rc = gemm_mat_init(&Um, U, U_lo, cols, cols, cols)) != LC_OK) return rc;
  }
  // Only columns [0, n_quant) are quantised; q_end rounds that up to whole 128-column blocks.  The block
  // kernel writes zero errors for the columns of a ragged last block it does not quantise, so the
  // GEMM levels may contract over whole blocks.
  const int64_t q_end = (n_quant + 127) / 128 * 128;
  for (int64_t p1 = 0; p1 < q_end; p1 += kPanel) {
    const int64_t p2 = (p1 + kPanel < cols) ? p1 + kPanel : cols;
    const int64_t pq = (p2 < q_end) ? p2 : q_end;
    for (int64_t s1 = p1; s1 < pq; s1 += kSub) {
      const int64_t s2 = (s1 + kSub < p2) ? s1 + kSub : p2;
      const int64_t sq = (s2 < q_end) ? s2 : q_end;
      for (int64_t i1 = s1; i1 < sq; i1 += 128) {
        const int count = (int)((n_quant - i1 < 128) ? (n_quant - i1) : 128);
        int rc = gptq_block_launch(W, U, rows, cols, i1, count, bits, sym, scratch_err, scales, zeros, n_groups,
                                   codes_u8, loss_rows, st, panel_hi, panel_lo, (int)(i1 - p1), col_group);
        if (rc != LC_OK) return rc;
        // level 1, eager: the rest of the 256-column sub-panel (K <= 128, at most 255 columns: FFMA kernel)
        rc = gptq_trail_launch(W, scratch_err, U, rows, cols, i1, count, i1 + count, st, s2);
        if (rc != LC_OK) return rc;
      }
      // level 2: the rest of the panel, once per sub-panel (K = 256)
      if (s2 < p2) {
        const int rc = tf32x3_gemm_launch(W + s2, cols, E, s1 - p1, 0, Um, s1, s2, rows, p2 - s2, sq - s1, 1, -1.f, 0,
                                          status, st);
        if (rc != LC_OK) return rc;
      }
    }
    // level 3: everything to the right of the panel, once per panel (K = 1024)
    if (p2 < cols) {
      const int rc = tf32x3_gemm_launch(W + p2, cols, E, 0, 0, Um, p1, p2, rows, cols - p2, pq - p1, 1, -1.f, 0, status,
                                        st);
      if (rc != LC_OK) return rc;
    }
  }
  return LC_OK;
}

extern "C" LC_API int lc_gptq_weight_transform_tc_owq(float* W, const float* U, const float* U_lo, int64_t rows,
                                                      int64_t cols, int64_t n_quant, int bits, int sym,
                                                      float* scratch_err, float* panel_hi, float* panel_lo,
                                                      float* scales, float* zeros, uint8_t* codes_u8,
                                                      float* loss_rows, int32_t* status, lc_stream_t stream) {
  return transform_tc(W, U, U_lo, rows, cols, n_quant, bits, sym, scratch_err, panel_hi, panel_lo, scales, zeros,
                      nullptr, codes_u8, loss_rows, status, stream);
}

extern "C" LC_API int lc_gptq_weight_transform_tc_static(float* W, const float* U, const float* U_lo, int64_t rows,
                                                         int64_t cols, int bits, int sym, float* scratch_err,
                                                         float* panel_hi, float* panel_lo, const float* scales,
                                                         const float* zeros, const int32_t* col_group,
                                                         uint8_t* codes_u8, float* loss_rows, int32_t* status,
                                                         lc_stream_t stream) {
  if (!col_group) return LC_ERR_ARG;
  return transform_tc(W, U, U_lo, rows, cols, cols, bits, sym, scratch_err, panel_hi, panel_lo,
                      const_cast<float*>(scales), const_cast<float*>(zeros), col_group, codes_u8, loss_rows, status,
                      stream);
}

extern "C" LC_API int lc_gptq_weight_transform_tc(float* W, const float* U, const float* U_lo, int64_t rows,
                                                  int64_t cols, int bits, int sym, float* scratch_err,
                                                  float* panel_hi, float* panel_lo, float* scales, float* zeros,
                                                  uint8_t* codes_u8, float* loss_rows, int32_t* status,
                                                  lc_stream_t stream) {
  return lc_gptq_weight_transform_tc_owq(W, U, U_lo, rows, cols, cols, bits, sym, scratch_err, panel_hi, panel_lo, scales,
                                         zeros, codes_u8, loss_rows, status, stream);
}
