// Family 3: the 128-column in-block step of the GPTQ solver.
//
// Rows of W are independent (they only share the inverse-Hessian factor U), so one warp owns
// one row: lane l keeps columns l, l+32, l+64, l+96 of the block in registers.  The 128x128
// diagonal block of U sits in shared memory and is shared by the 16 rows of the CTA.  The 128
// dependent column steps run entirely in registers / shuffles; nothing is written to global
// memory until the block is finished.
#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int kBlk = 128;          // block size == group size
constexpr int kRowsPerCta = 16;    // one warp per row
constexpr int kThreads = kRowsPerCta * 32;

struct BlockArgs {
  float* W;
  const float* U;
  float* err_t;       // [128][rows]
  float* panel_hi;    // optional [panel depth][rows]: err again, row panel_k0 + i (tensor-core operand)
  float* panel_lo;    // optional: err - tf32_truncate(err), same layout
  int panel_k0;
  float* scales;
  float* zeros;
  uint8_t* codes;
  float* loss_rows;
  int64_t rows, cols, col0, n_groups;
  int count, sym;
  QRange qr;
};

__global__ void __launch_bounds__(kThreads) gptq_block_kernel(BlockArgs a) {
  extern __shared__ float u1[];  // [128][128], zero outside count x count; then 128 reciprocals of its diagonal
  float* dinv = u1 + kBlk * kBlk;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int idx = threadIdx.x; idx < kBlk * kBlk; idx += kThreads) {
    const int i = idx >> 7, j = idx & 127;
    float v = 0.f;
    if (i < a.count && j < a.count && j >= i) v = a.U[(a.col0 + i) * a.cols + a.col0 + j];
    u1[idx] = v;
    if (i == j) dinv[i] = __frcp_rn(v);
  }
  __syncthreads();

  const int64_t r = (int64_t)blockIdx.x * kRowsPerCta + warp;
  if (r >= a.rows) return;

  float* wrow = a.W + r * a.cols + a.col0;
  float w[4], er[4];
  int cd[4];
  bool valid[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int j = lane + 32 * c;
    valid[c] = j < a.count;
    w[c] = valid[c] ? wrow[j] : 0.f;
    er[c] = 0.f;
    cd[c] = 0;
  }

  // group qparams from the block's current columns (GPTQ.search_column_qparams)
  float mx = -INFINITY, mn = INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (valid[c]) {
      mx = nan_max(mx, w[c]);
      mn = nan_min(mn, w[c]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  float s, z;
  int_qparams<float>(mn, mx, a.qr, a.sym, s, z);
  // error feedback can move a weight a little outside the block's initial range: leave headroom
  const QuantCtx qc = make_quant_ctx(s, z, 16.f * nan_max(fabsf(mx), fabsf(mn)));

  float loss = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int lim = min(32, a.count - 32 * c);
    for (int il = 0; il < lim; ++il) {
      const int i = 32 * c + il;
      const float wi = __shfl_sync(0xffffffffu, w[c], il);
      const float d = u1[i * kBlk + i], rd = dinv[i];
      const float q = int_quant_fast<float>(wi, qc, a.qr);   // the same code the IEEE division gives
      const float dq = int_dequant_fast<float>(q, qc);
      const float diff = __fsub_rn(wi, dq);
      // (w - q) / d through the precomputed reciprocal and one residual correction: within an ulp
      // of the IEEE quotient (the value only feeds the error propagation)
      const float e0 = __fmul_rn(diff, rd);
      const float err = __fmaf_rn(__fmaf_rn(-e0, d, diff), rd, e0);
      loss = fmaf(0.5f * err, err, loss);
      if (lane == il) {
        er[c] = err;
        cd[c] = code_to_int(q) - (int)a.qr.qmin;
      }
      // W1[:, i:] -= err * U1[i, i:]; column i itself is never read again
#pragma unroll
      for (int c2 = c; c2 < 4; ++c2) {
        const float u = u1[i * kBlk + lane + 32 * c2];
        const float upd = __fsub_rn(w[c2], __fmul_rn(err, u));
        if (c2 > c || lane > il) w[c2] = upd;
      }
    }
  }

#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int j = lane + 32 * c;
    if (valid[c]) {
      wrow[j] = w[c];
      if (a.codes) a.codes[r * a.cols + a.col0 + j] = (uint8_t)cd[c];
    }
    a.err_t[(int64_t)j * a.rows + r] = er[c];
    if (a.panel_hi) {
      const float hi = __uint_as_float(__float_as_uint(er[c]) & 0xffffe000u);
      a.panel_hi[(int64_t)(a.panel_k0 + j) * a.rows + r] = er[c];
      a.panel_lo[(int64_t)(a.panel_k0 + j) * a.rows + r] = er[c] - hi;
    }
  }
  if (lane == 0) {
    const int64_t g = r * a.n_groups + a.col0 / kBlk;
    a.scales[g] = s;
    a.zeros[g] = z;
    if (a.loss_rows) a.loss_rows[r] += loss;
  }
}

}  // namespace

int gptq_block_launch(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0, int count,
                      int bits, int sym, float* err_t, float* scales, float* zeros, int64_t n_groups,
                      uint8_t* codes, float* loss_rows, cudaStream_t st, float* panel_hi, float* panel_lo,
                      int panel_k0) {
  // per-device attribute; setting it on every call keeps multi-device processes correct
  if (cudaFuncSetAttribute(gptq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (kBlk * kBlk + kBlk) * (int)sizeof(float)) != cudaSuccess)
    return LC_ERR_CUDA;
  BlockArgs a;
  a.W = W;
  a.U = U;
  a.err_t = err_t;
  a.panel_hi = panel_hi;
  a.panel_lo = panel_lo;
  a.panel_k0 = panel_k0;
  a.scales = scales;
  a.zeros = zeros;
  a.codes = codes;
  a.loss_rows = loss_rows;
  a.rows = rows;
  a.cols = cols;
  a.col0 = col0;
  a.n_groups = n_groups;
  a.count = count;
  a.sym = sym ? 1 : 0;
  a.qr = int_qrange(bits, a.sym);
  const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
  gptq_block_kernel<<<grid, kThreads, (kBlk * kBlk + kBlk) * sizeof(float), st>>>(a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace lc

extern "C" LC_API int lc_gptq_block_quant(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0,
                                   int count, int bits, int sym, float* err_out, float* scales,
                                   float* zeros, int64_t n_groups, uint8_t* codes_u8, float* loss_rows,
                                   lc_stream_t stream) {
  if (!W || !U || !err_out || !scales || !zeros) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || col0 < 0 || col0 % 128 != 0 || count < 1 || count > 128) return LC_ERR_ARG;
  if (col0 + count > cols) return LC_ERR_SHAPE;
  if (bits < 2 || bits > 8) return LC_ERR_ARG;
  if (n_groups < (cols + 127) / 128) return LC_ERR_SHAPE;
  return lc::gptq_block_launch(W, U, rows, cols, col0, count, bits, sym, err_out, scales, zeros, n_groups,
                               codes_u8, loss_rows, reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr, 0);
}
