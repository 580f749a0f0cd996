// Family 3: the 128-column in-block step of the GPTQ solver.
//
// Rows of W are independent (they only share the inverse-Hessian factor U) and every row is a
// chain of 128 dependent column steps (quantise column i, spread its error over columns > i), so
// the kernel is bound by the latency of that chain and by how many instructions a row-step costs,
// not by memory.  Two mappings:
//
//  * quad kernel (full 128-column blocks, 16-byte aligned rows): four lanes own one row, eight rows
//    per warp.  Lane `sub` keeps, for each 16-column slot g, columns 16g + 4*sub .. +3 (one float4
//    of W and of the U row).  The quantisation arithmetic of a step, identical for all lanes of a
//    row, is thereby shared by 8 rows per instruction instead of 1, and the error spread costs
//    32 columns per lane.  Slots are retired front to back: after 16 steps the finished slot is
//    stored and the register file shifts down by one slot, so that all register indices stay
//    static without unrolling the 128 steps.
//  * warp kernel (any block width up to 128): one warp per row, lane l keeps columns l, l+32, l+64,
//    l+96.  Used for ragged tails and unaligned tensors.
//
// Both run the same per-element arithmetic in the same order and give bit-identical results.  The
// 128x128 diagonal block of U sits in shared memory; nothing is written to global memory until a
// slot (quad) or the block (warp) is finished.
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
  // static groups (gptq.py:224-227): scales / zeros are INPUT tables (rows x n_groups) and column
  // col0 + i uses group col_group[col0 + i] of its row; NULL = qparams from the block's columns
  const int32_t* col_group;
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
  const bool is_static = a.col_group != nullptr;
  float s = 1.f, z = 0.f;
  if (!is_static) int_qparams<float>(mn, mx, a.qr, a.sym, s, z);
  // error feedback can move a weight a little outside the block's initial range: leave headroom
  const float bound = 16.f * nan_max(fabsf(mx), fabsf(mn));
  const QuantCtx qc = make_quant_ctx(s, z, bound);
  // static groups: every lane prepares the contexts of its own four columns; the column loop fetches
  // them with shuffles that do not depend on the weights (off the sequential chain)
  float ls[4], lz[4], lr[4];
  int lex[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    ls[c] = 1.f, lz[c] = 0.f, lr[c] = 1.f, lex[c] = 0;
    if (is_static && valid[c]) {
      const int64_t g = r * a.n_groups + a.col_group[a.col0 + lane + 32 * c];
      const QuantCtx t = make_quant_ctx(a.scales[g], a.sym ? 0.f : a.zeros[g], bound);
      ls[c] = t.s, lz[c] = t.z, lr[c] = t.r, lex[c] = t.exact ? 1 : 0;
    }
  }

  float loss = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int lim = min(32, a.count - 32 * c);
    for (int il = 0; il < lim; ++il) {
      const int i = 32 * c + il;
      const float wi = __shfl_sync(0xffffffffu, w[c], il);
      const float d = u1[i * kBlk + i], rd = dinv[i];
      QuantCtx qi = qc;
      if (is_static) {
        qi.s = __shfl_sync(0xffffffffu, ls[c], il);
        qi.z = __shfl_sync(0xffffffffu, lz[c], il);
        qi.r = __shfl_sync(0xffffffffu, lr[c], il);
        qi.exact = __shfl_sync(0xffffffffu, lex[c], il) != 0;
      }
      const float q = int_quant_fast<float>(wi, qi, a.qr);   // the same code the IEEE division gives
      const float dq = int_dequant_fast<float>(q, qi);
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
    if (!is_static) {
      const int64_t g = r * a.n_groups + a.col0 / kBlk;
      a.scales[g] = s;
      a.zeros[g] = z;
    }
    if (a.loss_rows) a.loss_rows[r] += loss;
  }
}


// ---- quad kernel -----------------------------------------------------------------------------------
constexpr int kQuadWarps = 4;
constexpr int kQuadRowsPerCta = kQuadWarps * 8;
constexpr int kQuadThreads = kQuadWarps * 32;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gsrc));
}

// clamp(rint(w / s) + z, qmin, qmax) like int_quant_fast<float>, with the rounding done by adding
// and subtracting 1.5 * 2^23 (two FADDs on the dependent chain instead of a conversion-unit op).
// For |q| < 2^22 that is exactly rintf (round-half-even); beyond it the value is saturated by the
// clamp whichever integer comes out, and NaN / inf fall to the IEEE path through the guard.
__device__ __forceinline__ float quad_quant(float w, const QuantCtx& c, QRange qr) {
  const float q0 = __fmul_rn(w, c.r);
  const float e = __fmaf_rn(-q0, c.s, w);
  const float q1 = __fmaf_rn(e, c.r, q0);
  float k = __fsub_rn(__fadd_rn(q1, 12582912.f), 12582912.f);
  if (c.exact || !(fabsf(fabsf(__fsub_rn(q1, k)) - 0.5f) >= 1e-4f)) k = rintf(ieee_div(w, c.s));
  return clampf(__fadd_rn(k, c.z), qr.qmin, qr.qmax);
}

struct QuadRow {
  float w[32];       // slot g (16 columns) of the not yet retired part of the row: w[4g .. 4g+3]
  float loss;
};

// The 16 column steps of slot `t` with NG live slots (the current one and NG-1 to its right), then
// the slot is stored and the register file shifts down by one slot.  All U values of a step are
// fetched before the step's dependent chain starts, so the chain never waits on shared memory.
// ST (static groups): the context of column i comes from the row's table of per-group contexts in
// shared memory (tab: s, z, 1/s per group; 1/s = NaN marks a scale the reciprocal scheme cannot take),
// indexed by the column's group cg[i]; like the U values it is fetched before the dependent chain.
template <int NG, bool ST>
__device__ __forceinline__ void quad_slot(QuadRow& row, const BlockArgs& a, const float* u1, const float* dinv,
                                          const QuantCtx& qc, int t, int sub, int quad_base, bool live, int64_t r,
                                          float* wrow, const float* tab, const int* cg) {
  float er[4] = {0.f, 0.f, 0.f, 0.f};
  int cd[4] = {0, 0, 0, 0};
  float (&w)[32] = row.w;
#pragma unroll
  for (int st = 0; st < 16; ++st) {
    const int owner = st >> 2, k = st & 3;
    const int i = 16 * t + st;
    const float* urow = u1 + i * kBlk;
    const float d = urow[i], rd = dinv[i];
    float4 u[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) u[g] = *reinterpret_cast<const float4*>(urow + 16 * (t + g) + 4 * sub);

    QuantCtx qi = qc;
    if constexpr (ST) {
      const float* e = tab + 3 * cg[i];
      qi.s = e[0], qi.z = e[1], qi.r = e[2];
      qi.exact = !(qi.r == qi.r);
    }
    const float wi = __shfl_sync(0xffffffffu, w[k], quad_base | owner);
    const float q = quad_quant(wi, qi, a.qr);
    const float dq = int_dequant_fast<float>(q, qi);
    const float diff = __fsub_rn(wi, dq);
    const float e0 = __fmul_rn(diff, rd);
    const float err = __fmaf_rn(__fmaf_rn(-e0, d, diff), rd, e0);
    row.loss = fmaf(0.5f * err, err, row.loss);
    if (sub == owner) {
      er[k] = err;
      cd[k] = code_to_int(q) - (int)a.qr.qmin;
    }
    // current slot: only the columns behind column i move
    {
      const float uu[4] = {u[0].x, u[0].y, u[0].z, u[0].w};
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) {
        const float upd = __fsub_rn(w[k2], __fmul_rn(err, uu[k2]));
        if (sub > owner || (sub == owner && k2 > k)) w[k2] = upd;
      }
    }
#pragma unroll
    for (int g = 1; g < NG; ++g) {
      w[4 * g + 0] = __fsub_rn(w[4 * g + 0], __fmul_rn(err, u[g].x));
      w[4 * g + 1] = __fsub_rn(w[4 * g + 1], __fmul_rn(err, u[g].y));
      w[4 * g + 2] = __fsub_rn(w[4 * g + 2], __fmul_rn(err, u[g].z));
      w[4 * g + 3] = __fsub_rn(w[4 * g + 3], __fmul_rn(err, u[g].w));
    }
  }
  if (live) {
    const int j0 = 16 * t + 4 * sub;
    *reinterpret_cast<float4*>(wrow + j0) = make_float4(w[0], w[1], w[2], w[3]);
    if (a.codes)
      *reinterpret_cast<uchar4*>(a.codes + r * a.cols + a.col0 + j0) =
          make_uchar4((unsigned char)cd[0], (unsigned char)cd[1], (unsigned char)cd[2], (unsigned char)cd[3]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      a.err_t[(int64_t)(j0 + k) * a.rows + r] = er[k];
      if (a.panel_hi) {
        const float hi = __uint_as_float(__float_as_uint(er[k]) & 0xffffe000u);
        a.panel_hi[(int64_t)(a.panel_k0 + j0 + k) * a.rows + r] = er[k];
        a.panel_lo[(int64_t)(a.panel_k0 + j0 + k) * a.rows + r] = er[k] - hi;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 28; ++k) w[k] = w[k + 4];
}

// odd row pitch of the per-row context tables: the eight rows of a warp fall into eight different banks
__host__ __device__ inline int quad_tab_pitch(int64_t n_groups) { return (int)(3 * n_groups) | 1; }

template <bool ST>
__global__ void __launch_bounds__(kQuadThreads) gptq_block_quad_kernel(BlockArgs a) {
  extern __shared__ float u1[];  // [128][128]; row i is only filled from column (i & ~3) on
  float* dinv = u1 + kBlk * kBlk;
  int* cg = reinterpret_cast<int*>(dinv + kBlk);       // ST: [128] group of each column of the block
  float* tabs = reinterpret_cast<float*>(cg + kBlk);    // ST: [32 rows][pitch]
  const int pitch = quad_tab_pitch(a.n_groups);
  if constexpr (ST) {
    if (threadIdx.x < kBlk) cg[threadIdx.x] = a.col_group[a.col0 + threadIdx.x];
    const int64_t row0 = (int64_t)blockIdx.x * kQuadRowsPerCta;
    for (int idx = threadIdx.x; idx < kQuadRowsPerCta * (int)a.n_groups; idx += kQuadThreads) {
      const int rl = idx / (int)a.n_groups, g = idx - rl * (int)a.n_groups;
      const int64_t rr = (row0 + rl < a.rows) ? row0 + rl : a.rows - 1;
      const float sv = a.scales[rr * a.n_groups + g];
      float* e = tabs + rl * pitch + 3 * g;
      e[0] = sv;
      e[1] = a.sym ? 0.f : a.zeros[rr * a.n_groups + g];
      e[2] = (sv > 1e-30f && sv < 1e30f) ? __frcp_rn(sv) : __int_as_float(0x7fc00000);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 3;

  // U block -> shared memory, 16 bytes per copy, upper triangle only (all copies in flight at once)
  {
    const float* ublk = a.U + a.col0 * a.cols + a.col0;
    for (int idx = threadIdx.x; idx < kBlk * (kBlk / 4); idx += kQuadThreads) {
      const int i = idx >> 5, j4 = (idx & 31) << 2;
      if (j4 + 3 >= i) cp_async16(&u1[i * kBlk + j4], ublk + (int64_t)i * a.cols + j4);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x < kBlk) dinv[threadIdx.x] = __frcp_rn(u1[threadIdx.x * kBlk + threadIdx.x]);
  __syncthreads();

  const int64_t r_raw = (int64_t)blockIdx.x * kQuadRowsPerCta + warp * 8 + (lane >> 2);
  const bool live = r_raw < a.rows;
  const int64_t r = live ? r_raw : a.rows - 1;   // idle lanes shadow the last row and store nothing

  float* wrow = a.W + r * a.cols + a.col0;
  QuadRow row;
  float (&w)[32] = row.w;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 v = *reinterpret_cast<const float4*>(wrow + 16 * g + 4 * sub);
    w[4 * g + 0] = v.x, w[4 * g + 1] = v.y, w[4 * g + 2] = v.z, w[4 * g + 3] = v.w;
  }
  float mx = w[0], mn = w[0];
#pragma unroll
  for (int k = 1; k < 32; ++k) {
    mx = nan_max(mx, w[k]);
    mn = nan_min(mn, w[k]);
  }
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = nan_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  float s = 1.f, z = 0.f;
  if constexpr (!ST) int_qparams<float>(mn, mx, a.qr, a.sym, s, z);
  const QuantCtx qc = make_quant_ctx(s, z, 16.f * nan_max(fabsf(mx), fabsf(mn)));
  row.loss = 0.f;
  const int quad_base = lane & ~3;
  const float* tab = tabs + (warp * 8 + (lane >> 2)) * pitch;

  // live slots shrink as slots retire; four code copies (8, 6, 4, 2 live slots), two slots each
#pragma unroll 1
  for (int t = 0; t < 2; ++t) quad_slot<8, ST>(row, a, u1, dinv, qc, t, sub, quad_base, live, r, wrow, tab, cg);
#pragma unroll 1
  for (int t = 2; t < 4; ++t) quad_slot<6, ST>(row, a, u1, dinv, qc, t, sub, quad_base, live, r, wrow, tab, cg);
#pragma unroll 1
  for (int t = 4; t < 6; ++t) quad_slot<4, ST>(row, a, u1, dinv, qc, t, sub, quad_base, live, r, wrow, tab, cg);
#pragma unroll 1
  for (int t = 6; t < 8; ++t) quad_slot<2, ST>(row, a, u1, dinv, qc, t, sub, quad_base, live, r, wrow, tab, cg);

  if (live && sub == 0) {
    if constexpr (!ST) {
      const int64_t g = r * a.n_groups + a.col0 / kBlk;
      a.scales[g] = s;
      a.zeros[g] = z;
    }
    if (a.loss_rows) a.loss_rows[r] += row.loss;
  }
}

}  // namespace

int gptq_block_launch(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0, int count,
                      int bits, int sym, float* err_t, float* scales, float* zeros, int64_t n_groups,
                      uint8_t* codes, float* loss_rows, cudaStream_t st, float* panel_hi, float* panel_lo,
                      int panel_k0, const int32_t* col_group) {
  constexpr int kSmem = (kBlk * kBlk + kBlk) * (int)sizeof(float);
  // per-device attribute; setting it on every call keeps multi-device processes correct
  if (cudaFuncSetAttribute(gptq_block_quad_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
      cudaSuccess)
    return LC_ERR_CUDA;
  // static groups: plus the block's column groups and 32 per-row context tables
  const int64_t smem_static = kSmem + kBlk * (int)sizeof(int) +
                              (int64_t)kQuadRowsPerCta * quad_tab_pitch(n_groups) * (int)sizeof(float);
  const bool static_fits = smem_static <= 200 * 1024;
  if (col_group && static_fits &&
      cudaFuncSetAttribute(gptq_block_quad_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem_static) != cudaSuccess)
    return LC_ERR_CUDA;
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
  a.col_group = col_group;
  const bool quad = (!col_group || static_fits) && count == kBlk && cols % 4 == 0 && aligned16(W) && aligned16(U) &&
                    (!codes || (reinterpret_cast<uintptr_t>(codes) & 3u) == 0);
  if (quad) {
    const unsigned grid = (unsigned)((rows + kQuadRowsPerCta - 1) / kQuadRowsPerCta);
    if (col_group) gptq_block_quad_kernel<true><<<grid, kQuadThreads, (size_t)smem_static, st>>>(a);
    else gptq_block_quad_kernel<false><<<grid, kQuadThreads, kSmem, st>>>(a);
  } else {
    const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
    gptq_block_kernel<<<grid, kThreads, kSmem, st>>>(a);
  }
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
                               codes_u8, loss_rows, reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr, 0,
                               nullptr);
}
