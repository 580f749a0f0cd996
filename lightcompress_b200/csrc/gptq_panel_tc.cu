// Family 3: the GPTQ trailing update on the tensor cores, with two-level (lazy) batching.
//
// The reference updates all columns to the right after every 128-column block
// (W[:, i2:] -= Err1 @ Hinv[i1:i2, i2:], gptq.py:244): K = 128, 32 flop per byte of W traffic.  Here
// the eager update only covers the rest of a 1024-column panel (fp32 FFMA kernel); everything to the
// right of the panel is updated once per panel,
//     W[:, p2:] -= E^T (rows x 1024) * U[p1:p2, p2:],
// a K = 1024 GEMM that runs on tcgen05 with kind::tf32.  The sums are the reference's, associated
// differently.  fp32 accuracy is kept with the three-term split a*b ~ a_hi*b_hi + a_hi*b_lo +
// a_lo*b_hi, where x_hi is what the tensor core sees of an fp32 value (its top 19 bits) and
// x_lo = x - x_hi is stored next to it by the producer (block kernel for E, lc_gptq_split_tf32 for U).
//
// Both operands are MN-major (E is stored k-major, U row-major), like the Hessian kernel: TMA boxes
// of 32 floats x 16 k-rows (128-byte rows; 128B swizzle with 32-byte atoms, the only layout 32-bit
// MN-major operands have), MMA 128x256x8, accumulator in TMEM.
// CTA roles and the bounded-wait / drain discipline are those of hessian_umma.cu.
#include "umma_common.cuh"

namespace lc {
namespace {

using namespace umma;

constexpr int PM = 128, PN = 256;
constexpr int PBK = 16;                       // k rows per pipeline stage
constexpr int PK = 8;                         // tf32 MMA depth
constexpr int PSTAGES = 4;
constexpr int ATOM_F = 32;                    // floats per 128-byte swizzle row
constexpr int P_ATOM_BYTES = ATOM_F * 4 * PBK;   // 2048: one 32-float x 16-row box
constexpr int A_ATOMS = PM / ATOM_F;          // 4
constexpr int B_ATOMS = PN / ATOM_F;          // 8
constexpr int P_STAGE_BYTES = 2 * (A_ATOMS + B_ATOMS) * P_ATOM_BYTES;  // 49152: A_hi, A_lo, B_hi, B_lo
constexpr int P_SMEM_BYTES = PSTAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_TMEM_COLS = 256;
constexpr int kThreads = 192;

// kind::tf32, fp32 accumulate, both operands MN-major, M = 128, N = 256
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) |
                                ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);

struct PanelMaps {
  CUtensorMap e_hi, e_lo, u_hi, u_lo;
};

struct PanelArgs {
  float* W;
  int32_t* status;
  int64_t rows, cols;
  int p1, p2;        // panel columns [p1, p2); updates columns [p2, cols)
  int m_tiles, n_tiles;
};

__global__ void __launch_bounds__(kThreads, 1) gptq_panel_update_kernel(const __grid_constant__ PanelMaps maps, PanelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + PSTAGES * P_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = base + PSTAGES * P_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (PSTAGES + s); };
  const uint32_t accum_full = bar0 + 8u * (2 * PSTAGES);
  const uint32_t accum_empty = bar0 + 8u * (2 * PSTAGES + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(accum_full, 1);
    mbar_init(accum_empty, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)P_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  const int n_tiles_total = a.m_tiles * a.n_tiles;
  const int k_iters = (a.p2 - a.p1) / PBK;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t n = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        const int mt = t % a.m_tiles, nt = t / a.m_tiles;
        const int m0 = mt * PM, n0 = a.p2 + nt * PN;
        for (int k = 0; k < k_iters; ++k, ++n) {
          const int s = n % PSTAGES;
          const uint32_t ph = (n / PSTAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), P_STAGE_BYTES);
          const uint32_t sa = base + s * P_STAGE_BYTES;
          const int krow = k * PBK;
#pragma unroll
          for (int q = 0; q < A_ATOMS; ++q) {
            tma_load_2d(sa + q * P_ATOM_BYTES, &maps.e_hi, m0 + q * ATOM_F, krow, full_bar(s));
            tma_load_2d(sa + (A_ATOMS + q) * P_ATOM_BYTES, &maps.e_lo, m0 + q * ATOM_F, krow, full_bar(s));
          }
#pragma unroll
          for (int q = 0; q < B_ATOMS; ++q) {
            tma_load_2d(sa + (2 * A_ATOMS + q) * P_ATOM_BYTES, &maps.u_hi, n0 + q * ATOM_F, a.p1 + krow, full_bar(s));
            tma_load_2d(sa + (2 * A_ATOMS + B_ATOMS + q) * P_ATOM_BYTES, &maps.u_lo, n0 + q * ATOM_F, a.p1 + krow,
                        full_bar(s));
          }
          issued = n + 1;
        }
      }
      if (*abort_flag) {
        const uint32_t first = issued > PSTAGES ? issued - PSTAGES : 0;
        for (uint32_t i = first; i < issued; ++i) {
          const int s = i % PSTAGES;
          const uint32_t ph = (i / PSTAGES) & 1u;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_test(full_bar(s), ph); ++it) __nanosleep(50);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t n = 0, tiles_done = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        if (!mbar_wait(accum_empty, (tiles_done & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        for (int k = 0; k < k_iters; ++k, ++n) {
          const int s = n % PSTAGES;
          const uint32_t ph = (n / PSTAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = base + s * P_STAGE_BYTES;
          const uint32_t a_hi = sa, a_lo = sa + A_ATOMS * P_ATOM_BYTES;
          const uint32_t b_hi = sa + 2 * A_ATOMS * P_ATOM_BYTES, b_lo = b_hi + B_ATOMS * P_ATOM_BYTES;
#pragma unroll
          for (int kk = 0; kk < PBK / PK; ++kk) {
            // one MMA consumes 8 k-rows = two 4-row swizzle atoms of 512 bytes; atoms along M/N are
            // 2048 bytes apart
            const uint32_t off = kk * 1024;
            const uint64_t dah = make_desc_mn_sw128_32b(a_hi + off, P_ATOM_BYTES, 512);
            const uint64_t dal = make_desc_mn_sw128_32b(a_lo + off, P_ATOM_BYTES, 512);
            const uint64_t dbh = make_desc_mn_sw128_32b(b_hi + off, P_ATOM_BYTES, 512);
            const uint64_t dbl = make_desc_mn_sw128_32b(b_lo + off, P_ATOM_BYTES, 512);
            umma_tf32(tmem_acc, dah, dbh, kIdescTf32, (k > 0 || kk > 0) ? 1u : 0u);
            umma_tf32(tmem_acc, dah, dbl, kIdescTf32, 1u);
            umma_tf32(tmem_acc, dal, dbh, kIdescTf32, 1u);
          }
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(accum_full);
        ++tiles_done;
      }
      if (*abort_flag) {
        umma_commit(accum_full);
        for (uint32_t it = 0; it < kSpinLimit && !mbar_test(accum_full, tiles_done & 1u); ++it) __nanosleep(50);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tiles_done = 0;
    for (int t = blockIdx.x; t < n_tiles_total; t += gridDim.x) {
      const int mt = t % a.m_tiles, nt = t / a.m_tiles;
      if (!mbar_wait(accum_full, tiles_done & 1u, abort_flag) || *abort_flag) break;
      tcgen05_fence_after();
      const int64_t m = (int64_t)mt * PM + q * 32 + lane;
      const int64_t n_base = (int64_t)a.p2 + (int64_t)nt * PN;
#pragma unroll 1
      for (int cc = 0; cc < PN / 32; ++cc) {
        const int64_t n0 = n_base + cc * 32;
        if (n0 >= a.cols) break;
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(cc * 32), v);
        if (m < a.rows) {
          float* row = a.W + m * a.cols + n0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (n0 + j < a.cols) {
              float4 c = *reinterpret_cast<float4*>(row + j);
              c.x -= v[j];
              c.y -= v[j + 1];
              c.z -= v[j + 2];
              c.w -= v[j + 3];
              *reinterpret_cast<float4*>(row + j) = c;
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accum_empty);
      ++tiles_done;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)P_TMEM_COLS)
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)LC_ERR_TIMEOUT);
}

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

int encode_f32_2d(CUtensorMap* m, const float* base, int64_t inner, int64_t outer, int64_t pitch_elems) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  const cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t gstride[1] = {(cuuint64_t)pitch_elems * 4};
  const cuuint32_t box[2] = {ATOM_F, PBK};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LC_ERR_CUDA;
  return LC_OK;
}

int panel_update_launch(float* W, const float* e_hi, const float* e_lo, const float* U, const float* U_lo,
                        int64_t rows, int64_t cols, int p1, int p2, int32_t* status, cudaStream_t st) {
  if (p2 >= cols) return LC_OK;
  PanelMaps maps;
  int rc;
  if ((rc = encode_f32_2d(&maps.e_hi, e_hi, rows, p2 - p1, rows)) != LC_OK) return rc;
  if ((rc = encode_f32_2d(&maps.e_lo, e_lo, rows, p2 - p1, rows)) != LC_OK) return rc;
  if ((rc = encode_f32_2d(&maps.u_hi, U, cols, cols, cols)) != LC_OK) return rc;
  if ((rc = encode_f32_2d(&maps.u_lo, U_lo, cols, cols, cols)) != LC_OK) return rc;
  PanelArgs a;
  a.W = W;
  a.status = status;
  a.rows = rows;
  a.cols = cols;
  a.p1 = p1;
  a.p2 = p2;
  a.m_tiles = (int)((rows + PM - 1) / PM);
  a.n_tiles = (int)((cols - p2 + PN - 1) / PN);
  int dev = 0, sms = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int tiles = a.m_tiles * a.n_tiles;
  LC_CHECK_CUDA(cudaFuncSetAttribute(gptq_panel_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     P_SMEM_BYTES));
  gptq_panel_update_kernel<<<tiles < sms ? tiles : sms, kThreads, P_SMEM_BYTES, st>>>(maps, a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace

int gptq_trail_launch(float* W, const float* err_t, const float* U, int64_t rows, int64_t cols, int64_t col0,
                      int k, int64_t col1, cudaStream_t st, int64_t col_end);
int gptq_block_launch(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0, int count,
                      int bits, int sym, float* err_t, float* scales, float* zeros, int64_t n_groups,
                      uint8_t* codes, float* loss_rows, cudaStream_t st, float* panel_hi, float* panel_lo,
                      int panel_k0);

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

extern "C" LC_API int lc_gptq_weight_transform_tc(float* W, const float* U, const float* U_lo, int64_t rows,
                                                  int64_t cols, int bits, int sym, float* scratch_err,
                                                  float* panel_hi, float* panel_lo, float* scales, float* zeros,
                                                  uint8_t* codes_u8, float* loss_rows, int32_t* status,
                                                  lc_stream_t stream) {
  using namespace lc;
  constexpr int kPanel = 1024;
  if (!W || !U || !U_lo || !scratch_err || !panel_hi || !panel_lo || !scales || !zeros) return LC_ERR_ARG;
  if (rows <= 0 || cols <= 0 || bits < 2 || bits > 8) return LC_ERR_ARG;
  if (cols % 128 != 0 || rows % 4 != 0) return LC_ERR_SHAPE;      // TMA pitch / whole blocks; use the FFMA entry point otherwise
  if (!aligned16(W) || !aligned16(U) || !aligned16(U_lo) || !aligned16(panel_hi) || !aligned16(panel_lo)) return LC_ERR_ALIGN;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_groups = cols / 128;
  if (loss_rows) LC_CHECK_CUDA(cudaMemsetAsync(loss_rows, 0, rows * sizeof(float), st));
  for (int64_t p1 = 0; p1 < cols; p1 += kPanel) {
    const int64_t p2 = (p1 + kPanel < cols) ? p1 + kPanel : cols;
    const bool has_right = p2 < cols;
    for (int64_t i1 = p1; i1 < p2; i1 += 128) {
      int rc = gptq_block_launch(W, U, rows, cols, i1, 128, bits, sym, scratch_err, scales, zeros, n_groups, codes_u8,
                                 loss_rows, st, has_right ? panel_hi : nullptr, has_right ? panel_lo : nullptr,
                                 (int)(i1 - p1));
      if (rc != LC_OK) return rc;
      rc = gptq_trail_launch(W, scratch_err, U, rows, cols, i1, 128, i1 + 128, st, p2);   // rest of the panel only
      if (rc != LC_OK) return rc;
    }
    if (has_right) {
      const int rc = panel_update_launch(W, panel_hi, panel_lo, U, U_lo, rows, cols, (int)p1, (int)p2, status, st);
      if (rc != LC_OK) return rc;
    }
  }
  return LC_OK;
}
