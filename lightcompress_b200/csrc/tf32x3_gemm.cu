// fp32-accurate GEMM on the tensor cores: C = beta * C + sign * A^T B with tcgen05 kind::tf32 and the
// three-term split a*b ~ a_hi*b_hi + a_hi*b_lo + a_lo*b_hi, where x_hi is what the tensor core sees
// of an fp32 value (its top 19 bits) and x_lo = x - x_hi is stored by the producer of x.
//
// Used by the GPTQ solver for the per-panel trailing update of W and for every large product of the
// Hessian factorisation (gptq_factor.cu).  Both operands are "k-row" matrices, A [K][M] and B [K][N]
// with the M / N index contiguous (MN-major for the MMA), which is how the solver's data lie in
// memory: E^T, rows of U, row panels of the Cholesky factor.  TMA boxes of 32 floats x 16 k-rows
// (128-byte rows, 128B swizzle with 32-byte atoms -- the only layout 32-bit MN-major operands have),
// MMA 128x256x8, two 256-column accumulators in TMEM so that the epilogue of one tile overlaps the
// MMAs of the next.  Persistent CTAs; warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 =
// epilogue.  Triangular operands shorten a tile's k range instead of multiplying zeros.
// Every wait is bounded; on expiry the CTA raises its abort flag, drains its copies in flight, frees
// its tensor memory and reports LC_ERR_TIMEOUT through the caller's status word.
#include "umma_common.cuh"
#include "tf32x3_gemm.cuh"

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
constexpr int P_TMEM_COLS = 512;              // two accumulators of 256 columns
constexpr int kThreads = 192;

// kind::tf32, fp32 accumulate, both operands MN-major, M = 128, N = 256
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) |
                                ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);

struct GemmMaps {
  CUtensorMap a_hi, a_lo, b_hi, b_lo;
};

struct GemmArgs {
  float* C;
  int32_t* status;
  int64_t ldc;
  int a_k0, a_m0, b_k0, b_n0;   // origins of the operand sub-matrices inside their tensor maps
  int M, N, K;
  int m_tiles, n_tiles;
  int beta;
  float sign;
  int flags;
  int use3d;   // operand tiles fetched by one 3-D copy each instead of one 2-D copy per 32-float atom
  int b_tri_shift;
};

struct TileWork {
  int m0, n0, k0, k1;
  bool skip;
};

__device__ __forceinline__ TileWork tile_work(const GemmArgs& a, int t) {
  TileWork w;
  w.m0 = (t % a.m_tiles) * PM;
  w.n0 = (t / a.m_tiles) * PN;
  w.k0 = (a.flags & kGemmBLower) ? min(a.K, ((w.n0 + a.b_tri_shift) / PBK) * PBK) : 0;
  w.k1 = (a.flags & kGemmAUpper) ? min(a.K, w.m0 + PM) : a.K;
  w.skip = (a.flags & kGemmUpperOnly) && (w.n0 + PN <= w.m0);
  return w;
}

__global__ void __launch_bounds__(kThreads, 1) tf32x3_gemm_kernel(const __grid_constant__ GemmMaps maps, GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + PSTAGES * P_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = base + PSTAGES * P_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (PSTAGES + s); };
  auto accum_full = [&](int b) { return bar0 + 8u * (2 * PSTAGES + b); };
  auto accum_empty = [&](int b) { return bar0 + 8u * (2 * PSTAGES + 2 + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accum_full(b), 1);
      mbar_init(accum_empty(b), 4);
    }
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
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles_total = a.m_tiles * a.n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t n = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        const TileWork w = tile_work(a, t);
        if (w.skip) continue;
        for (int krow = w.k0; krow < w.k1; krow += PBK, ++n) {
          const int s = n % PSTAGES;
          const uint32_t ph = (n / PSTAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), P_STAGE_BYTES);
          const uint32_t sa = base + s * P_STAGE_BYTES;
          if (a.use3d) {
            // atoms land 2048 bytes apart, exactly like the per-atom copies below
            tma_load_3d(sa, &maps.a_hi, 0, a.a_k0 + krow, (a.a_m0 + w.m0) / ATOM_F, full_bar(s));
            tma_load_3d(sa + A_ATOMS * P_ATOM_BYTES, &maps.a_lo, 0, a.a_k0 + krow, (a.a_m0 + w.m0) / ATOM_F,
                        full_bar(s));
            tma_load_3d(sa + 2 * A_ATOMS * P_ATOM_BYTES, &maps.b_hi, 0, a.b_k0 + krow, (a.b_n0 + w.n0) / ATOM_F,
                        full_bar(s));
            tma_load_3d(sa + (2 * A_ATOMS + B_ATOMS) * P_ATOM_BYTES, &maps.b_lo, 0, a.b_k0 + krow,
                        (a.b_n0 + w.n0) / ATOM_F, full_bar(s));
            issued = n + 1;
            continue;
          }
#pragma unroll
          for (int q = 0; q < A_ATOMS; ++q) {
            tma_load_2d(sa + q * P_ATOM_BYTES, &maps.a_hi, a.a_m0 + w.m0 + q * ATOM_F, a.a_k0 + krow, full_bar(s));
            tma_load_2d(sa + (A_ATOMS + q) * P_ATOM_BYTES, &maps.a_lo, a.a_m0 + w.m0 + q * ATOM_F, a.a_k0 + krow,
                        full_bar(s));
          }
#pragma unroll
          for (int q = 0; q < B_ATOMS; ++q) {
            tma_load_2d(sa + (2 * A_ATOMS + q) * P_ATOM_BYTES, &maps.b_hi, a.b_n0 + w.n0 + q * ATOM_F, a.b_k0 + krow,
                        full_bar(s));
            tma_load_2d(sa + (2 * A_ATOMS + B_ATOMS + q) * P_ATOM_BYTES, &maps.b_lo, a.b_n0 + w.n0 + q * ATOM_F,
                        a.b_k0 + krow, full_bar(s));
          }
          issued = n + 1;
        }
      }
      if (*abort_flag) {
        // let the copies still in flight land before the CTA's shared memory is released
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
        const TileWork w = tile_work(a, t);
        if (w.skip) continue;
        const uint32_t buf = tiles_done & 1u;
        if (!mbar_wait(accum_empty(buf), ((tiles_done >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * PN;
        for (int krow = w.k0; krow < w.k1; krow += PBK, ++n) {
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
            umma_tf32(tmem_acc, dah, dbh, kIdescTf32, (krow > w.k0 || kk > 0) ? 1u : 0u);
            umma_tf32(tmem_acc, dah, dbl, kIdescTf32, 1u);
            umma_tf32(tmem_acc, dal, dbh, kIdescTf32, 1u);
          }
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(accum_full(buf));
        ++tiles_done;
      }
      if (*abort_flag) {
        // the MMAs already issued must retire before the tensor memory is freed
        const uint32_t buf = tiles_done & 1u;
        umma_commit(accum_full(buf));
        for (uint32_t it = 0; it < kSpinLimit && !mbar_test(accum_full(buf), (tiles_done >> 1) & 1u); ++it)
          __nanosleep(50);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tiles_done = 0;
    for (int t = blockIdx.x; t < n_tiles_total; t += gridDim.x) {
      const TileWork w = tile_work(a, t);
      if (w.skip) continue;
      const uint32_t buf = tiles_done & 1u;
      if (!mbar_wait(accum_full(buf), (tiles_done >> 1) & 1u, abort_flag) || *abort_flag) break;
      tcgen05_fence_after();
      const uint32_t tmem_acc = tmem_base + buf * PN;
      const int m = w.m0 + q * 32 + lane;
#pragma unroll 1
      for (int cc = 0; cc < PN / 32; ++cc) {
        const int n0 = w.n0 + cc * 32;
        if (n0 >= a.N) break;
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(cc * 32), v);
        if (m < a.M) {
          float* row = a.C + (int64_t)m * a.ldc + n0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (n0 + j < a.N) {
              float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
              if (a.beta) c = *reinterpret_cast<float4*>(row + j);
              c.x = fmaf(a.sign, v[j], c.x);
              c.y = fmaf(a.sign, v[j + 1], c.y);
              c.z = fmaf(a.sign, v[j + 2], c.z);
              c.w = fmaf(a.sign, v[j + 3], c.w);
              *reinterpret_cast<float4*>(row + j) = c;
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accum_empty(buf));
      ++tiles_done;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P_TMEM_COLS)
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)LC_ERR_TIMEOUT);
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

// 3-D view of a k-row matrix: (32 floats, k rows, atoms of 32 floats along M / N); a box of `atoms`
// atoms x 16 rows is one operand tile of a pipeline stage
int encode_f32_3d(CUtensorMap* m, const float* base, int64_t mn_extent, int64_t k_extent, int64_t pitch_elems,
                  int atoms) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  const cuuint64_t gdim[3] = {(cuuint64_t)ATOM_F, (cuuint64_t)k_extent, (cuuint64_t)(mn_extent / ATOM_F)};
  const cuuint64_t gstride[2] = {(cuuint64_t)pitch_elems * 4, (cuuint64_t)ATOM_F * 4};
  const cuuint32_t box[3] = {ATOM_F, PBK, (cuuint32_t)atoms};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LC_ERR_CUDA;
  return LC_OK;
}

// SM count and the kernel's shared-memory attribute, once per device
int device_setup(int* sms_out) {
  static int sms_of[64] = {0};
  int dev = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return LC_ERR_ARG;
  if (sms_of[dev] == 0) {
    int sms = 0;
    LC_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    LC_CHECK_CUDA(cudaFuncSetAttribute(tf32x3_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
    sms_of[dev] = sms;
  }
  *sms_out = sms_of[dev];
  return LC_OK;
}

}  // namespace

int gemm_mat_init(GemmMat* m, const float* hi, const float* lo, int64_t k_extent, int64_t mn_extent, int64_t ld) {
  if (k_extent <= 0 || mn_extent <= 0 || ld % 4 != 0 || ld < mn_extent) return LC_ERR_SHAPE;
  if (!aligned16(hi) || !aligned16(lo)) return LC_ERR_ALIGN;
  int rc;
  if ((rc = encode_f32_2d(&m->map_hi, hi, mn_extent, k_extent, ld)) != LC_OK) return rc;
  if ((rc = encode_f32_2d(&m->map_lo, lo, mn_extent, k_extent, ld)) != LC_OK) return rc;
  m->k_extent = k_extent;
  m->mn_extent = mn_extent;
  m->has3 = false;
  if (mn_extent % ATOM_F == 0 && encode_f32_3d(&m->map3a_hi, hi, mn_extent, k_extent, ld, A_ATOMS) == LC_OK &&
      encode_f32_3d(&m->map3a_lo, lo, mn_extent, k_extent, ld, A_ATOMS) == LC_OK &&
      encode_f32_3d(&m->map3b_hi, hi, mn_extent, k_extent, ld, B_ATOMS) == LC_OK &&
      encode_f32_3d(&m->map3b_lo, lo, mn_extent, k_extent, ld, B_ATOMS) == LC_OK)
    m->has3 = true;
  return LC_OK;
}

int tf32x3_gemm_launch(float* C, int64_t ldc, const GemmMat& A, int64_t a_k0, int64_t a_m0, const GemmMat& B,
                       int64_t b_k0, int64_t b_n0, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                       int32_t* status, cudaStream_t st, int64_t b_tri_shift) {
  if (M <= 0 || N <= 0 || K <= 0) return LC_OK;
  if (K % PBK != 0 || M % 4 != 0 || N % 4 != 0 || ldc % 4 != 0 || a_m0 % 4 != 0 || b_n0 % 4 != 0) return LC_ERR_SHAPE;
  if (b_tri_shift < 0 || ((flags & kGemmBLower) && b_tri_shift + N > K)) return LC_ERR_SHAPE;
  if (a_k0 < 0 || a_m0 < 0 || b_k0 < 0 || b_n0 < 0 || a_k0 + K > A.k_extent || a_m0 + M > A.mn_extent ||
      b_k0 + K > B.k_extent || b_n0 + N > B.mn_extent)
    return LC_ERR_SHAPE;
  if (A.k_extent > (1 << 30) || A.mn_extent > (1 << 30) || B.k_extent > (1 << 30) || B.mn_extent > (1 << 30))
    return LC_ERR_SHAPE;
  if (!aligned16(C)) return LC_ERR_ALIGN;
  GemmMaps maps;
  GemmArgs a;
  a.use3d = (A.has3 && B.has3 && a_m0 % ATOM_F == 0 && b_n0 % ATOM_F == 0) ? 1 : 0;
  maps.a_hi = a.use3d ? A.map3a_hi : A.map_hi;
  maps.a_lo = a.use3d ? A.map3a_lo : A.map_lo;
  maps.b_hi = a.use3d ? B.map3b_hi : B.map_hi;
  maps.b_lo = a.use3d ? B.map3b_lo : B.map_lo;
  a.C = C;
  a.status = status;
  a.ldc = ldc;
  a.a_k0 = (int)a_k0;
  a.a_m0 = (int)a_m0;
  a.b_k0 = (int)b_k0;
  a.b_n0 = (int)b_n0;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  a.m_tiles = (int)((M + PM - 1) / PM);
  a.n_tiles = (int)((N + PN - 1) / PN);
  a.beta = beta ? 1 : 0;
  a.sign = sign;
  a.flags = flags;
  a.b_tri_shift = (int)b_tri_shift;
  int sms = 0, rc;
  if ((rc = device_setup(&sms)) != LC_OK) return rc;
  const int tiles = a.m_tiles * a.n_tiles;
  tf32x3_gemm_kernel<<<tiles < sms ? tiles : sms, kThreads, P_SMEM_BYTES, st>>>(maps, a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

int tf32x3_gemm_tn(float* C, int64_t ldc, const float* A_hi, const float* A_lo, int64_t lda, const float* B_hi,
                   const float* B_lo, int64_t ldb, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                   int32_t* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return LC_OK;
  GemmMat A, B;
  int rc;
  if ((rc = gemm_mat_init(&A, A_hi, A_lo, K, M, lda)) != LC_OK) return rc;
  if ((rc = gemm_mat_init(&B, B_hi, B_lo, K, N, ldb)) != LC_OK) return rc;
  return tf32x3_gemm_launch(C, ldc, A, 0, 0, B, 0, 0, M, N, K, beta, sign, flags, status, st);
}

}  // namespace lc

extern "C" LC_API int lc_tf32x3_gemm_tn(float* C, int64_t ldc, const float* A_hi, const float* A_lo, int64_t lda,
                                        const float* B_hi, const float* B_lo, int64_t ldb, int64_t M, int64_t N,
                                        int64_t K, int beta, float sign, int flags, int32_t* status,
                                        lc_stream_t stream) {
  if (!C || !A_hi || !A_lo || !B_hi || !B_lo) return LC_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || (sign != 1.f && sign != -1.f) || (flags & ~7)) return LC_ERR_ARG;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  return lc::tf32x3_gemm_tn(C, ldc, A_hi, A_lo, lda, B_hi, B_lo, ldb, M, N, K, beta, sign, flags, status,
                            reinterpret_cast<cudaStream_t>(stream));
}
