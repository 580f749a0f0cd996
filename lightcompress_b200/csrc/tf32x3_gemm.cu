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
constexpr int P_STG_STRIDE = 36;                                   // floats per staged row of the epilogue
constexpr int P_STG_BYTES_PER_WARP = 32 * P_STG_STRIDE * 4;        // 4608
constexpr int P_SMEM_BYTES = PSTAGES * P_STAGE_BYTES + 1024 + 256 + 4 * P_STG_BYTES_PER_WARP;
constexpr int P_TMEM_COLS = 512;              // two accumulators of 256 columns
constexpr int kThreads = 192;

// kind::tf32, fp32 accumulate, both operands MN-major, M = 128, N = 256
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) |
                                ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);

struct GemmMaps {
  CUtensorMap a_hi, a_lo, b_hi, b_lo;
};

// One product of a batch: all problems of a launch share the operand matrices (tensor maps), the pitch
// of C, beta, sign and flags, and differ in their sub-matrix origins and sizes.
struct GemmProblem {
  float* C;
  int a_k0, a_m0, b_k0, b_n0;   // origins of the operand sub-matrices inside their tensor maps
  int M, N, K;
  int b_tri_shift;
  int m_tiles;
  int tile_end;                 // running tile count up to and including this problem
};

struct GemmArgs {
  int32_t* status;
  int64_t ldc;
  int n_problems;
  int total_tiles;
  int beta;
  float sign;
  int flags;
  int use3d;   // operand tiles fetched by one 3-D copy each instead of one 2-D copy per 32-float atom
  GemmProblem p[kGemmMaxBatch];
};

struct TileWork {
  int pi;          // problem index
  int m0, n0, k0, k1;
  bool skip;
};

__device__ __forceinline__ TileWork tile_work(const GemmArgs& a, int t) {
  TileWork w;
  int pi = 0;
  while (pi + 1 < a.n_problems && t >= a.p[pi].tile_end) ++pi;
  const GemmProblem& pr = a.p[pi];
  const int local = t - (pi ? a.p[pi - 1].tile_end : 0);
  w.pi = pi;
  w.m0 = (local % pr.m_tiles) * PM;
  w.n0 = (local / pr.m_tiles) * PN;
  w.k0 = (a.flags & kGemmBLower) ? min(pr.K, ((w.n0 + pr.b_tri_shift) / PBK) * PBK) : 0;
  w.k1 = (a.flags & kGemmAUpper) ? min(pr.K, w.m0 + PM) : pr.K;
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
  float* staging = reinterpret_cast<float*>(gen_base + PSTAGES * P_STAGE_BYTES + 256);
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
  const int n_tiles_total = a.total_tiles;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t n = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        const TileWork w = tile_work(a, t);
        if (w.skip) continue;
        const int a_k0 = a.p[w.pi].a_k0, a_m0 = a.p[w.pi].a_m0, b_k0 = a.p[w.pi].b_k0, b_n0 = a.p[w.pi].b_n0;
        for (int krow = w.k0; krow < w.k1; krow += PBK, ++n) {
          const int s = n % PSTAGES;
          const uint32_t ph = (n / PSTAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), P_STAGE_BYTES);
          const uint32_t sa = base + s * P_STAGE_BYTES;
          if (a.use3d) {
            // atoms land 2048 bytes apart, exactly like the per-atom copies below
            tma_load_3d(sa, &maps.a_hi, 0, a_k0 + krow, (a_m0 + w.m0) / ATOM_F, full_bar(s));
            tma_load_3d(sa + A_ATOMS * P_ATOM_BYTES, &maps.a_lo, 0, a_k0 + krow, (a_m0 + w.m0) / ATOM_F,
                        full_bar(s));
            tma_load_3d(sa + 2 * A_ATOMS * P_ATOM_BYTES, &maps.b_hi, 0, b_k0 + krow, (b_n0 + w.n0) / ATOM_F,
                        full_bar(s));
            tma_load_3d(sa + (2 * A_ATOMS + B_ATOMS) * P_ATOM_BYTES, &maps.b_lo, 0, b_k0 + krow,
                        (b_n0 + w.n0) / ATOM_F, full_bar(s));
            issued = n + 1;
            continue;
          }
#pragma unroll
          for (int q = 0; q < A_ATOMS; ++q) {
            tma_load_2d(sa + q * P_ATOM_BYTES, &maps.a_hi, a_m0 + w.m0 + q * ATOM_F, a_k0 + krow, full_bar(s));
            tma_load_2d(sa + (A_ATOMS + q) * P_ATOM_BYTES, &maps.a_lo, a_m0 + w.m0 + q * ATOM_F, a_k0 + krow,
                        full_bar(s));
          }
#pragma unroll
          for (int q = 0; q < B_ATOMS; ++q) {
            tma_load_2d(sa + (2 * A_ATOMS + q) * P_ATOM_BYTES, &maps.b_hi, b_n0 + w.n0 + q * ATOM_F, b_k0 + krow,
                        full_bar(s));
            tma_load_2d(sa + (2 * A_ATOMS + B_ATOMS + q) * P_ATOM_BYTES, &maps.b_lo, b_n0 + w.n0 + q * ATOM_F,
                        b_k0 + krow, full_bar(s));
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
      const int pM = a.p[w.pi].M, pN = a.p[w.pi].N;
      float* const pC = a.p[w.pi].C;
#pragma unroll 1
      for (int cc = 0; cc < PN / 32; ++cc) {
        const int n0 = w.n0 + cc * 32;
        if (n0 >= pN) break;
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(cc * 32), v);
        // A lane holds one row of the 32 x 32 chunk; through the warp's staging tile eight lanes cover 128
        // contiguous bytes of a row of C, so the read-modify-write moves whole sectors
        float* stg = staging + q * (P_STG_BYTES_PER_WARP / 4);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(&stg[lane * P_STG_STRIDE + j]) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        __syncwarp();
        const int nc = n0 + 4 * (lane & 7);
        const int mr0 = w.m0 + q * 32 + (lane >> 3);
        float4 cv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (a.beta && mr0 + 4 * i < pM && nc < pN)
            cv[i] = *reinterpret_cast<const float4*>(pC + (int64_t)(mr0 + 4 * i) * a.ldc + nc);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (mr0 + 4 * i < pM && nc < pN) {
            const float4 t = *reinterpret_cast<const float4*>(&stg[(4 * i + (lane >> 3)) * P_STG_STRIDE + 4 * (lane & 7)]);
            float4 c = cv[i];
            c.x = fmaf(a.sign, t.x, c.x);
            c.y = fmaf(a.sign, t.y, c.y);
            c.z = fmaf(a.sign, t.z, c.z);
            c.w = fmaf(a.sign, t.w, c.w);
            *reinterpret_cast<float4*>(pC + (int64_t)(mr0 + 4 * i) * a.ldc + nc) = c;
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

int tf32x3_gemm_batched(const GemmMat& A, const GemmMat& B, int64_t ldc, const GemmItem* items, int count, int beta,
                        float sign, int flags, int32_t* status, cudaStream_t st) {
  if (count <= 0) return LC_OK;
  if (ldc % 4 != 0) return LC_ERR_SHAPE;
  if (A.k_extent > (1 << 30) || A.mn_extent > (1 << 30) || B.k_extent > (1 << 30) || B.mn_extent > (1 << 30))
    return LC_ERR_SHAPE;
  int sms = 0, rc;
  if ((rc = device_setup(&sms)) != LC_OK) return rc;
  for (int first = 0; first < count; first += kGemmMaxBatch) {
    const int nb = count - first < kGemmMaxBatch ? count - first : kGemmMaxBatch;
    GemmMaps maps;
    GemmArgs a;
    bool all3 = A.has3 && B.has3;
    int tiles = 0, np = 0;
    for (int i = 0; i < nb; ++i) {
      const GemmItem& it = items[first + i];
      if (it.M <= 0 || it.N <= 0 || it.K <= 0) continue;
      if (it.K % PBK != 0 || it.M % 4 != 0 || it.N % 4 != 0 || it.a_m0 % 4 != 0 || it.b_n0 % 4 != 0) return LC_ERR_SHAPE;
      if (it.a_k0 < 0 || it.a_m0 < 0 || it.b_k0 < 0 || it.b_n0 < 0 || it.a_k0 + it.K > A.k_extent ||
          it.a_m0 + it.M > A.mn_extent || it.b_k0 + it.K > B.k_extent || it.b_n0 + it.N > B.mn_extent)
        return LC_ERR_SHAPE;
      if (it.b_tri_shift < 0 || ((flags & kGemmBLower) && it.b_tri_shift + it.N > it.K)) return LC_ERR_SHAPE;
      if (!aligned16(it.C)) return LC_ERR_ALIGN;
      all3 = all3 && it.a_m0 % ATOM_F == 0 && it.b_n0 % ATOM_F == 0;
      GemmProblem& pr = a.p[np++];
      pr.C = it.C;
      pr.a_k0 = (int)it.a_k0, pr.a_m0 = (int)it.a_m0, pr.b_k0 = (int)it.b_k0, pr.b_n0 = (int)it.b_n0;
      pr.M = (int)it.M, pr.N = (int)it.N, pr.K = (int)it.K;
      pr.b_tri_shift = (int)it.b_tri_shift;
      pr.m_tiles = (int)((it.M + PM - 1) / PM);
      tiles += pr.m_tiles * (int)((it.N + PN - 1) / PN);
      pr.tile_end = tiles;
    }
    if (np == 0) continue;
    a.use3d = all3 ? 1 : 0;
    maps.a_hi = all3 ? A.map3a_hi : A.map_hi;
    maps.a_lo = all3 ? A.map3a_lo : A.map_lo;
    maps.b_hi = all3 ? B.map3b_hi : B.map_hi;
    maps.b_lo = all3 ? B.map3b_lo : B.map_lo;
    a.status = status;
    a.ldc = ldc;
    a.n_problems = np;
    a.total_tiles = tiles;
    a.beta = beta ? 1 : 0;
    a.sign = sign;
    a.flags = flags;
    tf32x3_gemm_kernel<<<tiles < sms ? tiles : sms, kThreads, P_SMEM_BYTES, st>>>(maps, a);
    LC_LAUNCH_CHECK();
  }
  return LC_OK;
}

int tf32x3_gemm_launch(float* C, int64_t ldc, const GemmMat& A, int64_t a_k0, int64_t a_m0, const GemmMat& B,
                       int64_t b_k0, int64_t b_n0, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                       int32_t* status, cudaStream_t st, int64_t b_tri_shift) {
  GemmItem it;
  it.C = C;
  it.a_k0 = a_k0, it.a_m0 = a_m0, it.b_k0 = b_k0, it.b_n0 = b_n0;
  it.M = M, it.N = N, it.K = K;
  it.b_tri_shift = b_tri_shift;
  return tf32x3_gemm_batched(A, B, ldc, &it, 1, beta, sign, flags, status, st);
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
