// Family 2: Hessian accumulation  H <- beta*H + alpha * sum_s X_s^T X_s  on the sm_100a tensor cores.
//
// Each X_s is (tokens x cols) bf16 row-major, so for D[m][n] = sum_t X[t][m] X[t][n] both MMA
// operands are "MN-major": the contraction index (tokens) is the strided one.  TMA copies
// 64-channel x 32-token boxes (128-byte rows, 128B swizzle) into shared memory and tcgen05.mma
// (128x256x16, bf16 in, fp32 accumulate) consumes them through MN-major shared-memory descriptors.
//
// Work unit: a 256x256 "super-tile" of H on or above the diagonal.  Its two 128x256 halves share
// the B operand and live in the two halves of the SM's tensor memory (512 columns), so one
// pipeline stage (A0, A1, B = 512 channels x 32 tokens) feeds four MMAs.  Diagonal super-tiles
// load B only: A0 and A1 are its two halves.  CTAs are persistent (one per SM) and walk the
// (token-split, super-tile) items split-major, so that CTAs running at the same time stream the
// same token range and X is read from HBM about once.
//
// 6 warps per CTA:
//   warp 0      TMA producer (one elected lane)
//   warp 1      MMA issuer (one elected lane); owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld -> scale -> 128-bit red.global.add.f32 to H and, through a
//               per-warp shared-memory transpose, to the mirrored position
// Every wait is bounded: when a limit expires the kernel raises a flag, drains its own copies,
// frees its tensor memory and returns; the host sees LC_ERR_TIMEOUT in *status.
#include "umma_common.cuh"

namespace lc {
namespace {

constexpr int ST = 256;        // super-tile edge
constexpr int BK = 32;         // tokens per pipeline stage
constexpr int kMaxAccumTokens = 4096;   // most tokens one work item accumulates in the tensor core (see hessian_launch)
constexpr int UMMA_K = 16;     // bf16
constexpr int STAGES = 6;
constexpr int ATOM = 64;       // channels per 128-byte swizzle row
constexpr int ATOM_BYTES = ATOM * 2 * BK;   // 4096: one 64ch x 32tok box
constexpr int A_ATOMS = 2, B_ATOMS = 4;
constexpr int STAGE_BYTES = (2 * A_ATOMS + B_ATOMS) * ATOM_BYTES;  // 32768
constexpr int STG_STRIDE = 36;                                     // floats per staged row
constexpr int STG_BYTES_PER_WARP = 32 * STG_STRIDE * 4;            // 4608
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * STG_BYTES_PER_WARP + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;
constexpr int kThreads = 192;
constexpr int MAX_SEG = 8;

using namespace umma;

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 x bf16, both operands MN-major, M=128, N=256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                            ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

struct TmapArray {
  CUtensorMap m[MAX_SEG];
};

struct HessArgs {
  float* H;
  int32_t* status;
  int64_t cols;
  int n_st;        // super-tiles per dimension
  int n_super;     // super-tiles on or above the diagonal
  int n_items;     // n_super * ksplit: every super-tile's tokens in ksplit equal parts, walked part-major
  int ksplit;
  int k_total;     // pipeline iterations over all segments
  int nseg;
  int seg_k[MAX_SEG];
  float alpha;
  int use3d;       // tensor maps are 3-D views: two 64-channel atoms per copy
  int upper_only;  // only H[m][n] with n >= m is maintained: no mirrored adds (half the epilogue's atomics)
};

struct Item {
  int si, sj, k_begin, k_end;
};

__device__ __forceinline__ Item decode_item(const HessArgs& a, int item) {
  Item it;
  const int split = item / a.n_super;
  int t = item % a.n_super;
  const int parts = a.ksplit;
  int si = 0;
  for (; si < a.n_st; ++si) {
    const int cnt = a.n_st - si;
    if (t < cnt) break;
    t -= cnt;
  }
  it.si = si;
  it.sj = si + t;
  const int chunk = (a.k_total + parts - 1) / parts;
  it.k_begin = split * chunk;
  it.k_end = min(a.k_total, it.k_begin + chunk);
  return it;
}

__global__ void __launch_bounds__(kThreads, 1) hessian_umma_kernel(const __grid_constant__ TmapArray maps, HessArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  float* staging = reinterpret_cast<float*>(gen_base + STAGES * STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + STAGES * STAGE_BYTES + 4 * STG_BYTES_PER_WARP);
  // bars: [0,S) full, [S,2S) empty, 2S accumulator full, 2S+1 accumulator empty; then tmem slot, abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = base + STAGES * STAGE_BYTES + 4 * STG_BYTES_PER_WARP;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t accum_full = bar0 + 8u * (2 * STAGES);
  const uint32_t accum_empty = bar0 + 8u * (2 * STAGES + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
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
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  const int64_t C = a.cols;

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t n = 0;  // running stage counter across items
      uint32_t issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < a.n_items; item += gridDim.x) {
        const Item w = decode_item(a, item);
        if (w.k_begin >= w.k_end) continue;
        const bool diag = (w.si == w.sj);
        const bool has_a1 = (int64_t)w.si * ST + 128 < C;
        // locate the first iteration inside the segment list
        int seg = 0, kloc = w.k_begin;
        while (seg < a.nseg && kloc >= a.seg_k[seg]) kloc -= a.seg_k[seg++];
        for (int k = w.k_begin; k < w.k_end; ++k, ++n) {
          const int s = n % STAGES;
          const uint32_t ph = (n / STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const int n_atoms = B_ATOMS + (diag ? 0 : (has_a1 ? 2 * A_ATOMS : A_ATOMS));
          mbar_expect_tx(full_bar(s), n_atoms * ATOM_BYTES);
          const uint32_t sa = base + s * STAGE_BYTES;
          const CUtensorMap* map = &maps.m[seg];
          const int tok = kloc * BK;
          if (a.use3d) {
            // one copy per pair of 64-channel atoms (8 KB); atoms land 4096 bytes apart as below
            if (!diag) {
              tma_load_3d(sa, map, 0, tok, (w.si * ST) / ATOM, full_bar(s));
              if (has_a1) tma_load_3d(sa + A_ATOMS * ATOM_BYTES, map, 0, tok, (w.si * ST + 128) / ATOM, full_bar(s));
            }
            tma_load_3d(sa + 2 * A_ATOMS * ATOM_BYTES, map, 0, tok, (w.sj * ST) / ATOM, full_bar(s));
            tma_load_3d(sa + (2 * A_ATOMS + 2) * ATOM_BYTES, map, 0, tok, (w.sj * ST) / ATOM + 2, full_bar(s));
          } else {
          if (!diag) {
#pragma unroll
            for (int q = 0; q < A_ATOMS; ++q) tma_load_2d(sa + q * ATOM_BYTES, map, w.si * ST + q * ATOM, tok, full_bar(s));
            if (has_a1) {
#pragma unroll
              for (int q = 0; q < A_ATOMS; ++q)
                tma_load_2d(sa + (A_ATOMS + q) * ATOM_BYTES, map, w.si * ST + 128 + q * ATOM, tok, full_bar(s));
            }
          }
#pragma unroll
          for (int q = 0; q < B_ATOMS; ++q)
            tma_load_2d(sa + (2 * A_ATOMS + q) * ATOM_BYTES, map, w.sj * ST + q * ATOM, tok, full_bar(s));
          }
          issued = n + 1;
          if (++kloc >= a.seg_k[seg]) {
            kloc = 0;
            ++seg;
          }
        }
      }
      if (*abort_flag) {
        // drain: the copies this thread started must land before the CTA's shared memory goes away
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t i = first; i < issued; ++i) {
          const int s = i % STAGES;
          const uint32_t ph = (i / STAGES) & 1u;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_test(full_bar(s), ph); ++it) __nanosleep(50);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t n = 0, items_done = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < a.n_items; item += gridDim.x) {
        const Item w = decode_item(a, item);
        if (w.k_begin >= w.k_end) continue;
        const bool diag = (w.si == w.sj);
        const bool has_a1 = (int64_t)w.si * ST + 128 < C;
        // the epilogue must have drained the accumulators of the previous item
        if (!mbar_wait(accum_empty, (items_done & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        for (int k = w.k_begin; k < w.k_end; ++k, ++n) {
          const int s = n % STAGES;
          const uint32_t ph = (n / STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES;
          const uint32_t b_base = sa + 2 * A_ATOMS * ATOM_BYTES;
          const uint32_t a0_base = diag ? b_base : sa;
          const uint32_t a1_base = diag ? b_base + A_ATOMS * ATOM_BYTES : sa + A_ATOMS * ATOM_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // one MMA consumes 16 tokens = two 8-row groups of 1024 bytes
            const uint32_t acc = (k > w.k_begin || kk > 0) ? 1u : 0u;
            const uint64_t bd = make_desc_mn_sw128(b_base + kk * 2048, ATOM_BYTES, 1024);
            umma_bf16(tmem_acc, make_desc_mn_sw128(a0_base + kk * 2048, ATOM_BYTES, 1024), bd, kIdesc, acc);
            if (has_a1)
              umma_bf16(tmem_acc + 256, make_desc_mn_sw128(a1_base + kk * 2048, ATOM_BYTES, 1024), bd, kIdesc, acc);
          }
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(accum_full);  // arrives when every MMA of this item has completed
        ++items_done;
      }
      if (*abort_flag) {
        // make sure nothing is still writing tensor memory before it is freed
        umma_commit(accum_full);
        for (uint32_t it = 0; it < kSpinLimit && !mbar_test(accum_full, items_done & 1u); ++it) __nanosleep(50);
      }
    }
  } else {
    // ---- epilogue -----------------------------------------------------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    float* stg = staging + q * (STG_BYTES_PER_WARP / 4);
    uint32_t items_done = 0;
    for (int item = blockIdx.x; item < a.n_items; item += gridDim.x) {
      const Item w = decode_item(a, item);
      if (w.k_begin >= w.k_end) continue;
      if (!mbar_wait(accum_full, items_done & 1u, abort_flag) || *abort_flag) break;
      tcgen05_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int64_t m_blk0 = (int64_t)w.si * ST + h * 128 + q * 32;
        if ((int64_t)w.si * ST + h * 128 >= C) break;
        const int64_t m = m_blk0 + lane;
        if (a.upper_only) {
          // upper triangle only: the 32-column chunks strictly right of this warp's rows go out as plain
          // 128-bit atomic adds, two chunks' tensor-memory loads in flight at a time
          const uint32_t tbase = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 256);
          int cc = 0;
          while (cc < ST / 32 && (int64_t)w.sj * ST + cc * 32 <= m_blk0 && (int64_t)w.sj * ST + cc * 32 < C) {
            const int64_t n0 = (int64_t)w.sj * ST + cc * 32;
            if (n0 == m_blk0) {      // the diagonal chunk: element-wise, n >= m
              float v[32];
              tmem_ld32(tbase + (uint32_t)(cc * 32), v);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (m < C && n0 + j < C && j >= lane) red_add(a.H + m * C + n0 + j, v[j] * a.alpha);
            }
            ++cc;
          }
          for (; cc < ST / 32; cc += 2) {
            const int64_t n0 = (int64_t)w.sj * ST + cc * 32;
            if (n0 >= C) break;
            const bool two = cc + 1 < ST / 32 && n0 + 32 < C;
            uint32_t r0[32], r1[32];
            tmem_ld32_nowait(tbase + (uint32_t)(cc * 32), r0);
            if (two) tmem_ld32_nowait(tbase + (uint32_t)(cc * 32 + 32), r1);
            tmem_wait_ld();
            // A lane holds one row of the chunk.  Written straight from there, a 128-bit atomic of the warp would
            // touch 32 rows with 16 bytes each (32 half-used sectors); through the warp's staging tile eight
            // lanes cover 128 contiguous bytes of a row, so an instruction touches 4 rows x 4 full sectors.
            auto flush_chunk = [&](const uint32_t (&rv)[32], int64_t nbase) {
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(&stg[lane * STG_STRIDE + j]) =
                    make_float4(__uint_as_float(rv[j]) * a.alpha, __uint_as_float(rv[j + 1]) * a.alpha,
                                __uint_as_float(rv[j + 2]) * a.alpha, __uint_as_float(rv[j + 3]) * a.alpha);
              __syncwarp();
              const int64_t nc = nbase + 4 * (lane & 7);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = 4 * i + (lane >> 3);
                const float4 t = *reinterpret_cast<const float4*>(&stg[rr * STG_STRIDE + 4 * (lane & 7)]);
                if (m_blk0 + rr < C && nc < C) red_add_v4(a.H + (m_blk0 + rr) * C + nc, t.x, t.y, t.z, t.w);
              }
            };
            flush_chunk(r0, n0);
            if (two) flush_chunk(r1, n0 + 32);
          }
          continue;
        }
#pragma unroll 1
        for (int cc = 0; cc < ST / 32; ++cc) {
          const int64_t n0 = (int64_t)w.sj * ST + cc * 32;
          if (n0 >= C) break;
          if (n0 < m_blk0) continue;  // block strictly below the diagonal: covered by a mirror write
          float v[32];
          tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 256 + cc * 32), v);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= a.alpha;
          if (n0 > m_blk0) {
            // block strictly above the diagonal: every element goes to H[m][n] and H[n][m]
            if (m < C) {
              float* row = a.H + m * C + n0;
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                if (n0 + j < C) red_add_v4(row + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) stg[j * STG_STRIDE + lane] = v[j];
            __syncwarp();
            const int mq = lane & 7;
            if (m_blk0 + 4 * mq < C) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int nl = (lane >> 3) + 4 * i;
                const float4 t = *reinterpret_cast<const float4*>(&stg[nl * STG_STRIDE + 4 * mq]);
                if (n0 + nl < C) red_add_v4(a.H + (n0 + nl) * C + m_blk0 + 4 * mq, t.x, t.y, t.z, t.w);
              }
            }
          } else {
            // diagonal block (n0 == m_blk0): element-wise, n >= m direct and n > m mirrored
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int64_t nn = n0 + j;
              if (m < C && nn < C) {
                if (j >= lane) red_add(a.H + m * C + nn, v[j]);
                if (j > lane) red_add(a.H + nn * C + m, v[j]);
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accum_empty);
      ++items_done;
    }
  }

  // ---- teardown -------------------------------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)LC_ERR_TIMEOUT);
}

__global__ void scale_kernel(float* H, int64_t n, float beta) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = *reinterpret_cast<float4*>(H + i);
    if (beta == 0.f) v = make_float4(0.f, 0.f, 0.f, 0.f);
    else { v.x *= beta; v.y *= beta; v.z *= beta; v.w *= beta; }
    *reinterpret_cast<float4*>(H + i) = v;
  } else {
    for (int64_t k = i; k < n; ++k) H[k] = (beta == 0.f) ? 0.f : H[k] * beta;
  }
}

// Self-test of the bounded-wait path: one thread waits on a barrier that nothing ever arrives on,
// with a limit of about a millisecond, and reports the expiry the way the real kernels do.
__global__ void wait_expiry_selftest_kernel(int32_t* status, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, limit);
    if (!ok && abort_flag && status) atomicExch(status, (int)LC_ERR_TIMEOUT);
  }
}

int hessian_launch(const void* const* xs, const int64_t* tokens, int nseg, int64_t cols, float* H, float alpha,
                   float beta, int ksplit, int32_t* status, cudaStream_t st, int upper_only = 0) {
  if (!H || cols <= 0 || ksplit < 0 || nseg < 0 || nseg > MAX_SEG) return LC_ERR_ARG;
  if (cols % 8 != 0) return LC_ERR_ALIGN;
  if (!aligned16(H)) return LC_ERR_ALIGN;
  for (int s = 0; s < nseg; ++s) {
    if (tokens[s] < 0 || tokens[s] >= ((int64_t)1 << 31)) return LC_ERR_SHAPE;
    if (tokens[s] > 0 && (!xs[s] || !aligned16(xs[s]))) return xs[s] ? LC_ERR_ALIGN : LC_ERR_ARG;
  }
  int dev = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  int major = 0, sms = 0;
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));

  if (beta != 1.f) {
    const int64_t n = cols * cols;
    scale_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, st>>>(H, n, beta);
    LC_LAUNCH_CHECK();
  }

  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  TmapArray maps;
  HessArgs a;
  // whole 64-channel atoms only: the 3-D view cannot describe a ragged last atom
  const bool use3d = cols % ATOM == 0;
  a.use3d = use3d ? 1 : 0;
  a.nseg = 0;
  a.k_total = 0;
  for (int s = 0; s < nseg; ++s) {
    if (tokens[s] == 0) continue;
    if (use3d) {
      // (64 channels, tokens, atoms of 64 channels): a box of two atoms x 32 tokens per copy
      const cuuint64_t gdim[3] = {(cuuint64_t)ATOM, (cuuint64_t)tokens[s], (cuuint64_t)(cols / ATOM)};
      const cuuint64_t gstride[2] = {(cuuint64_t)cols * 2, (cuuint64_t)ATOM * 2};
      const cuuint32_t box[3] = {ATOM, BK, 2};
      const cuuint32_t estr[3] = {1, 1, 1};
      if (encode(&maps.m[a.nseg], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(xs[s]), gdim, gstride, box,
                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return LC_ERR_CUDA;
    } else {
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)tokens[s]};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {ATOM, BK};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&maps.m[a.nseg], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xs[s]), gdim, gstride, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return LC_ERR_CUDA;
    }
    a.seg_k[a.nseg] = (int)((tokens[s] + BK - 1) / BK);
    a.k_total += a.seg_k[a.nseg];
    ++a.nseg;
  }
  if (a.nseg == 0) return LC_OK;
  for (int s = a.nseg; s < MAX_SEG; ++s) {
    maps.m[s] = maps.m[0];
    a.seg_k[s] = 0;
  }
  a.H = H;
  a.status = status;
  a.cols = cols;
  a.n_st = (int)((cols + ST - 1) / ST);
  a.n_super = a.n_st * (a.n_st + 1) / 2;
  a.alpha = alpha;
  a.upper_only = upper_only;
  if (ksplit == 0) {
    // The tensor core adds every MMA's products into the fp32 accumulator with truncation, so a sum loses
    // about 2^-24 of its value per 16-token MMA step: a relative deficit that grows with the number of
    // tokens one work item accumulates (measured: -5.6e-5 over 16384 tokens, -2.7e-5 over 8192, -1.0e-5 over 4096), nearly uniform
    // over the matrix as long as every item accumulates the same number of tokens.  The uniform part does
    // not change the GPTQ solve (act-order, dampening and the ratios of U all scale together); the spread
    // around it does (it reorders near-equal diagonal entries), and it shrinks with the item length too.
    // So the token range of a launch is cut into equal parts of at most kMaxAccumTokens, every super-tile
    // the same way (no uneven split of a tail wave), and the parts are combined by fp32 atomic adds.
    ksplit = (a.k_total * BK + kMaxAccumTokens - 1) / kMaxAccumTokens;
    if (ksplit < 1) ksplit = 1;
    // Few super-tiles: split further so that about one item lands on every SM.
    if (a.n_super * ksplit * 2 <= sms) {
      int fill = sms / a.n_super;
      const int max_split = a.k_total / 8 > 0 ? a.k_total / 8 : 1;
      if (fill > max_split) fill = max_split;
      if (fill > ksplit) ksplit = fill;
    }
  }
  if (ksplit > a.k_total) ksplit = a.k_total;
  a.ksplit = ksplit;
  a.n_items = a.n_super * ksplit;
  const int grid = a.n_items < sms ? a.n_items : sms;
  LC_CHECK_CUDA(cudaFuncSetAttribute(hessian_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  hessian_umma_kernel<<<grid, kThreads, SMEM_BYTES, st>>>(maps, a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_selftest_wait_expiry(int32_t* status, lc_stream_t stream) {
  if (!status) return LC_ERR_ARG;
  lc::wait_expiry_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, 20000u);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_hessian_accum(const void* x_bf16, int64_t tokens, int64_t cols, float* H, float alpha,
                                       float beta, int ksplit, int32_t* status, lc_stream_t stream) {
  if (tokens < 0) return LC_ERR_ARG;
  const void* xs[1] = {x_bf16};
  const int64_t tk[1] = {tokens};
  if (tokens > 0 && !x_bf16) return LC_ERR_ARG;
  return lc::hessian_launch(xs, tk, 1, cols, H, alpha, beta, ksplit, status, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" LC_API int lc_hessian_accum_multi(const void* const* xs_host, const int64_t* tokens_host, int nseg,
                                             int64_t cols, float* H, float alpha, float beta, int ksplit,
                                             int32_t* status, lc_stream_t stream) {
  if (nseg < 0 || nseg > lc::MAX_SEG || (nseg > 0 && (!xs_host || !tokens_host))) return LC_ERR_ARG;
  return lc::hessian_launch(xs_host, tokens_host, nseg, cols, H, alpha, beta, ksplit, status,
                            reinterpret_cast<cudaStream_t>(stream));
}

extern "C" LC_API int lc_hessian_accum_upper(const void* const* xs_host, const int64_t* tokens_host, int nseg,
                                             int64_t cols, float* H, float alpha, float beta, int ksplit,
                                             int32_t* status, lc_stream_t stream) {
  if (nseg < 0 || nseg > lc::MAX_SEG || (nseg > 0 && (!xs_host || !tokens_host))) return LC_ERR_ARG;
  return lc::hessian_launch(xs_host, tokens_host, nseg, cols, H, alpha, beta, ksplit, status,
                            reinterpret_cast<cudaStream_t>(stream), 1);
}
