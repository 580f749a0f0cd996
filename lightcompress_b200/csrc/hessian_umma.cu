// Family 2: Hessian accumulation  H <- beta*H + alpha * X^T X  on the sm_100a tensor cores.
//
// X is (tokens x cols) bf16 row-major, so for D[m][n] = sum_t X[t][m] X[t][n] both MMA operands
// are "MN-major": the contraction index (tokens) is the strided one.  TMA copies 64-channel x
// 64-token boxes (128-byte rows, 128B swizzle) into shared memory; tcgen05.mma (128x256x16,
// bf16 in, fp32 accumulate in tensor memory) consumes them through MN-major shared-memory
// descriptors.  Only tiles that touch the upper triangle are computed; the epilogue adds each
// tile to H and to its transposed position.
//
// CTA = one (128x256 tile, token range) work item, 6 warps:
//   warp 0      TMA producer (one elected lane)
//   warp 1      MMA issuer (one elected lane); owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld -> scale -> red.global.add.f32
// Every wait is bounded: when a limit expires the kernel raises a flag, drains its own copies,
// frees its tensor memory and returns; the host sees LC_ERR_TIMEOUT in *status.
#include <cuda.h>

#include "lc_common.cuh"

namespace lc {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;        // tokens per pipeline stage
constexpr int UMMA_K = 16;    // bf16
constexpr int STAGES = 4;
constexpr int ATOM = 64;      // channels per 128-byte swizzle row
constexpr int ATOM_BYTES = ATOM * 2 * BK;          // 8192: one 64ch x 64tok box
constexpr int A_BYTES = (BM / ATOM) * ATOM_BYTES;  // 16384
constexpr int B_BYTES = (BN / ATOM) * ATOM_BYTES;  // 32768
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;     // 49152
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 256;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 20u * 1000u * 1000u;  // x >= 50 ns sleeps: about a second

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if the limit expired or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_test(bar, parity)) return true;
    if (it >= 64) __nanosleep(50);
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void red_add(float* p, float a) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory");
}

// Shared-memory matrix descriptor for an MN-major, 128B-swizzled operand:
//   start address, LBO = byte stride between 64-element atoms along M/N,
//   SBO = byte stride between groups of 8 contraction rows, descriptor version 1, SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 x bf16, both operands MN-major.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                            ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

struct HessArgs {
  float* H;
  int32_t* status;
  int64_t cols;
  int tokens;
  int m_tiles, n_tiles, ksplit;
  float alpha;
};

__global__ void __launch_bounds__(kThreads, 1) hessian_umma_kernel(const __grid_constant__ CUtensorMap tmap, HessArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + STAGES * STAGE_BYTES);
  // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulator ready, then tmem slot + abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t accum_bar = bar0 + 8u * (2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which work item ------------------------------------------------------------------------
  int t = blockIdx.x / a.ksplit;
  const int split = blockIdx.x % a.ksplit;
  int mi = 0, ni = 0;
  for (mi = 0; mi < a.m_tiles; ++mi) {
    const int first = mi >> 1;
    const int cnt = a.n_tiles - first;
    if (t < cnt) {
      ni = first + t;
      break;
    }
    t -= cnt;
  }
  const int k_iters_total = (a.tokens + BK - 1) / BK;
  const int chunk = (k_iters_total + a.ksplit - 1) / a.ksplit;
  const int k_begin = split * chunk;
  const int k_end = min(k_iters_total, k_begin + chunk);
  if (mi >= a.m_tiles || k_begin >= k_end) return;  // uniform for the CTA
  const int n_iters = k_end - k_begin;

  // ---- setup ----------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(accum_bar, 1);
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

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------
    if (lane == 0) {
      int issued = 0;
      for (int n = 0; n < n_iters; ++n) {
        const int s = n % STAGES;
        const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        const uint32_t sa = base + s * STAGE_BYTES;
        const int tok = (k_begin + n) * BK;
#pragma unroll
        for (int q = 0; q < BM / ATOM; ++q) tma_load_2d(sa + q * ATOM_BYTES, &tmap, mi * BM + q * ATOM, tok, full_bar(s));
#pragma unroll
        for (int q = 0; q < BN / ATOM; ++q)
          tma_load_2d(sa + A_BYTES + q * ATOM_BYTES, &tmap, ni * BN + q * ATOM, tok, full_bar(s));
        issued = n + 1;
      }
      if (*abort_flag) {
        // drain: the copies this thread started must land before the CTA's shared memory goes away
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int n = first; n < issued; ++n) {
          const int s = n % STAGES;
          const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_test(full_bar(s), ph); ++it) __nanosleep(50);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      bool any = false;
      for (int n = 0; n < n_iters; ++n) {
        const int s = n % STAGES;
        const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
        if (!mbar_wait(full_bar(s), ph, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t sa = base + s * STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // one MMA consumes 16 tokens = two 8-row groups of 1024 bytes
          const uint64_t ad = make_desc_mn_sw128(sa + k * 2048, ATOM_BYTES, 1024);
          const uint64_t bd = make_desc_mn_sw128(sa + A_BYTES + k * 2048, ATOM_BYTES, 1024);
          umma_bf16(tmem_acc, ad, bd, kIdesc, (n > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));
        any = true;
      }
      umma_commit(accum_bar);  // arrives when every MMA issued above has completed
      if (*abort_flag && any) {
        for (uint32_t it = 0; it < kSpinLimit && !mbar_test(accum_bar, 0); ++it) __nanosleep(50);
      }
    }
  } else {
    // ---- epilogue -----------------------------------------------------------------------------
    const bool ready = mbar_wait(accum_bar, 0, abort_flag);
    tcgen05_fence_after();
    if (ready && !*abort_flag) {
      const int q = warp & 3;  // TMEM lane quarter this warp may read
      const int64_t m = (int64_t)mi * BM + q * 32 + lane;
      const int64_t n_base = (int64_t)ni * BN;
      const int64_t C = a.cols;
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(cc * 32), v);
        const int64_t n0 = n_base + cc * 32;
        if (n0 >= C) continue;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= a.alpha;
        // direct: H[m][n] for n >= m
        if (m < C) {
          float* row = a.H + m * C;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int64_t n = n0 + j;
            if (n + 3 < C && n >= m) {
              red_add_v4(row + n, v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (n + e < C && n + e >= m) red_add(row + n + e, v[j + e]);
            }
          }
        }
        // mirror: H[n][m] for n > m (lanes hold consecutive m: coalesced)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int64_t n = n0 + j;
          if (m < C && n < C && n > m) red_add(a.H + n * C + m, v[j]);
        }
      }
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_hessian_accum(const void* x_bf16, int64_t tokens, int64_t cols, float* H, float alpha, float beta,
                                int ksplit, int32_t* status, lc_stream_t stream) {
  using namespace lc;
  if (!H || cols <= 0 || tokens < 0 || ksplit < 0) return LC_ERR_ARG;
  if (tokens > 0 && !x_bf16) return LC_ERR_ARG;
  if (cols % 8 != 0) return LC_ERR_ALIGN;
  if (!aligned16(H) || (tokens > 0 && !aligned16(x_bf16))) return LC_ERR_ALIGN;
  if (tokens >= (int64_t)1 << 31) return LC_ERR_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  int dev = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  int major = 0;
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;

  if (beta != 1.f) {
    const int64_t n = cols * cols;
    scale_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, st>>>(H, n, beta);
    LC_LAUNCH_CHECK();
  }
  if (tokens == 0) return LC_OK;

  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)tokens};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {ATOM, BK};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LC_ERR_CUDA;

  HessArgs a;
  a.H = H;
  a.status = status;
  a.cols = cols;
  a.tokens = (int)tokens;
  a.m_tiles = (int)((cols + BM - 1) / BM);
  a.n_tiles = (int)((cols + BN - 1) / BN);
  a.alpha = alpha;
  int64_t tiles = 0;
  for (int mi = 0; mi < a.m_tiles; ++mi) tiles += a.n_tiles - (mi >> 1);
  const int k_iters = (int)((tokens + BK - 1) / BK);
  if (ksplit == 0) {
    // Fill whole waves of 148 CTAs while keeping at least 32 pipeline iterations per CTA.
    int best = 1;
    double best_eff = 0.0;
    const int max_split = k_iters / 32 > 0 ? k_iters / 32 : 1;
    for (int s = 1; s <= max_split && s <= 64; ++s) {
      const int64_t items = tiles * s;
      const int64_t waves = (items + kNumSMsB200 - 1) / kNumSMsB200;
      const double eff = (double)items / (double)(waves * kNumSMsB200);
      if (eff > best_eff + 0.02) {
        best_eff = eff;
        best = s;
      }
    }
    ksplit = best;
  }
  if (ksplit > k_iters) ksplit = k_iters;
  a.ksplit = ksplit;
  LC_CHECK_CUDA(cudaFuncSetAttribute(hessian_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  hessian_umma_kernel<<<(unsigned)(tiles * ksplit), kThreads, SMEM_BYTES, st>>>(tmap, a);
  LC_LAUNCH_CHECK();
  return LC_OK;
}
