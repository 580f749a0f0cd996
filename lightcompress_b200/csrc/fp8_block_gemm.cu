// Block-scaled FP8 GEMM of the block-wise FP8 linear: C = sum over 128-wide k blocks of
// (A_kb B_kb^T) * (a_s[m][kb] * b_s[n / 128][kb]), A (M x K) e4m3 activations with one fp32 scale per
// row and k block (act_quant), B (N x K) e4m3 weights with one fp32 scale per 128 x 128 block
// (the reference's Triton fp8_gemm, llmc/compression/quantization/kernel.py:153-242, called from
// block_wise_fp8_forward_func, module_utils.py:41-46).
//
// tcgen05 kind::f8f6f4, both operands K-major (a 128-byte swizzle row holds exactly one k block of a
// row), 256 x 128 output tiles as two 128-row halves that share the B tile (128 x 128 tiles were bound by
// the L2 -> shared-memory traffic: 32 KB per 4.2 MFLOP).  The scales differ per k block, so a k block's
// product cannot stay in the tensor-core accumulator: each k block is accumulated on its own (4 MMAs of
// K = 32 per half) into one of two 256-column TMEM buffers, and the eight epilogue warps fold it into
// fp32 registers with the product of the block's two scales while the tensor core already works on the
// next k block.  One TMA copy per operand and k block (32 + 16 KB), four stages; persistent CTAs; warp 0 =
// TMA producer, warp 1 = MMA issuer, warps 2-9 = promotion + epilogue (a thread owns one output row of
// the tile: 128 fp32 accumulators, 128 FMAs per k block).
// Every wait is bounded; on expiry the CTA raises its abort flag, drains its copies in flight, frees
// its tensor memory and reports LC_ERR_TIMEOUT through the caller's status word.
#include "umma_common.cuh"

namespace lc {
namespace {

using namespace umma;

constexpr int TM = 128, TN = 128, KB = 128;   // MMA tile and k block (bytes = elements for fp8)
constexpr int HALVES = 2;                      // 128-row halves of a CTA tile
constexpr int CTA_M = HALVES * TM;             // 256
constexpr int UK = 32;                         // MMA depth for 8-bit operands
constexpr int STAGES = 4;
constexpr int OPERAND_BYTES = TM * KB;         // 16384: one 128-row operand tile
constexpr int STAGE_BYTES = (HALVES + 1) * OPERAND_BYTES;   // A: two halves, B: one
constexpr int NBUF = 2;                        // TMEM accumulators of HALVES * 128 columns
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int kEpiWarps = 4 * HALVES;          // one warp per TMEM lane quarter and half
constexpr int kThreads = 64 + 32 * kEpiWarps;

// kind::f8f6f4: D fp32, A = B = e4m3 (format 0), both K-major, N = 128, M = 128
constexpr uint32_t kIdescF8 = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

struct F8Maps {
  CUtensorMap a, b;
};

struct F8Args {
  const float* a_s;   // [M][k_blocks]
  const float* b_s;   // [ceil(N / 128)][k_blocks]
  void* C;            // [M][N]
  int32_t* status;
  int M, N, k_blocks;
  int m_tiles, n_tiles;
  int out_dtype;
};

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) fp8_block_gemm_kernel(const __grid_constant__ F8Maps maps, F8Args a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (2 * STAGES + NBUF + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), kEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)(NBUF * HALVES * TN))
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
        const int m0 = (t % a.m_tiles) * CTA_M, n0 = (t / a.m_tiles) * TN;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++n) {
          const int s = n % STAGES;
          const uint32_t ph = (n / STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t sa = base + s * STAGE_BYTES;
          tma_load_2d(sa, &maps.a, kb * KB, m0, full_bar(s));                         // 256 rows: both halves
          tma_load_2d(sa + HALVES * OPERAND_BYTES, &maps.b, kb * KB, n0, full_bar(s));
          issued = n + 1;
        }
      }
      if (*abort_flag) {
        // let the copies still in flight land before the CTA's shared memory is released
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t i = first; i < issued; ++i) {
          const int s = i % STAGES;
          const uint32_t ph = (i / STAGES) & 1u;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_test(full_bar(s), ph); ++it) __nanosleep(50);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t n = 0;   // k blocks issued so far: stage n % STAGES, accumulator n % NBUF
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        for (int kb = 0; kb < a.k_blocks; ++kb, ++n) {
          const int s = n % STAGES;
          const uint32_t buf = n % NBUF;
          if (!mbar_wait(acc_empty(buf), ((n / NBUF) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(full_bar(s), (n / STAGES) & 1u, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const uint32_t tmem_acc = tmem_base + (buf * HALVES + h) * TN;
#pragma unroll
            for (int j = 0; j < KB / UK; ++j) {
              // K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart; stepping 32 bytes along the
              // swizzled row selects the next 32 values of k
              const uint64_t da = make_desc_mn_sw128(sa + h * OPERAND_BYTES + j * UK, 16, 1024);
              const uint64_t db = make_desc_mn_sw128(sa + HALVES * OPERAND_BYTES + j * UK, 16, 1024);
              umma_f8(tmem_acc, da, db, kIdescF8, j > 0 ? 1u : 0u);
            }
          }
          umma_commit(empty_bar(s));
          umma_commit(acc_full(buf));
        }
      }
      if (*abort_flag && n > 0) {
        // the MMAs already issued must retire before the tensor memory is freed
        const uint32_t last = n - 1, buf = last % NBUF;
        for (uint32_t it = 0; it < kSpinLimit && !mbar_test(acc_full(buf), (last / NBUF) & 1u); ++it) __nanosleep(50);
      }
    }
  } else {
    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    const int h = (warp - 2) >> 2;              // which 128-row half of the tile
    uint32_t n = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
      const int m0 = (t % a.m_tiles) * CTA_M, n0 = (t / a.m_tiles) * TN;
      const int m = m0 + h * TM + q * 32 + lane;
      const bool row_ok = m < a.M;
      const float* as_row = a.a_s + (int64_t)(row_ok ? m : 0) * a.k_blocks;
      const float* bs_row = a.b_s + (int64_t)(n0 / TN) * a.k_blocks;
      float acc[TN];
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < a.k_blocks; ++kb, ++n) {
        const uint32_t buf = n % NBUF;
        const float sc = __fmul_rn(as_row[kb], bs_row[kb]);
        if (!mbar_wait(acc_full(buf), (n / NBUF) & 1u, abort_flag) || *abort_flag) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + (buf * HALVES + h) * TN + ((uint32_t)(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < TN / 32; ++c) {
          float v[32];
          tmem_ld32(taddr + (uint32_t)(c * 32), v);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(v[j], sc, acc[c * 32 + j]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(buf));
      }
      if (!ok) break;
      if (row_ok) {
        if (a.out_dtype == LC_BF16) {
          __nv_bfloat16* row = static_cast<__nv_bfloat16*>(a.C) + (int64_t)m * a.N + n0;
          if (n0 + TN <= a.N && (a.N & 7) == 0) {
#pragma unroll
            for (int j = 0; j < TN; j += 8) {
              __nv_bfloat16 o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[j + e]);
              *reinterpret_cast<uint4*>(row + j) = *reinterpret_cast<const uint4*>(o);
            }
          } else {
#pragma unroll
            for (int j = 0; j < TN; ++j)
              if (n0 + j < a.N) row[j] = __float2bfloat16_rn(acc[j]);
          }
        } else {
          float* row = static_cast<float*>(a.C) + (int64_t)m * a.N + n0;
#pragma unroll
          for (int j = 0; j < TN; ++j)
            if (n0 + j < a.N) row[j] = acc[j];
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(NBUF * HALVES * TN))
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)LC_ERR_TIMEOUT);
}

int encode_u8_2d(CUtensorMap* m, const void* base, int64_t k, int64_t rows, int box_rows) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {KB, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LC_ERR_CUDA;
  return LC_OK;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_fp8_block_gemm(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M,
                                        int64_t N, int64_t K, void* c, int out_dtype, int32_t* status,
                                        lc_stream_t stream) {
  using namespace lc;
  if (!a || !a_s || !b || !b_s || !c) return LC_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return LC_ERR_ARG;
  if (out_dtype != LC_BF16 && out_dtype != LC_F32) return LC_ERR_ARG;
  if (K % 128 != 0) return LC_ERR_SHAPE;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return LC_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return LC_ERR_ALIGN;
  int dev = 0, major = 0, sms = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  F8Maps maps;
  int rc;
  if ((rc = encode_u8_2d(&maps.a, a, K, M, CTA_M)) != LC_OK) return rc;
  if ((rc = encode_u8_2d(&maps.b, b, K, N, TN)) != LC_OK) return rc;
  F8Args args;
  args.a_s = a_s;
  args.b_s = b_s;
  args.C = c;
  args.status = status;
  args.M = (int)M;
  args.N = (int)N;
  args.k_blocks = (int)(K / 128);
  args.m_tiles = (int)((M + CTA_M - 1) / CTA_M);
  args.n_tiles = (int)((N + TN - 1) / TN);
  args.out_dtype = out_dtype;
  const int tiles = args.m_tiles * args.n_tiles;
  // per-device attribute; setting it on every call keeps multi-device processes correct
  LC_CHECK_CUDA(cudaFuncSetAttribute(fp8_block_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  fp8_block_gemm_kernel<<<tiles < sms ? tiles : sms, kThreads, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(
      maps, args);
  LC_LAUNCH_CHECK();
  return LC_OK;
}
