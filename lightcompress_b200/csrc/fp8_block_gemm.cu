// Block-scaled FP8 GEMM of the block-wise FP8 linear: C = sum over 128-wide k blocks of
// (A_kb B_kb^T) * (a_s[m][kb] * b_s[n / 128][kb]), A (M x K) e4m3 activations with one fp32 scale per
// row and k block (act_quant), B (N x K) e4m3 weights with one fp32 scale per 128 x 128 block
// (the reference's Triton fp8_gemm, llmc/compression/quantization/kernel.py:153-242, called from
// block_wise_fp8_forward_func, module_utils.py:41-46).
//
// tcgen05 kind::f8f6f4, both operands K-major (a 128-byte swizzle row holds exactly one k block of a
// row), 128 x 128 output tiles.  The scales differ per k block, so a k block's product cannot stay in
// the tensor-core accumulator: each k block is accumulated on its own (4 MMAs of K = 32) into one of
// four 128-column TMEM buffers, and the eight epilogue warps fold it into fp32 registers with the
// product of the block's two scales while the tensor core already works on the next k blocks.  One TMA copy per operand
// and k block (16 KB each), six stages; persistent CTAs; warp 0 = TMA producer, warp 1 = MMA issuer,
// warps 2-9 = promotion + epilogue (a thread owns 64 columns of one output row; one 64-column
// tensor-memory load and 64 FMAs per k block).
// Every wait is bounded; on expiry the CTA raises its abort flag, drains its copies in flight, frees
// its tensor memory and reports LC_ERR_TIMEOUT through the caller's status word.
#include "umma_common.cuh"

namespace lc {
namespace {

using namespace umma;

constexpr int TM = 128, TN = 128, KB = 128;   // tile and k block (bytes = elements for fp8)
constexpr int UK = 32;                         // MMA depth for 8-bit operands
constexpr int STAGES = 6;
constexpr int OPERAND_BYTES = TM * KB;         // 16384
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;
constexpr int NBUF = 4;                        // TMEM accumulators of 128 columns
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int kEpiWarps = 8;                   // two warps per TMEM lane quarter, 64 columns each
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int EPI_COLS = TN / (kEpiWarps / 4);  // 64

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

// 64 consecutive columns of this warp's 32 TMEM lanes, one row per lane
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
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
                 "r"((uint32_t)(NBUF * TN))
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
        const int m0 = (t % a.m_tiles) * TM, n0 = (t / a.m_tiles) * TN;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++n) {
          const int s = n % STAGES;
          const uint32_t ph = (n / STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t sa = base + s * STAGE_BYTES;
          tma_load_2d(sa, &maps.a, kb * KB, m0, full_bar(s));
          tma_load_2d(sa + OPERAND_BYTES, &maps.b, kb * KB, n0, full_bar(s));
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
          const uint32_t tmem_acc = tmem_base + buf * TN;
#pragma unroll
          for (int j = 0; j < KB / UK; ++j) {
            // K-major, 128-byte swizzle: 8-row groups are 1024 bytes apart; stepping 32 bytes along the
            // swizzled row selects the next 32 values of k
            const uint64_t da = make_desc_mn_sw128(sa + j * UK, 16, 1024);
            const uint64_t db = make_desc_mn_sw128(sa + OPERAND_BYTES + j * UK, 16, 1024);
            umma_f8(tmem_acc, da, db, kIdescF8, j > 0 ? 1u : 0u);
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
    const int half = (warp - 2) >> 2;           // which 64 columns of the tile
    uint32_t n = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
      const int m0 = (t % a.m_tiles) * TM, n0 = (t / a.m_tiles) * TN;
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < a.M;
      const float* as_row = a.a_s + (int64_t)(row_ok ? m : 0) * a.k_blocks;
      const float* bs_row = a.b_s + (int64_t)(n0 / TN) * a.k_blocks;
      float acc[EPI_COLS];
#pragma unroll
      for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < a.k_blocks; ++kb, ++n) {
        const uint32_t buf = n % NBUF;
        const float sc = __fmul_rn(as_row[kb], bs_row[kb]);
        if (!mbar_wait(acc_full(buf), (n / NBUF) & 1u, abort_flag) || *abort_flag) { ok = false; break; }
        tcgen05_fence_after();
        float v[EPI_COLS];
        tmem_ld64(tmem_base + buf * TN + half * EPI_COLS + ((uint32_t)(q * 32) << 16), v);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(buf));   // the values are in registers: the buffer is free again
#pragma unroll
        for (int j = 0; j < EPI_COLS; ++j) acc[j] = fmaf(v[j], sc, acc[j]);
      }
      if (!ok) break;
      if (row_ok) {
        const int c0 = n0 + half * EPI_COLS;
        if (a.out_dtype == LC_BF16) {
          __nv_bfloat16* row = static_cast<__nv_bfloat16*>(a.C) + (int64_t)m * a.N + c0;
          if (c0 + EPI_COLS <= a.N && (a.N & 7) == 0) {
#pragma unroll
            for (int j = 0; j < EPI_COLS; j += 8) {
              __nv_bfloat16 o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[j + e]);
              *reinterpret_cast<uint4*>(row + j) = *reinterpret_cast<const uint4*>(o);
            }
          } else {
#pragma unroll
            for (int j = 0; j < EPI_COLS; ++j)
              if (c0 + j < a.N) row[j] = __float2bfloat16_rn(acc[j]);
          }
        } else {
          float* row = static_cast<float*>(a.C) + (int64_t)m * a.N + c0;
#pragma unroll
          for (int j = 0; j < EPI_COLS; ++j)
            if (c0 + j < a.N) row[j] = acc[j];
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(NBUF * TN))
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)LC_ERR_TIMEOUT);
}

int encode_u8_2d(CUtensorMap* m, const void* base, int64_t k, int64_t rows) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return LC_ERR_CUDA;
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {KB, TM};
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
  if ((rc = encode_u8_2d(&maps.a, a, K, M)) != LC_OK) return rc;
  if ((rc = encode_u8_2d(&maps.b, b, K, N)) != LC_OK) return rc;
  F8Args args;
  args.a_s = a_s;
  args.b_s = b_s;
  args.C = c;
  args.status = status;
  args.M = (int)M;
  args.N = (int)N;
  args.k_blocks = (int)(K / 128);
  args.m_tiles = (int)((M + TM - 1) / TM);
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
