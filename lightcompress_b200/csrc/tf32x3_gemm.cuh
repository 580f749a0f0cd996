// Internal interface of the three-term tf32 tensor-core GEMM (tf32x3_gemm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lc {

// flags (same values as LC_GEMM_* of the C ABI)
constexpr int kGemmUpperOnly = 1;   // C is a diagonal-aligned square: tiles entirely below the diagonal are skipped
constexpr int kGemmBLower = 2;      // B[k][n] == 0 for k < n: a tile's k range starts at its first column
constexpr int kGemmAUpper = 4;      // A[k][m] == 0 for k > m: a tile's k range ends after its last row

// C[M][N] (pitch ldc) = beta * C + sign * A^T B; A = A_hi + A_lo: [K][M] (pitch lda), B = B_hi + B_lo:
// [K][N] (pitch ldb).  K % 16 == 0; M, N and the pitches multiples of 4; pointers 16-byte aligned.
// x_hi is the fp32 value itself (the tensor core truncates it), x_lo = x - truncate_tf32(x).
int tf32x3_gemm_tn(float* C, int64_t ldc, const float* A_hi, const float* A_lo, int64_t lda, const float* B_hi,
                   const float* B_lo, int64_t ldb, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                   int32_t* status, cudaStream_t st);

}  // namespace lc
