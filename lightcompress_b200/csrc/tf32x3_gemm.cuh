// Internal interface of the three-term tf32 tensor-core GEMM (tf32x3_gemm.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lc {

// flags (same values as LC_GEMM_* of the C ABI)
constexpr int kGemmUpperOnly = 1;   // C is a diagonal-aligned square: tiles entirely below the diagonal are skipped
constexpr int kGemmBLower = 2;      // B[k][n] == 0 for k < n: a tile's k range starts at its first column
constexpr int kGemmAUpper = 4;      // A[k][m] == 0 for k > m: a tile's k range ends after its last row

// A k-row operand matrix X = hi + lo, [k_extent][mn_extent] with pitch ld, and its two tensor maps.
// Prepared once, then any sub-matrix of it can be an operand (origin given per launch), which keeps
// tensor-map encoding out of loops that launch hundreds of small products.
struct GemmMat {
  CUtensorMap map_hi, map_lo;      // 2-D: one 32-float x 16-row box per copy
  // 3-D views (32 floats, k rows, 32-float atoms): a whole operand tile per copy, 4 atoms when the matrix
  // is the A operand, 8 when it is B
  CUtensorMap map3a_hi, map3a_lo, map3b_hi, map3b_lo;
  bool has3 = false;               // mn_extent % 32 == 0 and the driver accepted the views
  int64_t k_extent = 0, mn_extent = 0;
};
// hi, lo: 16-byte aligned, ld % 4 == 0.  x_hi is the fp32 value itself (the tensor core truncates it),
// x_lo = x - truncate_tf32(x).
int gemm_mat_init(GemmMat* m, const float* hi, const float* lo, int64_t k_extent, int64_t mn_extent, int64_t ld);

// C[M][N] (pitch ldc) = beta * C + sign * A'^T B', A' = A[a_k0 : a_k0 + K, a_m0 : a_m0 + M],
// B' = B[b_k0 : b_k0 + K, b_n0 : b_n0 + N].  K % 16 == 0; M, N, ldc and the origins multiples of 4.
// Rows / columns of a tile beyond M / N read whatever follows in the operand matrix (or zeros beyond
// its extent) and are never stored.
// b_tri_shift: with kGemmBLower, B' is columns [shift, shift + N) of a lower-triangular matrix whose rows
// start at B''s first row, i.e. B'[k][n] == 0 for k < n + shift.
int tf32x3_gemm_launch(float* C, int64_t ldc, const GemmMat& A, int64_t a_k0, int64_t a_m0, const GemmMat& B,
                       int64_t b_k0, int64_t b_n0, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                       int32_t* status, cudaStream_t st, int64_t b_tri_shift = 0);

// Several products in one launch: same operand matrices, pitch of C, beta, sign and flags; each item
// has its own sub-matrix origins, sizes and C.  Used for the many small products of one recursion level.
constexpr int kGemmMaxBatch = 56;   // items per launch (more are issued in several launches)
struct GemmItem {
  float* C = nullptr;
  int64_t a_k0 = 0, a_m0 = 0, b_k0 = 0, b_n0 = 0, M = 0, N = 0, K = 0, b_tri_shift = 0;
};
int tf32x3_gemm_batched(const GemmMat& A, const GemmMat& B, int64_t ldc, const GemmItem* items, int count, int beta,
                        float sign, int flags, int32_t* status, cudaStream_t st);

// One-off product: prepares both operands and launches.
int tf32x3_gemm_tn(float* C, int64_t ldc, const float* A_hi, const float* A_lo, int64_t lda, const float* B_hi,
                   const float* B_lo, int64_t ldb, int64_t M, int64_t N, int64_t K, int beta, float sign, int flags,
                   int32_t* status, cudaStream_t st);

}  // namespace lc
