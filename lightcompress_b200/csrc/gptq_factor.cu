// Family 3: the factorisation step of the GPTQ solver, U upper-triangular with U^T U = H^-1 for the
// permuted and dampened Hessian (the three cuSOLVER factorisations of
// GPTQ.process_hessian_and_weights, llmc/compression/quantization/gptq.py:172-174).
//
// With A = J H J (H with rows and columns reversed) and its upper Cholesky factor A = G^T G, the
// wanted factor is U = J (G^-1)^T J: one Cholesky and one triangular inverse, no product of the two.
// Both run blocked on 128x128 diagonal blocks, with every large product on the tensor cores through
// the three-term tf32 GEMM (tf32x3_gemm.cu), whose operands are k-row matrices -- which is what row
// panels of G and blocks of (G^-1)^T are, so that no operand needs a transposed copy except the
// square blocks of the inverse that become left factors:
//
//  Cholesky (right-looking, two levels): for each 128-row block k
//      G_kk, V_kk = chol(A_kk), G_kk^-1                       one CTA (leaf kernel)
//      G[k, k+1:] = V_kk^T A[k, k+1:]                         GEMM, K = 128
//      A[k+1:o2, k+1:] -= G[k, k+1:o2]^T G[k, k+1:]           eager: only the rest of the 512-row outer block
//    and once per outer block [o, o2):
//      A[o2:, o2:] -= G[o:o2, o2:]^T G[o:o2, o2:]             lazy GEMM, K = 512, upper tiles only
//  Inverse Vt = (G^-1)^T (lower), recursively on index ranges split at multiples of 128:
//      Vt[hi, lo] = -Vt[hi, hi] (G[lo, hi])^T Vt[lo, lo]      two GEMMs; the leaves are the V_kk^T above
//  U = J Vt J.
//
// Everything is enqueued on the caller's stream; nothing synchronises.  A non-positive pivot sets
// the caller's status word to LC_ERR_NOT_PD (the reference raises torch.linalg.LinAlgError there).
#include <vector>

#include "lc_common.cuh"
#include "tf32x3_gemm.cuh"

namespace lc {
namespace {

constexpr int kB = 128;            // diagonal block
constexpr int kOuter = 512;        // rows per lazy trailing update
constexpr int kLeafThreads = 256;
constexpr int kLd = kB + 4;        // shared-memory pitch: a multiple of 4 floats for 16-byte accesses

__device__ __forceinline__ float tf32_lo(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// One CTA: Cholesky of the 128x128 block at A (pitch lda, upper triangle read) and the inverse of
// its factor.  Writes G_kk (upper; the lower part of the block is zeroed) and its low part, V_kk =
// G_kk^-1 (upper, dense 128x128 block in `v` / `v_lo`), and Vt_kk = V_kk^T with its low part into the
// lower-triangular result.
//
// The block lives in shared memory and both phases are blocked on 16 x 16 sub-blocks, so that the
// CTA-wide barriers number a few dozen instead of one per column:
//   Cholesky, right-looking over the 8 sub-blocks: (a) one warp factorises the 16 x 16 diagonal
//   sub-block in registers (lane = column, the pivot row travels by shuffles; this chain of 128
//   dependent sqrt / divide / update steps is what bounds the kernel), (b) a thread per column solves
//   the 16-row strip right of it by forward substitution, (c) all threads apply the rank-16 update to
//   the rest in 4 x 4 register tiles.
//   Inverse V = G^-1, block row by block row from the bottom: the eight 16 x 16 diagonal inverses first
//   (one warp each), then per block row i the products sum_k G_ik V_kj in 4 x 4 register tiles and a
//   thread per column applies -D_i^-1.
// Quotients are formed as x * (1/d) with one residual correction (the IEEE quotient up to rare last-bit
// cases), like the column kernel this replaces; every accumulation is an fp32 FMA chain.
//
// kCholesky = false: A already holds the factor G_kk (upper); only the inverse is computed and only Vt /
// Vt_lo are written.  One CTA per diagonal block (blockIdx.x), all blocks of a matrix in one launch.
constexpr int kSB = 16;            // sub-block edge
constexpr int kLeafSmemFloats = 2 * kB * kLd;

__device__ __forceinline__ float quot(float x, float d, float dinv) {
  const float q0 = x * dinv;
  return fmaf(fmaf(-q0, d, x), dinv, q0);
}

template <bool kCholesky>
__global__ void __launch_bounds__(kLeafThreads, 1) chol_leaf_kernel(const float* __restrict__ A, int64_t lda,
                                                                     float* __restrict__ G, float* __restrict__ G_lo,
                                                                     int64_t ldg, float* __restrict__ v,
                                                                     float* __restrict__ v_lo, float* __restrict__ Vt,
                                                                     float* __restrict__ Vt_lo, int64_t ldv,
                                                                     int32_t* status) {
  extern __shared__ __align__(16) float leaf_sm[];
  float (*S)[kLd] = reinterpret_cast<float (*)[kLd]>(leaf_sm);              // A, then G (upper)
  float (*V)[kLd] = reinterpret_cast<float (*)[kLd]>(leaf_sm + kB * kLd);   // G^-1 (upper)
  __shared__ float Dinv[kB / kSB][kSB][kSB + 1];   // inverses of the diagonal sub-blocks of G
  __shared__ float rdiag[kB];                      // 1 / G_jj
  __shared__ int s_bad;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_bad = 0;
  if (!kCholesky) {
    A += (int64_t)blockIdx.x * kB * (lda + 1);
    Vt += (int64_t)blockIdx.x * kB * (ldv + 1);
    Vt_lo += (int64_t)blockIdx.x * kB * (ldv + 1);
  }
#pragma unroll 4
  for (int idx = tid; idx < kB * kB / 4; idx += kLeafThreads) {
    const int r = idx >> 5, c = (idx & 31) << 2;
    float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c + 3 >= r) a4 = *reinterpret_cast<const float4*>(A + (int64_t)r * lda + c);
    a4.x = (c >= r) ? a4.x : 0.f, a4.y = (c + 1 >= r) ? a4.y : 0.f;
    a4.z = (c + 2 >= r) ? a4.z : 0.f, a4.w = (c + 3 >= r) ? a4.w : 0.f;
    *reinterpret_cast<float4*>(&S[r][c]) = a4;
    *reinterpret_cast<float4*>(&V[r][c]) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();

  // ---- Cholesky: A = G^T G ----
  if (kCholesky) {
#pragma unroll 1
    for (int jb = 0; jb < kB / kSB; ++jb) {
      const int j0 = jb * kSB;
      // (a) the diagonal sub-block, in the registers of warp 0: lane c (and its twin c + 16) holds column c
      if (warp == 0) {
        const int c = lane & 15;
        float col[kSB];
#pragma unroll
        for (int r = 0; r < kSB; ++r) col[r] = S[j0 + r][j0 + c];
        bool bad = false;
        float rd = 0.f;
#pragma unroll
        for (int j = 0; j < kSB; ++j) {
          const float p = __shfl_sync(0xffffffffu, col[j], j);
          bad = bad || !(p > 0.f) || !(p < INFINITY);
          // 1 / sqrt(p) by the hardware approximation and one Newton step, then sqrt(p) = p * that with one
          // residual correction: both within an ulp, in a third of the latency of sqrtf followed by a divide
          // (this chain of 128 dependent pivots is what bounds the kernel)
          float dinv = rsqrtf(p);
          dinv = dinv * fmaf(-0.5f * p * dinv, dinv, 1.5f);
          float d = p * dinv;
          d = fmaf(fmaf(-d, d, p), 0.5f * dinv, d);
          const float g = (c == j) ? d : ((c > j) ? quot(col[j], d, dinv) : 0.f);
          col[j] = g;
          if (c == j) rd = dinv;
#pragma unroll
          for (int r = j + 1; r < kSB; ++r) {
            const float gr = __shfl_sync(0xffffffffu, g, r);
            col[r] = fmaf(-gr, g, col[r]);          // rows below the diagonal of this column: unused values
          }
        }
        if (lane < kSB) {
#pragma unroll
          for (int r = 0; r < kSB; ++r) S[j0 + r][j0 + c] = (c >= r) ? col[r] : 0.f;
          rdiag[j0 + c] = rd;
        }
        if (bad && lane == 0) s_bad = 1;
      }
      __syncthreads();
      const int ncol = kB - j0 - kSB;          // columns right of the sub-block (multiple of 16)
      if (ncol == 0) break;
      // (b) the strip right of it: X = D^-T S[j0 : j0 + 16, right], a thread per column
      if (tid < ncol) {
        const int c = j0 + kSB + tid;
        // right-looking substitution: as soon as x[k] is known it is taken out of every later row, so the
        // dependent chain per step is one FMA and one quotient instead of a k-term sum
        float x[kSB];
#pragma unroll
        for (int i = 0; i < kSB; ++i) x[i] = S[j0 + i][c];
#pragma unroll
        for (int k = 0; k < kSB; ++k) {
          x[k] = quot(x[k], S[j0 + k][j0 + k], rdiag[j0 + k]);
#pragma unroll
          for (int i = k + 1; i < kSB; ++i) x[i] = fmaf(-S[j0 + k][j0 + i], x[k], x[i]);
          S[j0 + k][c] = x[k];
        }
      }
      __syncthreads();
      // (c) S[r][c] -= sum_k X[k][r] X[k][c] for r, c right of the sub-block, tiles on or above the diagonal
      const int nt = ncol / 4, ntri = nt * (nt + 1) / 2;
      for (int t = tid; t < ntri; t += kLeafThreads) {
        // row-major index of the upper triangle -> (tr, tc)
        int tr = (int)((2.f * nt + 1.f - sqrtf((2.f * nt + 1.f) * (2.f * nt + 1.f) - 8.f * (float)t)) * 0.5f);
        while (tr > 0 && tr * nt - tr * (tr - 1) / 2 > t) --tr;
        while ((tr + 1) * nt - (tr + 1) * tr / 2 <= t) ++tr;
        const int tc = tr + (t - (tr * nt - tr * (tr - 1) / 2));
        const int r0 = j0 + kSB + 4 * tr, c0 = j0 + kSB + 4 * tc;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll
        for (int k = 0; k < kSB; ++k) {
          const float4 xr = *reinterpret_cast<const float4*>(&S[j0 + k][r0]);
          const float4 xc = *reinterpret_cast<const float4*>(&S[j0 + k][c0]);
          const float ar[4] = {xr.x, xr.y, xr.z, xr.w}, ac[4] = {xc.x, xc.y, xc.z, xc.w};
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ar[a], ac[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) S[r0 + a][c0 + b] -= acc[a][b];
      }
      __syncthreads();
    }
  } else {
    if (tid < kB) rdiag[tid] = __frcp_rn(S[tid][tid]);
    __syncthreads();
  }

  // ---- inverse V = G^-1 ----
  // diagonal sub-blocks: warp w inverts D_w (upper) by back substitution, lane c < 16 the column c
  {
    const int j0 = warp * kSB, c = lane & 15;
    float x[kSB];
#pragma unroll
    for (int i = 0; i < kSB; ++i) x[i] = (i == c) ? 1.f : 0.f;
#pragma unroll
    for (int k = kSB - 1; k >= 0; --k) {
      x[k] = (k <= c) ? quot(x[k], S[j0 + k][j0 + k], rdiag[j0 + k]) : 0.f;
#pragma unroll
      for (int i = 0; i < k; ++i) x[i] = fmaf(-S[j0 + i][j0 + k], x[k], x[i]);
    }
    if (lane < kSB) {
#pragma unroll
      for (int i = 0; i < kSB; ++i) {
        Dinv[warp][i][c] = x[i];
        V[j0 + i][j0 + c] = x[i];
      }
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int bi = kB / kSB - 2; bi >= 0; --bi) {
    const int i0 = bi * kSB, k0 = i0 + kSB, ncol = kB - k0;
    // T[r][c] = sum_{k = k0 .. c} G[i0 + r][k] V[k][c], stored where V[i0 + r][c] will go; 2 x 4 register
    // tiles (8 row pairs x ncol / 4 column quads: up to 224 threads), k in steps of 4 with 16-byte reads
    const int ntc = ncol / 4;
    for (int t = tid; t < 8 * ntc; t += kLeafThreads) {
      const int tr = t / ntc, tc = t % ntc;
      const int r0 = i0 + 2 * tr, c0 = k0 + 4 * tc;
      float acc[2][4];
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
      const int kend = c0 + 4;                      // V[k][c] == 0 for k > c; k0 and kend are multiples of 4
#pragma unroll 2
      for (int k = k0; k < kend; k += 4) {
        const float4 g0 = *reinterpret_cast<const float4*>(&S[r0][k]);
        const float4 g1 = *reinterpret_cast<const float4*>(&S[r0 + 1][k]);
        const float ga[2][4] = {{g0.x, g0.y, g0.z, g0.w}, {g1.x, g1.y, g1.z, g1.w}};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 vc = *reinterpret_cast<const float4*>(&V[k + q][c0]);
          const float ac[4] = {vc.x, vc.y, vc.z, vc.w};
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ga[a][q], ac[b], acc[a][b]);
        }
      }
      // rows i0 .. i0 + 15 of V are not read by this loop (k >= k0 = i0 + 16): safe to park T there
#pragma unroll
      for (int a = 0; a < 2; ++a)
        *reinterpret_cast<float4*>(&V[r0 + a][c0]) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
    __syncthreads();
    // V[i0 + r][c] = -sum_{k >= r} Dinv[r][k] T[k][c], a thread per column
    if (tid < ncol) {
      const int c = k0 + tid;
      float tcol[kSB];
#pragma unroll
      for (int k = 0; k < kSB; ++k) tcol[k] = V[i0 + k][c];
#pragma unroll
      for (int r = 0; r < kSB; ++r) {
        float sacc = 0.f;
#pragma unroll
        for (int k = r; k < kSB; ++k) sacc = fmaf(Dinv[bi][r][k], tcol[k], sacc);
        V[i0 + r][c] = -sacc;
      }
    }
    __syncthreads();
  }

  // ---- stores ----
  for (int idx = tid; idx < kB * kB / 4; idx += kLeafThreads) {
    const int r = idx >> 5, c = (idx & 31) << 2;
    if (kCholesky) {
      float gv[4], wv[4], gl[4], wl[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        gv[e] = (c + e >= r) ? S[r][c + e] : 0.f;
        wv[e] = (c + e >= r) ? V[r][c + e] : 0.f;
        gl[e] = tf32_lo(gv[e]), wl[e] = tf32_lo(wv[e]);
      }
      *reinterpret_cast<float4*>(G + (int64_t)r * ldg + c) = make_float4(gv[0], gv[1], gv[2], gv[3]);
      *reinterpret_cast<float4*>(G_lo + (int64_t)r * ldg + c) = make_float4(gl[0], gl[1], gl[2], gl[3]);
      *reinterpret_cast<float4*>(v + r * kB + c) = make_float4(wv[0], wv[1], wv[2], wv[3]);
      *reinterpret_cast<float4*>(v_lo + r * kB + c) = make_float4(wl[0], wl[1], wl[2], wl[3]);
    }
    // Vt[r][c + e] = V[c + e][r] (lower)
    float wt[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) wt[e] = (r >= c + e) ? V[c + e][r] : 0.f;
    *reinterpret_cast<float4*>(Vt + (int64_t)r * ldv + c) = make_float4(wt[0], wt[1], wt[2], wt[3]);
    *reinterpret_cast<float4*>(Vt_lo + (int64_t)r * ldv + c) =
        make_float4(tf32_lo(wt[0]), tf32_lo(wt[1]), tf32_lo(wt[2]), tf32_lo(wt[3]));
  }
  if (tid == 0 && s_bad && status) atomicCAS(status, 0, (int)LC_ERR_NOT_PD);
}

// G[k : k + 128, c] = V_kk^T A[k : k + 128, c] for the columns c right of a diagonal block (the panel
// solve of the blocked Cholesky), with the low part of the result: exact fp32 FMA chains, one launch
// instead of split + GEMM + split.  A CTA takes 64 columns; V_kk (upper, so the sum runs over r <= i)
// and the A tile sit in shared memory; a thread computes 8 rows x 4 columns.
constexpr int kPanelCols = 64;
__global__ void __launch_bounds__(256) chol_panel_kernel(const float* __restrict__ Vkk, const float* __restrict__ Ap,
                                                          int64_t lda, float* __restrict__ Gp, float* __restrict__ Gp_lo,
                                                          int64_t ldg, int64_t ncols) {
  extern __shared__ __align__(16) float panel_sm[];
  float (*Vs)[kB + 4] = reinterpret_cast<float (*)[kB + 4]>(panel_sm);                       // [r][i]
  float (*As)[kPanelCols + 4] = reinterpret_cast<float (*)[kPanelCols + 4]>(panel_sm + kB * (kB + 4));   // [r][c]
  const int tid = threadIdx.x;
  const int64_t c_base = (int64_t)blockIdx.x * kPanelCols;
#pragma unroll
  for (int idx = tid; idx < kB * kB / 4; idx += 256) {
    const int r = idx >> 5, i4 = (idx & 31) << 2;
    *reinterpret_cast<float4*>(&Vs[r][i4]) = *reinterpret_cast<const float4*>(Vkk + r * kB + i4);
  }
#pragma unroll
  for (int idx = tid; idx < kB * kPanelCols / 4; idx += 256) {
    const int r = idx >> 4, c4 = (idx & 15) << 2;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c_base + c4 < ncols) val = *reinterpret_cast<const float4*>(Ap + (int64_t)r * lda + c_base + c4);
    *reinterpret_cast<float4*>(&As[r][c4]) = val;
  }
  __syncthreads();
  const int ti = tid >> 4, tc = tid & 15;          // rows 8 ti .. 8 ti + 7, columns 4 tc .. 4 tc + 3
  const int i0 = ti * 8, c0 = tc * 4;
  float acc[8][4];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  // V upper: V[r][i] != 0 only for r <= i, so rows r beyond i0 + 7 contribute nothing
  for (int r = 0; r < i0 + 8; ++r) {
    const float4 av = *reinterpret_cast<const float4*>(&As[r][c0]);
    const float4 v0 = *reinterpret_cast<const float4*>(&Vs[r][i0]);
    const float4 v1 = *reinterpret_cast<const float4*>(&Vs[r][i0 + 4]);
    const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w}, aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(vv[a], aa[b], acc[a][b]);
  }
  if (c_base + c0 < ncols) {
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int64_t o = (int64_t)(i0 + a) * ldg + c_base + c0;
      *reinterpret_cast<float4*>(Gp + o) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
      *reinterpret_cast<float4*>(Gp_lo + o) =
          make_float4(tf32_lo(acc[a][0]), tf32_lo(acc[a][1]), tf32_lo(acc[a][2]), tf32_lo(acc[a][3]));
    }
  }
}

// A[r][c] -= sum_{i < 128} P[i][r] P[i][c] for r in [r_begin, r_end), c in [r, n): the eager part of the
// blocked Cholesky's trailing update (the rows of the current outer block), P = the panel row block just
// solved (pitch ldp, column index = matrix column).  64 x 64 tiles, tiles entirely below the diagonal
// skipped; exact fp32.
constexpr int kStripTile = 64;
__global__ void __launch_bounds__(256) chol_strip_kernel(const float* __restrict__ P, int64_t ldp, float* __restrict__ Am,
                                                          int64_t lda, int64_t r_begin, int64_t r_end, int64_t n) {
  extern __shared__ __align__(16) float strip_sm[];
  float (*Pr)[kStripTile + 4] = reinterpret_cast<float (*)[kStripTile + 4]>(strip_sm);
  float (*Pc)[kStripTile + 4] = reinterpret_cast<float (*)[kStripTile + 4]>(strip_sm + kB * (kStripTile + 4));
  const int64_t r0 = r_begin + (int64_t)blockIdx.y * kStripTile;
  const int64_t c0 = r_begin + (int64_t)blockIdx.x * kStripTile;
  if (c0 + kStripTile <= r0 || r0 >= r_end || c0 >= n) return;      // below the diagonal or outside
  const int tid = threadIdx.x;
#pragma unroll
  for (int idx = tid; idx < kB * kStripTile / 4; idx += 256) {
    const int i = idx >> 4, x4 = (idx & 15) << 2;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (r0 + x4 < n) a = *reinterpret_cast<const float4*>(P + (int64_t)i * ldp + r0 + x4);
    if (c0 + x4 < n) b = *reinterpret_cast<const float4*>(P + (int64_t)i * ldp + c0 + x4);
    *reinterpret_cast<float4*>(&Pr[i][x4]) = a;
    *reinterpret_cast<float4*>(&Pc[i][x4]) = b;
  }
  __syncthreads();
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 8
  for (int i = 0; i < kB; ++i) {
    const float4 xr = *reinterpret_cast<const float4*>(&Pr[i][tr]);
    const float4 xc = *reinterpret_cast<const float4*>(&Pc[i][tc]);
    const float ar[4] = {xr.x, xr.y, xr.z, xr.w}, ac[4] = {xc.x, xc.y, xc.z, xc.w};
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ar[a], ac[b], acc[a][b]);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int64_t r = r0 + tr + a;
    if (r >= r_end || c0 + tc >= n) continue;
    float4* p = reinterpret_cast<float4*>(Am + r * lda + c0 + tc);
    float4 cur = *p;
    cur.x -= acc[a][0], cur.y -= acc[a][1], cur.z -= acc[a][2], cur.w -= acc[a][3];
    *p = cur;
  }
}

constexpr int kMaxRegions = 64;

// lo = x - tf32_truncate(x) on up to kMaxRegions rows x cols regions (one pitch for all; region blockIdx.y)
struct SplitRegions {
  const float* x[kMaxRegions];
  float* lo[kMaxRegions];
  int rows[kMaxRegions], cols[kMaxRegions];
};
__global__ void __launch_bounds__(256) split_region_kernel(const __grid_constant__ SplitRegions rg, int64_t ld) {
  const int g = blockIdx.y;
  const float* x = rg.x[g];
  float* lo = rg.lo[g];
  const int64_t vec_per_row = rg.cols[g] >> 2;
  const int64_t total = (int64_t)rg.rows[g] * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vec_per_row, c = (idx % vec_per_row) << 2;
    const float4 v = *reinterpret_cast<const float4*>(x + r * ld + c);
    float4 o;
    o.x = tf32_lo(v.x), o.y = tf32_lo(v.y), o.z = tf32_lo(v.z), o.w = tf32_lo(v.w);
    *reinterpret_cast<float4*>(lo + r * ld + c) = o;
  }
}

// out = in^T on up to kMaxRegions square blocks (block blockIdx.z, edge n[z]; pitches ldi / ldo), with the
// low part of the result
struct TransposeBlocks {
  const float* in[kMaxRegions];
  float* out[kMaxRegions];
  float* out_lo[kMaxRegions];
  int n[kMaxRegions];
};
__global__ void __launch_bounds__(256) transpose_split_kernel(const __grid_constant__ TransposeBlocks tb, int64_t ldi,
                                                              int64_t ldo) {
  __shared__ float tile[32][33];
  const int z = blockIdx.z, n = tb.n[z];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  if (bx >= n || by >= n) return;
  const float* in = tb.in[z];
  float* out = tb.out[z];
  float* out_lo = tb.out_lo[z];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int r = ty; r < 32; r += 8)
    if (by + r < n && bx + tx < n) tile[r][tx] = in[(int64_t)(by + r) * ldi + bx + tx];
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    if (bx + r < n && by + tx < n) {
      const float v = tile[tx][r];
      out[(int64_t)(bx + r) * ldo + by + tx] = v;
      out_lo[(int64_t)(bx + r) * ldo + by + tx] = tf32_lo(v);
    }
  }
}

// U = J Vt J restricted to the upper triangle (zeros below), with its low part if asked for
__global__ void __launch_bounds__(256) flip_upper_kernel(const float* __restrict__ Vt, int64_t n,
                                                         float* __restrict__ U, float* __restrict__ U_lo) {
  const int64_t vec_per_row = n >> 2;
  const int64_t total = n * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = idx / vec_per_row, j = (idx % vec_per_row) << 2;
    float o[4];
    if (j + 3 < i) {
      o[0] = o[1] = o[2] = o[3] = 0.f;
    } else {
      // U[i][j + e] = Vt[n-1-i][n-1-j-e]: one reversed 16-byte vector
      const float4 v = *reinterpret_cast<const float4*>(Vt + (n - 1 - i) * n + (n - 4 - j));
      o[0] = v.w, o[1] = v.z, o[2] = v.y, o[3] = v.x;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (j + e < i) o[e] = 0.f;
    }
    *reinterpret_cast<float4*>(U + i * n + j) = make_float4(o[0], o[1], o[2], o[3]);
    if (U_lo)
      *reinterpret_cast<float4*>(U_lo + i * n + j) =
          make_float4(tf32_lo(o[0]), tf32_lo(o[1]), tf32_lo(o[2]), tf32_lo(o[3]));
  }
}

unsigned grid_1d(int64_t items) {
  const int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

struct Factor {
  int64_t n, h;   // h: pitch (and largest extent) of the scratch squares T and R
  float *A, *G, *G_lo, *Vt, *Vt_lo, *T, *T_lo, *R, *R_lo, *Vd, *Vd_lo;
  GemmMat mG, mVt, mT, mR, mVd, mA;   // operands with their tensor maps, prepared once (mA: A with G_lo as low part)
  int32_t* status;
  cudaStream_t st;
};

int prepare_operands(Factor& f, bool with_cholesky) {
  int rc;
  if ((rc = gemm_mat_init(&f.mG, f.G, f.G_lo, f.n, f.n, f.n)) != LC_OK) return rc;
  if ((rc = gemm_mat_init(&f.mVt, f.Vt, f.Vt_lo, f.n, f.n, f.n)) != LC_OK) return rc;
  if (f.n > kB) {
    if ((rc = gemm_mat_init(&f.mT, f.T, f.T_lo, f.n, f.h, f.h)) != LC_OK) return rc;
    if ((rc = gemm_mat_init(&f.mR, f.R, f.R_lo, f.n, f.h, f.h)) != LC_OK) return rc;
  }
  if (with_cholesky) {
    if ((rc = gemm_mat_init(&f.mVd, f.Vd, f.Vd_lo, f.n, kB, kB)) != LC_OK) return rc;
    if ((rc = gemm_mat_init(&f.mA, f.A, f.G_lo, f.n, f.n, f.n)) != LC_OK) return rc;
  }
  return LC_OK;
}

struct Region {
  const float* x;
  float* lo;
  int64_t rows, cols;
};

int split_regions(const Factor& f, const Region* r, int count, int64_t ld) {
  for (int first = 0; first < count; first += kMaxRegions) {
    const int nb = count - first < kMaxRegions ? count - first : kMaxRegions;
    SplitRegions rg;
    int64_t most = 1;
    for (int i = 0; i < nb; ++i) {
      rg.x[i] = r[first + i].x;
      rg.lo[i] = r[first + i].lo;
      rg.rows[i] = (int)r[first + i].rows;
      rg.cols[i] = (int)r[first + i].cols;
      const int64_t work = r[first + i].rows * (r[first + i].cols >> 2);
      most = work > most ? work : most;
    }
    const dim3 grid(grid_1d(most), (unsigned)nb);
    split_region_kernel<<<grid, 256, 0, f.st>>>(rg, ld);
    LC_LAUNCH_CHECK();
  }
  return LC_OK;
}

int split_region(const Factor& f, const float* x, float* lo, int64_t rows, int64_t cols, int64_t ld) {
  const Region r = {x, lo, rows, cols};
  return split_regions(f, &r, 1, ld);
}

struct Node {
  int64_t lo, h, hi;   // index range [lo, hi) split at h (multiples of 128)
};

// internal nodes of the recursion by depth; a range of one diagonal block is a leaf
void collect_nodes(int64_t lo, int64_t hi, size_t depth, std::vector<std::vector<Node>>& levels) {
  const int64_t len = hi - lo;
  if (len <= kB) return;
  const int64_t h = lo + ((len / kB + 1) / 2) * kB;
  if (levels.size() <= depth) levels.resize(depth + 1);
  levels[depth].push_back({lo, h, hi});
  collect_nodes(lo, h, depth + 1, levels);
  collect_nodes(h, hi, depth + 1, levels);
}

// Vt[hi, lo] = -Vt[hi, hi] (G[lo, hi])^T Vt[lo, lo] for every node of one level: two batched GEMMs, one
// batched transpose, two batched splits.  Scratch: node j uses rows [h_j, hi_j) of T and R (n x f.h each),
// which are disjoint across the nodes of a level.  [c0, c1): column slice of the off-diagonal block
// (whole block: 0, h - lo), only meaningful for a level of one node.
int invert_level(const Factor& f, const std::vector<Node>& nodes, int64_t c0 = 0, int64_t c1 = -1) {
  const int64_t n = f.n, hp = f.h;
  const int count = (int)nodes.size();
  std::vector<GemmItem> g1(count), g2(count);
  std::vector<Region> rt(count), rv(count);
  int rc;
  for (int first = 0; first < count; first += kMaxRegions) {
    const int nb = count - first < kMaxRegions ? count - first : kMaxRegions;
    TransposeBlocks tb;
    int64_t most = 1;
    for (int i = 0; i < nb; ++i) {
      const Node& nd = nodes[first + i];
      const int64_t m2 = nd.hi - nd.h;
      tb.in[i] = f.Vt + nd.h * n + nd.h;
      tb.out[i] = f.R + nd.h * hp;
      tb.out_lo[i] = f.R_lo + nd.h * hp;
      tb.n[i] = (int)m2;
      most = m2 > most ? m2 : most;
    }
    const dim3 grid((unsigned)((most + 31) / 32), (unsigned)((most + 31) / 32), (unsigned)nb);
    transpose_split_kernel<<<grid, 256, 0, f.st>>>(tb, n, hp);
    LC_LAUNCH_CHECK();
  }
  for (int i = 0; i < count; ++i) {
    const Node& nd = nodes[i];
    const int64_t m1 = nd.h - nd.lo, m2 = nd.hi - nd.h;
    const int64_t a = c1 < 0 ? 0 : c0, w = (c1 < 0 ? m1 : c1) - a;
    // T (m2 x m1) = G[lo:h, h:hi]^T Vt[lo:h, lo:h]
    g1[i].C = f.T + nd.h * hp + a;
    g1[i].a_k0 = nd.lo, g1[i].a_m0 = nd.h, g1[i].b_k0 = nd.lo, g1[i].b_n0 = nd.lo + a;
    g1[i].M = m2, g1[i].N = w, g1[i].K = m1, g1[i].b_tri_shift = a;
    rt[i] = {f.T + nd.h * hp + a, f.T_lo + nd.h * hp + a, m2, w};
    // Vt[h:hi, lo:h] = -R^T T, R = Vt[h:hi, h:hi]^T (upper)
    g2[i].C = f.Vt + nd.h * n + nd.lo + a;
    g2[i].a_k0 = nd.h, g2[i].a_m0 = 0, g2[i].b_k0 = nd.h, g2[i].b_n0 = a;
    g2[i].M = m2, g2[i].N = w, g2[i].K = m2;
    rv[i] = {f.Vt + nd.h * n + nd.lo + a, f.Vt_lo + nd.h * n + nd.lo + a, m2, w};
  }
  if ((rc = tf32x3_gemm_batched(f.mG, f.mVt, hp, g1.data(), count, 0, 1.f, kGemmBLower, f.status, f.st)) != LC_OK)
    return rc;
  if ((rc = split_regions(f, rt.data(), count, hp)) != LC_OK) return rc;
  if ((rc = tf32x3_gemm_batched(f.mR, f.mT, n, g2.data(), count, 0, -1.f, kGemmAUpper, f.status, f.st)) != LC_OK)
    return rc;
  return split_regions(f, rv.data(), count, n);
}

// Vt[lo:hi, lo:hi] from its leaves, deepest level first.  skip_root: leave the top node to the caller.
int invert_range(const Factor& f, int64_t lo, int64_t hi, bool skip_root = false) {
  std::vector<std::vector<Node>> levels;
  collect_nodes(lo, hi, 0, levels);
  for (size_t d = levels.size(); d-- > (skip_root ? 1 : 0);) {
    const int rc = invert_level(f, levels[d]);
    if (rc != LC_OK) return rc;
  }
  return LC_OK;
}

constexpr size_t kLeafSmemBytes = kLeafSmemFloats * sizeof(float);
constexpr size_t kPanelSmemBytes = (kB * (kB + 4) + kB * (kPanelCols + 4)) * sizeof(float);
constexpr size_t kStripSmemBytes = 2 * kB * (kStripTile + 4) * sizeof(float);

int factorize(const Factor& f) {
  const int64_t n = f.n;
  int rc;
  LC_CHECK_CUDA(cudaFuncSetAttribute(chol_leaf_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kLeafSmemBytes));
  LC_CHECK_CUDA(cudaFuncSetAttribute(chol_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kPanelSmemBytes));
  LC_CHECK_CUDA(cudaFuncSetAttribute(chol_strip_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kStripSmemBytes));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt, 0, n * n * sizeof(float), f.st));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt_lo, 0, n * n * sizeof(float), f.st));
  for (int64_t o = 0; o < n; o += kOuter) {
    const int64_t o2 = o + kOuter < n ? o + kOuter : n;
    for (int64_t k = o; k < o2; k += kB) {
      const int64_t kk = k * n + k, blk = (k / kB) * kB * kB;
      chol_leaf_kernel<true><<<1, kLeafThreads, kLeafSmemBytes, f.st>>>(
          f.A + kk, n, f.G + kk, f.G_lo + kk, n, f.Vd + blk, f.Vd_lo + blk, f.Vt + kk, f.Vt_lo + kk, n, f.status);
      LC_LAUNCH_CHECK();
      const int64_t k2 = k + kB, right = n - k2;
      if (right == 0) break;
      // G[k:k2, k2:] = V_kk^T A[k:k2, k2:], with its low part
      chol_panel_kernel<<<(unsigned)((right + kPanelCols - 1) / kPanelCols), 256, kPanelSmemBytes, f.st>>>(
          f.Vd + blk, f.A + k * n + k2, n, f.G + k * n + k2, f.G_lo + k * n + k2, n, right);
      LC_LAUNCH_CHECK();
      // eager update of the rest of the outer block's rows
      if (k2 < o2) {
        const dim3 grid((unsigned)((right + kStripTile - 1) / kStripTile), (unsigned)((o2 - k2) / kStripTile));
        chol_strip_kernel<<<grid, 256, kStripSmemBytes, f.st>>>(f.G + k * n, n, f.A, n, k2, o2, n);
        LC_LAUNCH_CHECK();
      }
    }
    if (o2 < n && (rc = tf32x3_gemm_launch(f.A + o2 * n + o2, n, f.mG, o, o2, f.mG, o, o2, n - o2, n - o2, o2 - o, 1,
                                           -1.f, kGemmUpperOnly, f.status, f.st)) != LC_OK)
      return rc;
  }
  return invert_range(f, 0, n);
}

// The top node of the recursion with the off-diagonal block Vt[h:n, 0:h] restricted to columns
// [c0, c1): both children in full, then the two products on that column slice only.  Ranks of a
// process group take different slices and exchange them afterwards.
int invert_top_slice(const Factor& f, int64_t c0, int64_t c1) {
  const int64_t n = f.n;
  if (n <= kB) return LC_OK;
  const int rc = invert_range(f, 0, n, true);
  if (rc != LC_OK || c1 <= c0) return rc;
  const std::vector<Node> root = {{0, ((n / kB + 1) / 2) * kB, n}};
  return invert_level(f, root, c0, c1);
}

// Leaves and low parts common to the whole and the sliced inverse
int invert_prologue(const Factor& f) {
  const int64_t n = f.n;
  int rc;
  LC_CHECK_CUDA(cudaFuncSetAttribute(chol_leaf_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kLeafSmemBytes));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt, 0, n * n * sizeof(float), f.st));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt_lo, 0, n * n * sizeof(float), f.st));
  if ((rc = split_region(f, f.G, f.G_lo, n, n, n)) != LC_OK) return rc;
  chol_leaf_kernel<false><<<(unsigned)(n / kB), kLeafThreads, kLeafSmemBytes, f.st>>>(
      f.G, n, nullptr, nullptr, 0, nullptr, nullptr, f.Vt, f.Vt_lo, n, nullptr);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

// Workspace carve-up of the inverse-only entry points
void carve_inverse(Factor& f, const float* G, int64_t n, float* workspace, int32_t* status, cudaStream_t st) {
  const int64_t h = ((n / 128 + 1) / 2) * 128;
  f.n = n;
  f.h = h;
  f.A = nullptr;
  f.G = const_cast<float*>(G);
  float* p = workspace;
  f.G_lo = p, p += n * n;
  f.Vt = p, p += n * n;
  f.Vt_lo = p, p += n * n;
  f.T = p, p += n * h;
  f.T_lo = p, p += n * h;
  f.R = p, p += n * h;
  f.R_lo = p;
  f.Vd = f.Vd_lo = nullptr;
  f.status = status;
  f.st = st;
}

// Vt = (G^-1)^T for a given upper factor G: all diagonal blocks inverted by one launch, then the
// recursion.
int invert_factor(const Factor& f) {
  const int rc = invert_prologue(f);
  if (rc != LC_OK) return rc;
  return invert_range(f, 0, f.n);
}

}  // namespace
}  // namespace lc

extern "C" LC_API int64_t lc_gptq_factor_workspace_floats(int64_t n) {
  if (n <= 0) return 0;
  const int64_t h = ((n / 128 + 1) / 2) * 128;
  // G, G_lo, Vt, Vt_lo (n^2 each), T, T_lo, R, R_lo (n x h each), V_kk blocks and their low parts
  return 4 * n * n + 4 * n * h + 2 * n * 128;
}

extern "C" LC_API int lc_gptq_factorize(float* A, int64_t n, float* U, float* U_lo, float* workspace,
                                        int64_t workspace_floats, int32_t* status, lc_stream_t stream) {
  using namespace lc;
  if (!A || !U || !workspace || !status || n <= 0) return LC_ERR_ARG;
  if (n % 128 != 0) return LC_ERR_SHAPE;
  if (workspace_floats < lc_gptq_factor_workspace_floats(n)) return LC_ERR_WORKSPACE;
  if (!aligned16(A) || !aligned16(U) || !aligned16(workspace) || (U_lo && !aligned16(U_lo))) return LC_ERR_ALIGN;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  const int64_t h = ((n / 128 + 1) / 2) * 128;
  Factor f;
  f.n = n;
  f.A = A;
  float* p = workspace;
  f.G = p, p += n * n;
  f.G_lo = p, p += n * n;
  f.Vt = p, p += n * n;
  f.Vt_lo = p, p += n * n;
  f.T = p, p += n * h;
  f.T_lo = p, p += n * h;
  f.R = p, p += n * h;
  f.R_lo = p, p += n * h;
  f.Vd = p, p += n * 128;
  f.Vd_lo = p;
  f.status = status;
  f.st = reinterpret_cast<cudaStream_t>(stream);
  f.h = h;
  int rc = prepare_operands(f, true);
  if (rc != LC_OK) return rc;
  rc = factorize(f);
  if (rc != LC_OK) return rc;
  flip_upper_kernel<<<grid_1d(n * (n >> 2)), 256, 0, f.st>>>(f.Vt, n, U, U_lo);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int lc_gptq_invert_factor(const float* G, int64_t n, float* U, float* U_lo, float* workspace,
                                            int64_t workspace_floats, int32_t* status, lc_stream_t stream) {
  using namespace lc;
  if (!G || !U || !workspace || !status || n <= 0) return LC_ERR_ARG;
  if (n % 128 != 0) return LC_ERR_SHAPE;
  if (workspace_floats < lc_gptq_factor_workspace_floats(n)) return LC_ERR_WORKSPACE;
  if (!aligned16(G) || !aligned16(U) || !aligned16(workspace) || (U_lo && !aligned16(U_lo))) return LC_ERR_ALIGN;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  Factor f;
  carve_inverse(f, G, n, workspace, status, reinterpret_cast<cudaStream_t>(stream));
  int rc = prepare_operands(f, false);
  if (rc != LC_OK) return rc;
  rc = invert_factor(f);
  if (rc != LC_OK) return rc;
  flip_upper_kernel<<<grid_1d(n * (n >> 2)), 256, 0, f.st>>>(f.Vt, n, U, U_lo);
  LC_LAUNCH_CHECK();
  return LC_OK;
}

extern "C" LC_API int64_t lc_gptq_factor_split(int64_t n) { return n <= 128 ? n : ((n / 128 + 1) / 2) * 128; }

extern "C" LC_API int64_t lc_gptq_factor_vt_offset(int64_t n) { return n * n; }

extern "C" LC_API int lc_gptq_invert_factor_part(const float* G, int64_t n, float* workspace,
                                                 int64_t workspace_floats, int64_t col_begin, int64_t col_end,
                                                 int32_t* status, lc_stream_t stream) {
  using namespace lc;
  if (!G || !workspace || !status || n <= 0) return LC_ERR_ARG;
  if (n % 128 != 0 || n <= 128) return LC_ERR_SHAPE;
  const int64_t h = lc_gptq_factor_split(n);
  if (col_begin < 0 || col_end < col_begin || col_end > h || col_begin % 128 != 0 || col_end % 128 != 0)
    return LC_ERR_ARG;
  if (workspace_floats < lc_gptq_factor_workspace_floats(n)) return LC_ERR_WORKSPACE;
  if (!aligned16(G) || !aligned16(workspace)) return LC_ERR_ALIGN;
  int dev = 0, major = 0;
  LC_CHECK_CUDA(cudaGetDevice(&dev));
  LC_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LC_ERR_ARCH;
  Factor f;
  carve_inverse(f, G, n, workspace, status, reinterpret_cast<cudaStream_t>(stream));
  int rc = prepare_operands(f, false);
  if (rc != LC_OK) return rc;
  if ((rc = invert_prologue(f)) != LC_OK) return rc;
  return invert_top_slice(f, col_begin, col_end);
}

extern "C" LC_API int lc_gptq_invert_factor_finish(int64_t n, const float* workspace, int64_t workspace_floats,
                                                   float* U, float* U_lo, lc_stream_t stream) {
  using namespace lc;
  if (!workspace || !U || n <= 0) return LC_ERR_ARG;
  if (n % 128 != 0) return LC_ERR_SHAPE;
  if (workspace_floats < lc_gptq_factor_workspace_floats(n)) return LC_ERR_WORKSPACE;
  if (!aligned16(workspace) || !aligned16(U) || (U_lo && !aligned16(U_lo))) return LC_ERR_ALIGN;
  flip_upper_kernel<<<grid_1d(n * (n >> 2)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      workspace + lc_gptq_factor_vt_offset(n), n, U, U_lo);
  LC_LAUNCH_CHECK();
  return LC_OK;
}
