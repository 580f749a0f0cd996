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
constexpr int kLd = kB + 1;        // padded shared-memory pitch

__device__ __forceinline__ float tf32_lo(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// One CTA: Cholesky of the 128x128 block at A (pitch lda, upper triangle read) and the inverse of
// its factor.  Writes G_kk (upper; the lower part of the block is zeroed) and its low part, V_kk =
// G_kk^-1 (upper, dense 128x128 block in `v` / `v_lo`), and Vt_kk = V_kk^T with its low part into the
// lower-triangular result.
//
// The block lives in registers: 256 threads as a 16 x 16 grid, thread (ty, tx) holding the 8 x 8
// elements (ty + 16a, tx + 16b).  Each of the 128 steps of the right-looking Cholesky broadcasts one
// scaled row through shared memory (double-buffered, one barrier per step) and applies the rank-1
// update to the register tiles; the pivots are tracked redundantly by the 16 threads that own a row,
// so that no second barrier is needed.  The inverse is a Gauss-Jordan elimination of [G | I] from the
// bottom row up with the same communication pattern (column j of G and row j of the right-hand side
// per step).  The loops over the 16-row bands are unrolled, which keeps every register index static.
//
// kCholesky = false: A already holds the factor G_kk (upper); only the inverse is computed and only Vt /
// Vt_lo are written.  One CTA per diagonal block (blockIdx.x), all blocks of a matrix in one launch.
template <bool kCholesky>
__global__ void __launch_bounds__(kLeafThreads, 1) chol_leaf_kernel(const float* __restrict__ A, int64_t lda,
                                                                     float* __restrict__ G, float* __restrict__ G_lo,
                                                                     int64_t ldg, float* __restrict__ v,
                                                                     float* __restrict__ v_lo, float* __restrict__ Vt,
                                                                     float* __restrict__ Vt_lo, int64_t ldv,
                                                                     int32_t* status) {
  extern __shared__ float stage[];          // [128][129]: staging for the transposed store
  __shared__ float rowbuf[2][kB], colbuf[2][kB];
  __shared__ int s_bad;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  if (tid == 0) s_bad = 0;
  if (!kCholesky) {
    // block b of the diagonal
    A += (int64_t)blockIdx.x * kB * (lda + 1);
    Vt += (int64_t)blockIdx.x * kB * (ldv + 1);
    Vt_lo += (int64_t)blockIdx.x * kB * (ldv + 1);
  }

  float t[8][8], pd[8], dg[8];
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int r = ty + 16 * a;
#pragma unroll
    for (int b = 0; b < 8; ++b) t[a][b] = A[(int64_t)r * lda + tx + 16 * b];
    pd[a] = A[(int64_t)r * lda + r];
    dg[a] = kCholesky ? 1.f : pd[a];
  }
  __syncthreads();

  // ---- Cholesky: A = G^T G ----
#pragma unroll
  for (int jb = 0; jb < (kCholesky ? 8 : 0); ++jb) {
#pragma unroll 1
    for (int jj = 0; jj < 16; ++jj) {
      const int j = 16 * jb + jj, buf = j & 1;
      if (ty == jj) {
        const float p = pd[jb];
        const float d = sqrtf(p), dinv = __frcp_rn(d);
        if (tx == 0 && (!(p > 0.f) || !(p < INFINITY))) s_bad = 1;
        dg[jb] = d;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int c = tx + 16 * b;
          float x = t[jb][b];
          if (c == j) {
            x = d;
          } else if (c > j) {
            // IEEE quotient through the reciprocal and one residual correction
            const float q0 = x * dinv;
            x = fmaf(fmaf(-q0, d, x), dinv, q0);
          }
          t[jb][b] = x;
          rowbuf[buf][c] = x;
        }
      }
      __syncthreads();
      float gr[8], gc[8];
#pragma unroll
      for (int a = jb; a < 8; ++a) gr[a] = rowbuf[buf][ty + 16 * a];
#pragma unroll
      for (int b = jb; b < 8; ++b) gc[b] = rowbuf[buf][tx + 16 * b];
#pragma unroll
      for (int a = jb; a < 8; ++a) {
        if (a > jb || ty > jj) {
#pragma unroll
          for (int b = jb; b < 8; ++b) t[a][b] = fmaf(-gr[a], gc[b], t[a][b]);
          pd[a] = fmaf(-gr[a], gr[a], pd[a]);
        }
      }
    }
  }

  // ---- inverse: Gauss-Jordan on [G | I], bottom row first ----
  __syncthreads();   // the last row buffer of the Cholesky loop is about to be reused
  float w[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) w[a][b] = (ty + 16 * a == tx + 16 * b) ? 1.f : 0.f;
#pragma unroll
  for (int jb = 7; jb >= 0; --jb) {
#pragma unroll 1
    for (int jj = 15; jj >= 0; --jj) {
      const int j = 16 * jb + jj, buf = j & 1;
      if (ty == jj) {
        const float d = dg[jb];
#pragma unroll
        for (int b = jb; b < 8; ++b) {
          w[jb][b] = __fdiv_rn(w[jb][b], d);
          rowbuf[buf][tx + 16 * b] = w[jb][b];
        }
      }
      if (tx == jj) {
#pragma unroll
        for (int a = 0; a <= jb; ++a) colbuf[buf][ty + 16 * a] = t[a][jb];
      }
      __syncthreads();
      float cr[8], rw[8];
#pragma unroll
      for (int a = 0; a <= jb; ++a) cr[a] = colbuf[buf][ty + 16 * a];
#pragma unroll
      for (int b = jb; b < 8; ++b) rw[b] = rowbuf[buf][tx + 16 * b];
#pragma unroll
      for (int a = 0; a <= jb; ++a) {
        if (a < jb || ty < jj) {
#pragma unroll
          for (int b = jb; b < 8; ++b) w[a][b] = fmaf(-cr[a], rw[b], w[a][b]);
        }
      }
    }
  }

  // ---- stores ----
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int r = ty + 16 * a;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int c = tx + 16 * b;
      const float gv = (c >= r) ? t[a][b] : 0.f;
      const float wv = (c >= r) ? w[a][b] : 0.f;
      if (kCholesky) {
        G[(int64_t)r * ldg + c] = gv;
        G_lo[(int64_t)r * ldg + c] = tf32_lo(gv);
        v[r * kB + c] = wv;
        v_lo[r * kB + c] = tf32_lo(wv);
      }
      stage[c * kLd + r] = wv;           // transposed
    }
  }
  __syncthreads();
  for (int idx = tid; idx < kB * kB; idx += kLeafThreads) {
    const int i = idx >> 7, jcol = idx & 127;
    const float wt = stage[i * kLd + jcol];
    Vt[(int64_t)i * ldv + jcol] = wt;
    Vt_lo[(int64_t)i * ldv + jcol] = tf32_lo(wt);
  }
  if (tid == 0 && s_bad && status) atomicCAS(status, 0, (int)LC_ERR_NOT_PD);
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

int factorize(const Factor& f) {
  const int64_t n = f.n;
  int rc;
  LC_CHECK_CUDA(cudaFuncSetAttribute(chol_leaf_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kB * kLd * (int)sizeof(float)));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt, 0, n * n * sizeof(float), f.st));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt_lo, 0, n * n * sizeof(float), f.st));
  for (int64_t o = 0; o < n; o += kOuter) {
    const int64_t o2 = o + kOuter < n ? o + kOuter : n;
    for (int64_t k = o; k < o2; k += kB) {
      const int64_t kk = k * n + k, blk = (k / kB) * kB * kB;
      chol_leaf_kernel<true><<<1, kLeafThreads, kB * kLd * sizeof(float), f.st>>>(
          f.A + kk, n, f.G + kk, f.G_lo + kk, n, f.Vd + blk, f.Vd_lo + blk, f.Vt + kk, f.Vt_lo + kk, n, f.status);
      LC_LAUNCH_CHECK();
      const int64_t k2 = k + kB, right = n - k2;
      if (right == 0) break;
      // G[k:k2, k2:] = V_kk^T A[k:k2, k2:]; the low part of the A panel borrows the place of the result's
      if ((rc = split_region(f, f.A + k * n + k2, f.G_lo + k * n + k2, kB, right, n)) != LC_OK) return rc;
      if ((rc = tf32x3_gemm_launch(f.G + k * n + k2, n, f.mVd, k, 0, f.mA, k, k2, kB, right, kB, 0, 1.f, kGemmAUpper,
                                   f.status, f.st)) != LC_OK)
        return rc;
      if ((rc = split_region(f, f.G + k * n + k2, f.G_lo + k * n + k2, kB, right, n)) != LC_OK) return rc;
      // eager update of the rest of the outer block's rows
      if (k2 < o2 && (rc = tf32x3_gemm_launch(f.A + k2 * n + k2, n, f.mG, k, k2, f.mG, k, k2, o2 - k2, right, kB, 1,
                                              -1.f, kGemmUpperOnly, f.status, f.st)) != LC_OK)
        return rc;
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
                                     kB * kLd * (int)sizeof(float)));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt, 0, n * n * sizeof(float), f.st));
  LC_CHECK_CUDA(cudaMemsetAsync(f.Vt_lo, 0, n * n * sizeof(float), f.st));
  if ((rc = split_region(f, f.G, f.G_lo, n, n, n)) != LC_OK) return rc;
  chol_leaf_kernel<false><<<(unsigned)(n / kB), kLeafThreads, kB * kLd * sizeof(float), f.st>>>(
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
