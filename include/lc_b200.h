/*
 * lc_b200.h -- C ABI of the B200 (sm_100a) kernels behind LightCompress's
 * calibration-time quantization plugins (RTN / GPTQ / AWQ, IntegerQuantizer /
 * FloatQuantizer).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *   - Nothing here allocates or frees memory: the caller passes every output and
 *     every scratch buffer.
 *   - Every function enqueues its work on `stream` and returns without
 *     synchronising.  The int result is a host-side status (argument, shape and
 *     alignment validation, launch errors).  Failures that only the device can
 *     see (a bounded wait that expired) are written to the optional `int32_t*
 *     status` word and must be read after the stream is synchronised.
 *   - Matrices are row-major and contiguous.  "rows x cols" weights follow
 *     torch.nn.Linear: rows = out_features, cols = in_features; quantization
 *     groups run along cols.
 *   - Reference citations are paths inside the LightCompress source tree.
 */
#ifndef LC_B200_H_
#define LC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* lc_stream_t; /* a cudaStream_t / CUstream handle; NULL = legacy default stream */

enum lc_status_code {
  LC_OK = 0,
  LC_ERR_ARG = -1,       /* null pointer / unknown enum / unsupported combination */
  LC_ERR_SHAPE = -2,     /* sizes that the reference itself rejects (e.g. cols % group != 0) */
  LC_ERR_ALIGN = -3,     /* pointer or row pitch not aligned as the kernel requires */
  LC_ERR_ARCH = -4,      /* device is not sm_100 */
  LC_ERR_WORKSPACE = -5, /* scratch buffer too small */
  LC_ERR_NOT_PD = -6,    /* matrix not positive definite */
  LC_ERR_TIMEOUT = -7,   /* device-side bounded wait expired (reported through *status) */
  LC_ERR_CUDA = -8       /* CUDA runtime / driver error */
};

enum lc_dtype { LC_F32 = 0, LC_BF16 = 1, LC_F16 = 2 };

/* How integer codes are written by lc_rtn_int_quant. */
enum lc_code_fmt {
  LC_CODES_NONE = 0,
  LC_CODES_I32 = 1,  /* one int32 per element: dtype of IntegerQuantizer.real_quant_weight_* for bit != 8 */
  LC_CODES_I8 = 2,   /* one byte per element (int8 if symmetric, uint8 otherwise): the bit == 8 dtype */
  LC_CODES_PACK4 = 3 /* bits == 4 only: two codes per byte along cols, low nibble first, stored as q - qmin */
};

int lc_version(void);
const char* lc_status_string(int status);

/* Makes `device` current for the calling thread inside this library's CUDA runtime. */
int lc_set_device(int device);

/* ------------------------------------------------------------------------------------------
 * Family 1: integer quant / dequant in one pass over HBM.
 *
 * Replaces IntegerQuantizer.get_tensor_qparams, quant, dequant, quant_dequant,
 * fake_quant_weight_dynamic / _static, fake_quant_act_dynamic and real_quant_weight_dynamic
 * (llmc/compression/quantization/quant.py:689-716, :753-868, :915-952) for calib_algo
 * 'minmax', round_zp = True, granularity per_group / per_channel / per_token.
 *
 *   in         rows x cols, element type `dtype`
 *   group      quantization group length along cols; 0 = the whole row (per_channel/per_token)
 *   bits, sym  integer width (2..8) and symmetric flag; the code range is the reference's
 *              (quant.py:664-676): sym -> [-2^(b-1), 2^(b-1)-1], asym -> [0, 2^b-1]
 *   scales_in, zeros_in
 *              NULL = dynamic (min/max computed here).  Non-NULL = static: one value per
 *              group in `dtype`, laid out (rows * cols/group); zeros_in may be NULL when sym.
 *   fake_out   rows x cols dequantised values in `dtype`, or NULL
 *   codes_out  integer codes in the layout `code_fmt` names, or NULL with LC_CODES_NONE
 *   scales_out, zeros_out
 *              per-group scale / zero point in `dtype` (zero point is an integer held in a
 *              float, as get_qparams returns it), or NULL
 *
 * Arithmetic is the reference's, op for op, in `dtype` (IEEE divide, round-half-even, a
 * rounding to `dtype` after every torch-level op), so codes, scales, zeros and dequantised
 * values are bit-identical to the reference's.
 * ------------------------------------------------------------------------------------------ */
int lc_rtn_int_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group,
                     int bits, int sym, const void* scales_in, const void* zeros_in,
                     void* fake_out, void* codes_out, int code_fmt, void* scales_out,
                     void* zeros_out, lc_stream_t stream);

/* QUIK's activation statistic (get_tensor_scale, llmc/compression/quantization/quik.py:35-42):
 * running[c] = max(running[c], max over tokens of |x[t][c]|), fp32 on the device (the reference keeps
 * it on the host); start from zeros.  x: tokens x cols of `dtype`, cols a multiple of 8 (4 for fp32).
 * NaN sticks, like torch.max. */
int lc_quik_col_absmax(const void* x, int dtype, int64_t tokens, int64_t cols, float* running,
                       lc_stream_t stream);

/* IntegerQuantizer.fake_quant_weight_dynamic / fake_quant_act_dynamic with args['int_indices'] and
 * args['fp_indices'] (quant.py:753-782, :832-868; used by QUIK.w_qdq / a_qdq, quik.py:128-151) for
 * per_channel / per_token granularity: each row is quantised over its integer columns only, the
 * floating-point columns pass through.  col_mask holds one byte per column (8-byte aligned):
 * 0 = quantise, 1 = keep, 2 = write zero (a column in neither index list, as the reference's
 * zeros_like + two scatters leave it).  cols a multiple of 8 (4 for fp32), at most 32768 (16384).
 * Bit-identical to the reference's gather -> quant_dequant -> scatter chain. */
int lc_rtn_int_fake_quant_masked(const void* in, int dtype, int64_t rows, int64_t cols, int bits, int sym,
                                 const uint8_t* col_mask, void* out, lc_stream_t stream);

/* One level of Weight48IntegerQuantizer (llmc/compression/quantization/quant.py:1232-1287): the code
 * range (from `symmetric` or `int_range`), and the clamps get_qparams applies to the scale and the
 * zero point (quant.py:1318-1323): [scales_qmin, scales_qmax] from scales_bit / scales_symmetric, else
 * -inf .. inf; [zeros_qmin, zeros_qmax] from zeros_bit / zeros_symmetric, else [qmin, qmax]. */
typedef struct {
  float qmin, qmax;
  int symmetric;
  float scales_min, scales_max;
  float zeros_min, zeros_max;
} lc_w48_level;

/* Weight48IntegerQuantizer.fake_quant_weight_dynamic (quant.py:1338-1367) in one pass: quantise each
 * row with the bit8 level (per_channel), quantise those codes per `group` elements with the bit4 level
 * (per_group), dequantise back through both.  in / out: rows x cols of `dtype`; bit-identical to the
 * reference's op chain in that dtype.  cols % group == 0 (the reference raises otherwise); group a
 * multiple of 8 (4 for fp32) with group / 8 (group / 4) a power of two <= 32, e.g. 128; cols <= 32768
 * (16384 for fp32). */
int lc_rtn_w48_fake_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group,
                          const lc_w48_level* bit8, const lc_w48_level* bit4, void* out, lc_stream_t stream);

/* GPTQ.w_qdq (gptq.py:425-452: weight[:, perm] -> static fake quant -> [:, invperm] -> model dtype) from
 * the codes lc_gptq_weight_transform* already produced, in one pass: out[r][c] = ((codes[r][j] + qmin) -
 * zeros[r][j / 128]) * scales[r][j / 128], j = invperm[c] (invperm NULL: identity), rounded once to
 * out_dtype.  codes: rows x cols bytes in the permuted column order, stored as q - qmin; scales / zeros:
 * (rows * ceil(cols / 128)) fp32 in the permuted-group order the solver writes (zeros NULL when
 * symmetric).  The same bits as the reference's chain, because re-quantising a kept weight with the
 * parameters it was quantised with reproduces its code. */
int lc_gptq_dequant_unpermute(const uint8_t* codes, const float* scales, const float* zeros, const int64_t* invperm,
                              int64_t rows, int64_t cols, int bits, int sym, void* out, int out_dtype,
                              lc_stream_t stream);

/* Per-tensor ranges of a batch of calibration activations (static activation quantisation:
 * BaseQuantizer.get_minmax_range with granularity 'per_tensor' inside get_minmax_stats and
 * get_static_moving_minmax_range, llmc/compression/quantization/quant.py:134-137, :223-250, :523-542).
 *   tensors, numels  HOST arrays of `count` device pointers (contiguous tensors of `dtype`) and their
 *                    element counts (> 0: the reference's torch.max raises on an empty tensor)
 *   min_out, max_out count fp32 values each (exact: every `dtype` value is an fp32 value); NaN
 *                    propagates like torch.max / torch.min
 * Every tensor is read once, all of them by one launch per 64 tensors. */
int lc_act_range_per_tensor(const void* const* tensors, const int64_t* numels, int count, int dtype,
                            float* min_out, float* max_out, lc_stream_t stream);

/* 2048-bin (any `bins` <= 4096) histograms of a batch of calibration tensors, tensor i over its own range
 * [mins[i], maxs[i]] (device fp32 arrays) -- the torch.histc(tensor.float(), bins, min, max) calls of
 * BaseQuantizer.get_static_hist_range (quant.py:461-521), one launch for the whole batch.  Binning as
 * torch.histc on CUDA: values outside the range (and NaN) are not counted, bin = (int)((x - min) * bins /
 * (max - min)) in fp32, x == max falls into the last bin.  hist: count x bins fp32, overwritten. */
int lc_act_hist_per_tensor(const void* const* tensors, const int64_t* numels, int count, int dtype,
                           const float* mins, const float* maxs, int bins, float* hist, lc_stream_t stream);

/* The moving average of get_static_moving_minmax_range (quant.py:534-538) over the `count` per-tensor
 * values above, in order: m = v[0]; m = m + alpha * (v[i] - m), every op rounded to `dtype` as the
 * reference's 0-dim tensor arithmetic does.  out2[0] = moving min, out2[1] = moving max (fp32 holding
 * `dtype` values). */
int lc_act_range_moving(const float* mins, const float* maxs, int count, int dtype, double alpha,
                        float* out2, lc_stream_t stream);

/* MSE range search (calib_algo 'mse'): BaseQuantizer.get_mse_range with the integer quantizer's
 * get_qparams and quant_dequant inside its loop (llmc/compression/quantization/quant.py:147-205,
 * :544-558, :698-716).  For each group of `group` elements along cols (0 = the whole row) the range
 * [min, max] of the group is shrunk by p = 1 - i / mse_grid for i < int(maxshrink * mse_grid), always
 * from the best range found so far (the reference shrinks in place through views), and the range
 * with the smallest sum |qdq(x) - x|^norm (strict <) is written to min_out / max_out (fp32, one value
 * per group: the reference converts the tensor with .float() first).  Reference defaults:
 * maxshrink 0.8, mse_grid 100, norm 2.4.  Group lengths: 128, 256, 512, 1024, 2048. */
int lc_rtn_mse_range(const void* in, int dtype, int64_t rows, int64_t cols, int64_t group, int bits, int sym,
                     double maxshrink, int mse_grid, float norm, float* min_out, float* max_out,
                     lc_stream_t stream);

/* FP8 e4m3 per-row (per_channel weights / per_token activations) quant / dequant.
 * Replaces FloatQuantizer.get_tensor_qparams, quant, dequant, fake_quant_weight_dynamic,
 * fake_quant_act_dynamic and real_quant_weight_dynamic with use_qtorch (quant.py:1042-1080,
 * :1099-1108, :1141-1158, :1194-1220).  The third-party qtorch.float_quantize call
 * (quant.py:1065) is evaluated as round-to-nearest-even onto float8_e4m3fn.
 *   fake_out  rows x cols in `dtype`, or NULL;  codes_out  rows x cols e4m3 bytes, or NULL
 *   scales_out rows values in `dtype`, or NULL */
int lc_fp8_e4m3_quant(const void* in, int dtype, int64_t rows, int64_t cols, void* fake_out,
                      void* codes_out, void* scales_out, lc_stream_t stream);

/* FP8 e4m3 block-wise weights: one fp32 scale per 128 x 128 block (FloatQuantizer with granularity
 * 'per_block', llmc/compression/quantization/quant.py:637-641, :138-140, :544-551, :1060-1075, :1194-1220,
 * and weight_cast_to_fp8 / weight_cast_to_bf16, quant.py:20-45; the reference's Triton kernels for the
 * same two casts are kernel.py:56-131).  Ragged edge blocks are padded with zeros like the reference's
 * reshape.  in: rows x cols in `dtype`; fake_out (same dtype), codes_out (one e4m3 byte per element) and
 * scales_out (fp32, ceil(rows/128) x ceil(cols/128)) may each be NULL.  block must be 128. */
int lc_fp8_e4m3_block_quant(const void* in, int dtype, int64_t rows, int64_t cols, int64_t block, void* fake_out,
                            void* codes_out, float* scales_out, lc_stream_t stream);

/* The same cast with the arithmetic of the reference's Triton kernel weight_cast_to_fp8 (kernel.py:56-83), which
 * the reference binds instead of its torch helper on GPUs with FP8 support (base_blockwise_quantization.py:22-27):
 * scale = max|x| * fl(1/448) in fp32 (what its `/ 448.` compiles to) and no floor on the scale.  Bit-identical to
 * that kernel's codes and scales on a B200. */
int lc_fp8_e4m3_block_quant_triton(const void* in, int dtype, int64_t rows, int64_t cols, int64_t block, void* fake_out,
                            void* codes_out, float* scales_out, lc_stream_t stream);
/* out[r][c] = e4m3 value of codes[r][c] * scales[r/128][c/128], rounded once to out_dtype. */
int lc_fp8_e4m3_block_dequant(const void* codes, const float* scales, int64_t rows, int64_t cols, int64_t block,
                              void* out, int out_dtype, lc_stream_t stream);

/* The block-wise FP8 linear's forward (block_wise_fp8_forward_func, module_utils.py:41-46), the
 * reference's Triton kernels act_quant (kernel.py:7-53) and fp8_gemm (kernel.py:153-242):
 *   act_quant: per group of 128 values along the last dimension, scales[g] = max|x| * fl(1/448) (fp32, no
 *              floor: what the Triton kernel's `/ 448.0` computes; bit-identical to its scales and codes on a
 *              B200), y = e4m3(x / scales[g]); n = number of elements, a multiple of 128.
 *   gemm:      c[M][N] = sum over 128-wide k blocks kb of (a[:, kb] b[:, kb]^T) * (a_s[m][kb] *
 *              b_s[n / 128][kb]); a: M x K e4m3 (row-major), a_s: M x K/128 fp32; b: N x K e4m3, b_s:
 *              ceil(N/128) x K/128 fp32; c: bf16 or fp32.  K % 128 == 0.  tcgen05 kind::f8f6f4, each k
 *              block accumulated on its own in tensor memory and folded into fp32 registers with its
 *              scales.  *status receives LC_ERR_TIMEOUT if a bounded pipeline wait expires. */
int lc_fp8_e4m3_act_quant(const void* x, int dtype, int64_t n, int64_t group, void* y, float* scales,
                          lc_stream_t stream);
int lc_fp8_block_gemm(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                      int64_t K, void* c, int out_dtype, int32_t* status, lc_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Family 2: Hessian accumulation on the tcgen05 tensor cores.
 *
 * Replaces the matmul of GPTQ.add_batch (llmc/compression/quantization/gptq.py:283-290):
 *     H <- beta * H + alpha * X^T X
 *   X  tokens x cols, bf16, row-major (tokens of all sequences of the batch, flattened)
 *   H  cols x cols fp32, full symmetric matrix is maintained
 * cols must be a multiple of 8 (16-byte row pitch for TMA); X and H 16-byte aligned.
 * Products of bf16 values are exact in fp32; accumulation is fp32 in tensor memory.
 * Only 256x256 tiles on or above the diagonal are computed; each is added to H and to its
 * mirror with fp32 atomic adds.  `ksplit` > 1 splits the token range over that many work items
 * per tile (0 = choose); the order in which partial sums reach H may then vary between runs.
 * `status` (may be NULL) receives LC_ERR_TIMEOUT if a bounded pipeline wait expires.
 * ------------------------------------------------------------------------------------------ */
int lc_hessian_accum(const void* x_bf16, int64_t tokens, int64_t cols, float* H, float alpha,
                     float beta, int ksplit, int32_t* status, lc_stream_t stream);

/* Same update over up to 8 separate activation tensors in one launch,
 *     H <- beta * H + alpha * sum_s X_s^T X_s,
 * so that a caller whose forward hook delivers one sequence at a time (GPTQ.cache_input_hook,
 * gptq.py:247-251) can hand over several of them at once: the accumulators then stay in tensor
 * memory across all of them and H is updated once.  xs_host / tokens_host are HOST arrays of
 * `nseg` device pointers / token counts (each X_s is tokens_s x cols bf16, 16-byte aligned). */
int lc_hessian_accum_multi(const void* const* xs_host, const int64_t* tokens_host, int nseg,
                           int64_t cols, float* H, float alpha, float beta, int ksplit,
                           int32_t* status, lc_stream_t stream);

/* lc_hessian_accum_multi maintaining only the upper triangle of H (entries H[m][n] with n >= m; what
 * lies below the diagonal is left as it is and means nothing).  The mirrored atomic adds are half of the
 * epilogue's work, and the GPTQ solver reads the Hessian through lc_gptq_diag and lc_gptq_permute_damp
 * only, which can fetch entry (i, j) from the upper triangle (flag LC_H_UPPER there).  This is the form
 * GPTQ.add_batch's replacement uses (gptq.py:283-290 computes the full product).
 *
 * Accuracy (all three entry points): the tensor core adds every 16-token MMA into its fp32 accumulator
 * with truncation, so a sum over t tokens carries a relative deficit of about t / 16 * 2^-24, nearly but
 * not exactly uniform over the matrix.  With ksplit = 0 a launch's tokens are cut into equal parts of at
 * most 4096 per accumulation (parts are combined by fp32 atomic adds), which keeps the deficit below
 * 1.5e-5 and what remains after a uniform factor is taken out near 1e-6. */
int lc_hessian_accum_upper(const void* const* xs_host, const int64_t* tokens_host, int nseg,
                           int64_t cols, float* H, float alpha, float beta, int ksplit,
                           int32_t* status, lc_stream_t stream);

/* Exercises the bounded-wait path of the tensor-core kernels without touching them: a one-thread
 * kernel waits (about a millisecond) on a barrier nothing arrives on and must write LC_ERR_TIMEOUT
 * to *status and return normally.  (No counterpart in the reference.) */
int lc_selftest_wait_expiry(int32_t* status, lc_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Family 3: GPTQ layer solver pieces.
 * ------------------------------------------------------------------------------------------ */

/* diag_out[i] = H[i][i].  Feeds GPTQ.hessian_sorting's argsort (gptq.py:58-64). */
int lc_gptq_diag(const float* H, int64_t cols, float* diag_out, lc_stream_t stream);

/* The gather + dampening part of GPTQ.process_hessian_and_weights (gptq.py:135-170):
 *   Wp[r][j] = dead(perm[j]) ? 0 : float(W[r][perm[j]])
 *   Hp[i][j] = hscale * H[perm[i]][perm[j]]   (dead diagonal -> 1), then Hp[i][i] += damp
 * where dead(c) means H[c][c] == 0 and damp = percdamp * mean(diag(Hp)).  `hscale` lets the
 * caller keep H as the raw sum of X^T X and apply 2/nsamples here.
 *   W rows x cols in `w_dtype`; perm int64 (cols) or NULL for identity
 *   reverse_h: bit 0 (LC_H_REVERSE): Hp is written with both index orders reversed, Hp[i][j] <- entry
 *           (cols-1-i, cols-1-j), which is the input of the single-factorisation route to the
 *           upper factor of the inverse (see lc_gptq_flip); Wp is not affected.
 *           bit 1 (LC_H_UPPER): only the upper triangle of H is valid (lc_hessian_accum_upper); entry
 *           (i, j) is read from H[min(i,j)][max(i,j)].  Hp is a full symmetric matrix either way
 *           bit 2 (LC_H_LATE_DEAD): SpQR's order of operations (llmc/compression/quantization/spqr.py:143-149):
 *           damp = percdamp * mean|diag| with the dead columns counted as 0, and a dead column's diagonal
 *           becomes exactly 1 instead of 1 + damp
 *   scratch: at least 1 float (receives damp)
 * W/Wp may both be NULL (only the Hessian part runs: one factorisation serves every linear that
 * shares the input) and Hp may be NULL (only the weight gather runs). */
#define LC_H_REVERSE 1
#define LC_H_UPPER 2
#define LC_H_LATE_DEAD 4
int lc_gptq_permute_damp(const void* W, int w_dtype, const float* H, const int64_t* perm,
                         int64_t rows, int64_t cols, float hscale, float percdamp, int reverse_h,
                         float* Wp, float* Hp, float* scratch, lc_stream_t stream);

/* out[i][j] = in[n-1-i][n-1-j] (out-of-place).  With J the index reversal: if J H J = M M^T
 * (M lower Cholesky factor) then U = J M^-1 J is upper triangular with U^T U = H^-1, i.e. the
 * matrix that gptq.py:172-174 obtains with cholesky -> cholesky_inverse -> cholesky(upper). */
int lc_gptq_flip(const float* in, int64_t n, float* out, lc_stream_t stream);

/* One 128-column block of GPTQ.weight_transform (gptq.py:199-241), group_size == blocksize:
 * per row, asymmetric/symmetric int qparams from the block's current columns
 * (search_column_qparams, gptq.py:359-366), then for each column quantise, keep the
 * pre-quantisation value, propagate err * U[i][j] to the columns j > i of the block.
 *   W       rows x cols fp32 (permuted order), updated in place: on return columns
 *           [col0, col0+count) hold the kept ("tmp") values
 *   U       cols x cols fp32 upper Cholesky factor of the damped inverse Hessian
 *   err_out rows x 128 fp32: (w - q) / U[i][i] per column (zero for columns >= count)
 *   scales, zeros  (rows * n_groups) fp32 in the reference's merged layout
 *           (update_model_qparams, gptq.py:398-409): index r * n_groups + block
 *   codes_u8 rows x cols bytes (q - qmin), permuted order, or NULL
 *   loss_rows rows fp32, += sum over the block of (w-q)^2 / (2 U_ii^2), or NULL */
int lc_gptq_block_quant(float* W, const float* U, int64_t rows, int64_t cols, int64_t col0,
                        int count, int bits, int sym, float* err_out, float* scales,
                        float* zeros, int64_t n_groups, uint8_t* codes_u8, float* loss_rows,
                        lc_stream_t stream);

/* Trailing update of GPTQ.weight_transform (gptq.py:244):
 *   W[:, col1:] -= Err[:, :k] * U[col0:col0+k, col1:]      (fp32, K = k <= 128) */
int lc_gptq_trailing_update(float* W, const float* err, const float* U, int64_t rows,
                            int64_t cols, int64_t col0, int k, int64_t col1,
                            lc_stream_t stream);

/* Whole GPTQ.weight_transform loop (gptq.py:199-244): alternates the two kernels above on
 * `stream` without host synchronisation.  scratch_err: rows x 128 fp32. */
int lc_gptq_weight_transform(float* W, const float* U, int64_t rows, int64_t cols, int bits,
                             int sym, float* scratch_err, float* scales, float* zeros,
                             uint8_t* codes_u8, float* loss_rows, lc_stream_t stream);

/* lo[i] = x[i] - tf32_truncate(x[i]) (the part of an fp32 value a kind::tf32 tensor-core operand
 * drops).  Used once per factor U by the tensor-core variant below. */
int lc_gptq_split_tf32(const float* x, int64_t n, float* lo, lc_stream_t stream);

/* One per-panel trailing update on the tensor cores:
 *     W[:, p2:] -= E^T * U[p1:p2, p2:]        (E stored k-major: (p2 - p1) x rows)
 * with e_hi = E, e_lo = E - tf32_truncate(E), U_lo likewise (three-term tf32 split, fp32-level
 * accuracy).  The building block of lc_gptq_weight_transform_tc; p2 - p1 must be a multiple of 16. */
int lc_gptq_panel_update(float* W, const float* e_hi, const float* e_lo, const float* U, const float* U_lo,
                         int64_t rows, int64_t cols, int64_t p1, int64_t p2, int32_t* status, lc_stream_t stream);

/* fp32-accurate GEMM on the tensor cores (tcgen05 kind::tf32, three-term hi/lo split), the building
 * block of lc_gptq_panel_update and lc_gptq_factorize:
 *     C[M][N] (pitch ldc) = beta * C + sign * A^T B,   A: [K][M] (pitch lda), B: [K][N] (pitch ldb)
 * x_hi is the fp32 operand itself, x_lo = x - tf32_truncate(x) (lc_gptq_split_tf32).  K % 16 == 0; M, N
 * and the pitches multiples of 4; beta 0 or 1; sign +1 or -1; flags: LC_GEMM_*.  Replaces the fp32
 * cuBLAS products of the reference (gptq.py:244 and the GEMMs inside its factorisations). */
#define LC_GEMM_UPPER_ONLY 1 /* C is a diagonal-aligned square block: tiles below the diagonal are skipped */
#define LC_GEMM_B_LOWER 2    /* B[k][n] == 0 for k < n */
#define LC_GEMM_A_UPPER 4    /* A[k][m] == 0 for k > m */
int lc_tf32x3_gemm_tn(float* C, int64_t ldc, const float* A_hi, const float* A_lo, int64_t lda, const float* B_hi,
                      const float* B_lo, int64_t ldb, int64_t M, int64_t N, int64_t K, int beta, float sign,
                      int flags, int32_t* status, lc_stream_t stream);

/* U (n x n, upper triangular, zeros below) with U^T U = H^-1, from A = J H J, the permuted and
 * dampened Hessian with rows and columns reversed (lc_gptq_permute_damp with reverse_h = 1): the
 * factorisation chain of GPTQ.process_hessian_and_weights (gptq.py:172-174: cholesky, cholesky_inverse,
 * cholesky upper) as one blocked Cholesky and one blocked triangular inverse with the large products on
 * the tensor cores.  A is destroyed.  U_lo, if not NULL, receives U - tf32_truncate(U).  n % 128 == 0.
 * workspace: lc_gptq_factor_workspace_floats(n) floats.  A non-positive pivot sets *status to
 * LC_ERR_NOT_PD (the reference raises LinAlgError); a timed-out device wait to LC_ERR_TIMEOUT. */
int64_t lc_gptq_factor_workspace_floats(int64_t n);
int lc_gptq_factorize(float* A, int64_t n, float* U, float* U_lo, float* workspace, int64_t workspace_floats,
                      int32_t* status, lc_stream_t stream);

/* The second half of lc_gptq_factorize alone: G (n x n, row-major, upper triangle read) is the upper
 * Cholesky factor of A = J H J (A = G^T G), e.g. from cuSOLVER's potrf -- whose column-major lower
 * factor is this row-major upper factor, byte for byte.  Computes U = J (G^-1)^T J (and U_lo) with
 * the blocked triangular inverse on the tensor cores.  Same workspace and status as above; G is
 * not modified. */
int lc_gptq_invert_factor(const float* G, int64_t n, float* U, float* U_lo, float* workspace,
                          int64_t workspace_floats, int32_t* status, lc_stream_t stream);

/* lc_gptq_invert_factor in two steps, for a process group whose ranks all factorise the same Hessian
 * (the reference repeats the factorisation on every rank): the top node of the recursion holds three
 * quarters of the inverse's FLOPs in its off-diagonal block Vt[h:n, 0:h], h = lc_gptq_factor_split(n).
 * _part computes everything below the top node in full and that block only for columns
 * [col_begin, col_end) (multiples of 128, within [0, h)); the caller then exchanges the column slices
 * (the n x n row-major Vt starts lc_gptq_factor_vt_offset(n) floats into the workspace; collectives stay
 * with the caller) and _finish writes U and U_lo from the completed Vt.  Same values as the one-call
 * form, whatever the slicing. */
int64_t lc_gptq_factor_split(int64_t n);
int64_t lc_gptq_factor_vt_offset(int64_t n);
int lc_gptq_invert_factor_part(const float* G, int64_t n, float* workspace, int64_t workspace_floats,
                               int64_t col_begin, int64_t col_end, int32_t* status, lc_stream_t stream);
int lc_gptq_invert_factor_finish(int64_t n, const float* workspace, int64_t workspace_floats, float* U, float* U_lo,
                                 lc_stream_t stream);

/* GPTQ.weight_transform (gptq.py:199-244) with the trailing update on the tensor cores: the update
 * after each 128-column block covers only the rest of its 256-column sub-panel (fp32 FFMA); the rest of
 * the 1024-column panel is updated once per sub-panel (K = 256) and the columns to the right of a panel
 * once per panel (K = 1024), both by tcgen05 kind::tf32 GEMMs with a three-term hi/lo split
 * (lc_tf32x3_gemm_tn).  Same sums as the reference, associated differently.
 *   U_lo        cols x cols from lc_gptq_split_tf32(U)
 *   scratch_err 128 x rows;  panel_hi, panel_lo  1024 x rows each (fp32 scratch)
 *   status      optional, receives LC_ERR_TIMEOUT if a bounded pipeline wait expires
 * Needs cols % 128 == 0 and rows % 4 == 0 (LC_ERR_SHAPE otherwise: use lc_gptq_weight_transform). */
int lc_gptq_weight_transform_tc(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols,
                                int bits, int sym, float* scratch_err, float* panel_hi, float* panel_lo,
                                float* scales, float* zeros, uint8_t* codes_u8, float* loss_rows,
                                int32_t* status, lc_stream_t stream);

/* GPTQ.weight_transform in owq mode (gptq.py:44-50, :199-244 with n_nonout < columns): hessian_sorting
 * (gptq.py:66-83) has moved the outlier columns to the end; only columns [0, n_quant) are quantised
 * (the last group's qparams come from its columns below n_quant, gptq.py:216-223), the columns from
 * n_quant on receive the error feedback and stay fp32 (gptq.py:186-188).  Otherwise as
 * lc_gptq_weight_transform / lc_gptq_weight_transform_tc, which are these with n_quant == cols.
 * scales / zeros keep (rows * ceil(cols / 128)) entries; groups that start at or beyond n_quant are not
 * written; codes_u8 is written for columns below n_quant only. */
int lc_gptq_weight_transform_owq(float* W, const float* U, int64_t rows, int64_t cols, int64_t n_quant, int bits,
                                 int sym, float* scratch_err, float* scales, float* zeros, uint8_t* codes_u8,
                                 float* loss_rows, lc_stream_t stream);
int lc_gptq_weight_transform_tc_owq(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols,
                                    int64_t n_quant, int bits, int sym, float* scratch_err, float* panel_hi,
                                    float* panel_lo, float* scales, float* zeros, uint8_t* codes_u8,
                                    float* loss_rows, int32_t* status, lc_stream_t stream);

/* SpQR.weight_transform (llmc/compression/quantization/spqr.py:184-285): the GPTQ block loop with groups
 * of 16 columns (the reference's spqr_w_only.yml), asymmetric `bits`-bit codes with unrounded zero points
 * (round_zp False, quant.py:544-558, :698-711), the second-level quantisation of every group's scale and
 * zero point (spqr.py:325-346), leave-one-out outlier detection per group (spqr.py:185-203, unless
 * `simplified`) and outliers kept unquantised (spqr.py:262-267).
 *   W          rows x cols fp32 (permuted order), updated in place: on return the kept (error-compensated,
 *              unquantised) values, the reference's `tmp`
 *   U          cols x cols fp32 upper Cholesky factor of the damped inverse Hessian
 *   U_lo       lc_gptq_split_tf32(U), or NULL: with it the trailing update is batched over 256- and
 *              1024-column panels on the tensor cores (needs panel_hi / panel_lo, 1024 x rows each, and
 *              rows % 4 == 0); without it every block is followed by the fp32 update of all later columns
 *   threshold  device scalar, relative_threshold * mean(var(W, dim 0) / diag(U)^2) (spqr.py:205-207);
 *              +inf switches the detection off
 *   scratch_err 128 x rows fp32
 *   scales, zeros  rows x (cols / 16) fp32: group g of row r at r * (cols / 16) + g, the layout of the
 *              reference's buf_scales / buf_zeros (set_model_qparams, spqr.py:348-356)
 *   mask_u8    rows x cols bytes, 1 = outlier (permuted order), or NULL
 *   loss_rows  rows fp32, sum of squared errors per row, or NULL
 * cols % 128 == 0.  Per block bit-identical to the reference's fp32 arithmetic except for the
 * leave-one-out errors, which are only compared with the threshold. */
int lc_spqr_weight_transform(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols, int bits,
                             const float* threshold, int simplified, float* scratch_err, float* panel_hi,
                             float* panel_lo, float* scales, float* zeros, uint8_t* mask_u8, float* loss_rows,
                             int32_t* status, lc_stream_t stream);

/* SpQR.w_qdq (spqr.py:367-390) in one pass: out[r][c] = W[r][c] where mask is set, else the static fake
 * quantisation of W[r][c] with the statistics of group invperm[c] / 16 of row r (invperm NULL: c / 16);
 * W fp32 in original column order, mask_u8 in original column order, out in `out_dtype`. */
int lc_spqr_dequant(const float* W, const float* scales, const float* zeros, const uint8_t* mask_u8,
                    const int64_t* invperm, int64_t rows, int64_t cols, int bits, void* out, int out_dtype,
                    lc_stream_t stream);

/* GPTQ.weight_transform with static groups (special.static_groups, gptq.py:224-227, with
 * search_group_qparams :377-393): the qparams are not searched block by block but taken from the
 * layer's round-to-nearest buffers, and with act-order column i of the permuted weight uses the group
 * of its ORIGINAL column.
 *   scales, zeros  INPUT, rows x ceil(cols / 128) fp32 in the layer's buf_scales layout (row-major:
 *                  row r, group g at r * n_groups + g); zeros may be NULL when sym
 *   col_group      cols int32: group of permuted column j, i.e. perm[j] / 128 (j / 128 without act-order)
 * Everything else as lc_gptq_weight_transform / lc_gptq_weight_transform_tc; nothing is written to
 * scales / zeros. */
int lc_gptq_weight_transform_static(float* W, const float* U, int64_t rows, int64_t cols, int bits, int sym,
                                    float* scratch_err, const float* scales, const float* zeros,
                                    const int32_t* col_group, uint8_t* codes_u8, float* loss_rows,
                                    lc_stream_t stream);
int lc_gptq_weight_transform_tc_static(float* W, const float* U, const float* U_lo, int64_t rows, int64_t cols,
                                       int bits, int sym, float* scratch_err, float* panel_hi, float* panel_lo,
                                       const float* scales, const float* zeros, const int32_t* col_group,
                                       uint8_t* codes_u8, float* loss_rows, int32_t* status, lc_stream_t stream);

/* lc_gptq_weight_transform for callers that cannot allocate.  (No counterpart in the reference:
 * its solver allocates freely through torch.)
 *
 * Meant for processes that may pass their own W / U / output buffers but have no way to get
 * scratch memory when the call is made -- all device memory belongs to a fixed pool or arena, or
 * the calling context forbids cudaMalloc and the torch allocator.  The 128 x rows fp32 Err
 * scratch is a fixed array inside the library image instead (8 MiB, held on every GPU that loads
 * the library until the process exits), so this call makes no cudaMalloc / cudaFree and uses no
 * allocating library routine.
 *   - rows must be <= 16384; larger layers return LC_ERR_WORKSPACE (use the scratch-taking entry
 *     point with your own buffer instead).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current) and caches it.  Make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the last call left in it.
 *     Nothing in it needs to start at zero (each 128-column block overwrites it completely
 *     before reading it), but two calls whose kernels overlap on the GPU -- different streams,
 *     or different host threads -- race on it: serialise them.
 *   - The cached address belongs to the CUDA context that was current at that first call.  After
 *     a cudaDeviceReset, or from a second context on the same device ordinal, it is stale: such
 *     processes must not use this entry point.
 * Results are identical to lc_gptq_weight_transform. */
int lc_gptq_weight_transform_noalloc(float* W, const float* U, int64_t rows, int64_t cols, int bits,
                                     int sym, float* scales, float* zeros, uint8_t* codes_u8,
                                     float* loss_rows, lc_stream_t stream);

/* Un-permute the kept weights (gptq.py:186-193): out[r][perm[j]] = Wp[r][j], written in
 * `out_dtype`.  perm NULL = identity. */
int lc_gptq_unpermute(const float* Wp, const int64_t* perm, int64_t rows, int64_t cols,
                      void* out, int out_dtype, lc_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Family 4: AWQ scale + clip search.
 * ------------------------------------------------------------------------------------------ */

/* out[c] = mean over tokens of |x[t][c]| in `dtype` (fp32 accumulation, one rounding):
 * Awq.get_act_scale (llmc/compression/quantization/awq.py:74-76).
 * scratch: at least min(64, ceil(tokens/256)) * cols floats. */
int lc_awq_act_mean(const void* x, int dtype, int64_t tokens, int64_t cols, void* out, float* scratch,
                    int64_t scratch_floats, lc_stream_t stream);

/* fake_out = quant_dequant(round_to_dtype(w * col_scale[col])), per group of `group` columns:
 * Awq.scaling_weight + fake_quant_weight_dynamic (awq.py:40-46, :147-164) in one pass, without
 * touching w.  col_scale: `cols` values in `dtype`.  Same arithmetic as lc_rtn_int_quant. */
int lc_awq_scale_quant(const void* w, const void* col_scale, int dtype, int64_t rows, int64_t cols,
                       int64_t group, int bits, int sym, void* fake_out, lc_stream_t stream);

/* out[r][c] = x[r][c] / col_scale[c] rounded to `dtype`: scaling_input / update_input_feat
 * (llmc/compression/quantization/base_blockwise_quantization.py:900-920).  out may alias x. */
int lc_awq_div_cols(const void* x, const void* col_scale, int dtype, int64_t rows, int64_t cols, void* out,
                    lc_stream_t stream);

/* loss_out[0] = mean((a - b)^2), the subtraction rounded to `dtype`, squares and sum in fp32 or
 * wider: Awq.calculate_loss (awq.py:134-136).  scratch: at least 592 doubles. */
int lc_awq_loss(const void* a, const void* b, int dtype, int64_t n, float* loss_out, double* scratch,
                int64_t scratch_doubles, lc_stream_t stream);

/* AutoClipper.auto_clip_layer + apply_clip, clip_version v1
 * (llmc/compression/quantization/auto_clip.py:84-191, :194-212), fused: for every (row, group)
 * the grid of int(max_shrink * n_grid) shrink ratios 1 - i/n_grid is evaluated on the sampled
 * tokens x[0::x_token_step] with the reference's rounding after every op, the best range is
 * written to best_max / best_min ((rows, cols/group) in `dtype`) and, if W_out is not NULL, the
 * clamped weights to W_out (may alias W).
 *   W rows x cols, X x_tokens x cols, both `dtype` (bf16 or fp16); group must be 128; at most 512
 *   sampled tokens. */
int lc_awq_clip_search(const void* W, const void* X, int dtype, int64_t rows, int64_t cols, int64_t x_tokens,
                       int64_t x_token_step, int64_t group, int bits, int sym, int clip_sym, int n_grid,
                       double max_shrink, void* best_max, void* best_min, void* W_out, lc_stream_t stream);

/* The same search with the sums formed on the CUDA cores (an unpack and an fp32 add per product) instead of
 * by MMAs against a matrix of ones.  Both round every product to the tensor dtype first and differ only in
 * the order of the fp32 additions; kept for comparison and for token counts that are not a multiple of 16,
 * which lc_awq_clip_search routes here by itself. */
int lc_awq_clip_search_cuda_cores(const void* W, const void* X, int dtype, int64_t rows, int64_t cols, int64_t x_tokens,
                       int64_t x_token_step, int64_t group, int bits, int sym, int clip_sym, int n_grid,
                       double max_shrink, void* best_max, void* best_min, void* W_out, lc_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Export layouts for 4-bit codes (what follows the hot path when a real-quant model is saved).
 * ------------------------------------------------------------------------------------------ */

/* AutoAWQ GEMM layout, the packing loops of AutoawqRealQuantLinear.gemm_pack
 * (llmc/compression/quantization/module_utils.py:1130-1158): codes (rows = out_features x cols =
 * in_features, one byte per code, 0..15) -> out (cols x rows/8) int32, word (k, c) holding output
 * rows 8c + {0,2,4,6,1,3,5,7} of input column k in nibbles 0..7.  Zero points pack the same way
 * (codes = zeros (out x n_groups) -> (n_groups x out/8)).  rows must be a multiple of 8.
 * The compressed-tensors int4 layout of VllmRealQuantLinear.pack (module_utils.py:931-955) needs no
 * routine of its own: it is LC_CODES_PACK4 from lc_rtn_int_quant (symmetric, stored as q + 8). */
int lc_pack_int4_awq(const uint8_t* codes, int64_t rows, int64_t cols, int32_t* out, lc_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Element-wise pieces of the calibration block forward.  The reference has no functions of its
 * own here: block_forward (llmc/compression/quantization/base_blockwise_quantization.py:378-401)
 * runs the decoder block's stock module code, whose rotary embedding and gated activation are
 * chains of 7 and 2 separate tensor ops, and whose RMS norm is a chain of 8.  These routines replace
 * those chains, rounding to `dtype` after every op of the chain, so that the block's outputs do not
 * change by a bit.
 * ------------------------------------------------------------------------------------------ */

/* out = (x * cos) + (rotate_half(x) * sin), rotate_half(x) = cat(-x[d/2:], x[:d/2]) per head.
 * x, out: [tokens][heads][head_dim] contiguous; cos_tab, sin_tab: [table_tokens][head_dim], token t
 * using row t % table_tokens (table_tokens = tokens, or the sequence length when all sequences of a
 * batch share one table); all `dtype`.  head_dim must be a multiple of 8 (fp32) / 16 (bf16, fp16)
 * elements.  out must not alias x. */
int lc_rope_apply(const void* x, const void* cos_tab, const void* sin_tab, int dtype, int64_t tokens, int heads,
                  int head_dim, int64_t table_tokens, void* out, lc_stream_t stream);

/* out = silu(gate) * up over n elements, silu(x) = x / (1 + exp(-x)) evaluated in fp32 and rounded
 * to `dtype` before the product.  n must be a multiple of the 16-byte vector.  out may alias either input. */
int lc_silu_mul(const void* gate, const void* up, int dtype, int64_t n, void* out, lc_stream_t stream);

/* out = weight * (xf * rsqrt(mean(xf^2, last dim) + eps)).to(dtype), xf = x.float(): the RMS norm of
 * Llama-style decoder blocks.  x, out: [rows][cols], weight: [cols], all `dtype`.  The sum of squares
 * is associated like torch's row reduction of a contiguous fp32 tensor (see block_ops.cu), which fixes
 * 128 <= cols < 8192 and cols % 128 == 0 (LC_ERR_SHAPE otherwise); mean_factor is 1/cols as the
 * replaced mean computes it, (float)rows / (float)(rows * cols).  The host mirror verifies bit
 * equality with the module it replaces on random data before first use. */
int lc_rmsnorm(const void* x, const void* weight, int dtype, int64_t rows, int64_t cols, float mean_factor,
               float eps, void* out, lc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LC_B200_H_ */
