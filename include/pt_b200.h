/*
 * C ABI of the sm_100a (B200) low-precision GEMM path: quantize / dequantize,
 * dense and grouped FP8 / MXFP8 / MXFP4 GEMMs.
 *
 * This is the boundary a host binding talks to.  It replaces the operators the
 * reference registers in TORCH_LIBRARY(primus_turbo_cpp_extension, ...)
 * (csrc/pytorch/bindings_pytorch.cpp:15-135) and the Python-level custom ops
 * primus_turbo::gemm_fp8_impl / grouped_gemm_fp8_impl / ... that wrap its Triton and
 * FlyDSL kernels (primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:518-593,
 * primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:888-1030).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its comment says "host";
 *  - the caller allocates every output and every workspace (the reference's ops allocate
 *    with at::empty; here the binding does that and passes the pointers);
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing
 *    synchronises the device;
 *  - every function returns 0 on success or a negative pt_status; pt_last_error() gives
 *    the message of the last failure on the calling thread (the reference throws
 *    std::runtime_error through PRIMUS_TURBO_CHECK, csrc/include/primus_turbo/macros.h:71-84);
 *  - inputs are never written; outputs may be left unwritten only where stated.
 */
#ifndef PT_B200_H_
#define PT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { PT_OK = 0, PT_ERR_INVALID = -1, PT_ERR_CUDA = -2, PT_ERR_UNSUPPORTED = -3, PT_ERR_TIMEOUT = -4 } pt_status;

/* source / output element types */
typedef enum { PT_BF16 = 0, PT_F16 = 1, PT_F32 = 2 } pt_dtype;
/* quantized element formats: e4m3fn, e5m2 (1 byte each), e2m1 (two per byte, element 2j in the low nibble) */
typedef enum { PT_E4M3 = 0, PT_E5M2 = 1, PT_E2M1 = 2 } pt_format;
/* scaling granularity, in the order of ScalingGranularity (primus_turbo/pytorch/core/low_precision.py:123-132),
 * counted from 0 (the Python enum counts from 1) */
typedef enum { PT_TENSORWISE = 0, PT_ROWWISE = 1, PT_BLOCKWISE = 2, PT_MX_BLOCKWISE = 3 } pt_granularity;

const char *pt_last_error(void);
/* Library / device sanity: returns the number of SMs of the current device, or a negative status. */
int pt_device_sm_count(void);

/* Kernels wait on barriers (data arriving by TMA, tensor-core completion, peer CTAs) with a bound: a wait that outlasts
 * it gives up, the kernel unwinds and reports PT_ERR_TIMEOUT in a device status word instead of hanging the GPU; the
 * output of that launch is then invalid.  The GEMM entry points take the word as their `status` argument.  The
 * quantizers have none: they report into the word registered here for the current device (null: none, the default).
 * The word must stay allocated while registered.  A caller that never reads its status words gets unchecked results.
 * (The reference has no counterpart: its kernels wait without a bound.) */
int pt_set_default_status(int *status);

/* Self-test of the bounded wait: launches one CTA whose first thread waits `limit_ns` nanoseconds (1 us .. 1 s) on a
 * barrier that nothing completes; the wait gives up, the kernel returns, *status receives PT_ERR_TIMEOUT and
 * *observers (optional device int, zeroed by the caller) the number of warps (4) that saw the abort flag.  Nothing
 * faults and nothing waits without a bound.  (No counterpart in the reference.) */
int pt_wait_probe(int64_t limit_ns, int *status, int *observers, void *stream);

/* ------------------------------------------------------------------ tensorwise / rowwise FP8 */

/* Bytes of scratch pt_quantize_fp8_tensorwise needs (holds the running amax). */
size_t pt_quantize_fp8_tensorwise_workspace_bytes(void);

/* q = fp8(clamp(x * scale, +-qmax)), scale = qmax / max(amax(|x|), 1e-12), *scale_inv = 1 / scale.
 * x: n contiguous elements of x_dtype.  scale_opt: optional device float; when given it is used as
 * `scale` and no amax is taken.  workspace: >= pt_quantize_fp8_tensorwise_workspace_bytes() bytes.
 * Replaces quantize_fp8_tensorwise (csrc/pytorch/quantization/quantization.cpp:44-90). */
int pt_quantize_fp8_tensorwise(const void *x, int x_dtype, int64_t n, int fmt, void *q, float *scale_inv,
                               const float *scale_opt, void *workspace, size_t workspace_bytes, void *stream);

/* x viewed as [B, M, N] with the scaled axis being M when axis_is_last == 0 (scale_inv is [B, 1, N]) or
 * N when axis_is_last != 0 (pass B = 1, M = outer rows; scale_inv is [M, 1]).  scale_opt as above, same
 * shape as scale_inv.  workspace: B*N floats when axis_is_last == 0 and scale_opt is null, else unused.
 * Replaces quantize_fp8_rowwise (quantization.cpp:110-208). */
int pt_quantize_fp8_rowwise(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, int axis_is_last, int fmt,
                            void *q, float *scale_inv, const float *scale_opt, void *workspace,
                            size_t workspace_bytes, void *stream);

/* The column-scaled form of pt_quantize_fp8_rowwise (x viewed as [B, M, N], one scale per (b, n), scale_inv
 * [B, 1, N]) for callers that cannot hand over scratch memory because they cannot allocate any: a host runtime
 * that gave all of the GPU's memory to its own arena at start-up, or code that runs in a phase where calls into
 * the driver's allocator are not permitted.  The per-column maxima are kept in an array built into the library
 * (256 KiB on every GPU that loads it, until the process exits), so B * N may not exceed 65536 columns; larger
 * inputs are refused with PT_ERR_INVALID and belong to pt_quantize_fp8_rowwise.  Results are identical to
 * pt_quantize_fp8_rowwise(axis_is_last = 0, scale_opt = null).  The first call on each device looks up the
 * array's device address (make that call before starting a stream capture).  All calls share the one array:
 * two calls whose kernels overlap on the GPU (different streams) race; calls on one stream are safe.
 * This entry point has no counterpart in the reference. */
int pt_quantize_fp8_colscale_noalloc(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, int fmt, void *q,
                                     float *scale_inv, void *stream);

/* y = float(q) * scale_inv, cast to y_dtype.  Scale broadcast is described by [B, M, N] as above:
 * tensorwise: B = M = 1 and scale_kind = 0; per-row (axis last): scale_kind = 1; per-column: scale_kind = 2.
 * Replaces dequantize_fp8_tensorwise / dequantize_fp8_rowwise (quantization.cpp:211-330). */
int pt_dequantize_fp8(const void *q, int fmt, const float *scale_inv, int scale_kind, int64_t B, int64_t M,
                      int64_t N, void *y, int y_dtype, void *stream);

/* ------------------------------------------------------------------ 128-blockwise FP8 */

/* 1 x 128 (row) and / or 128 x 1 (col) block scales of x [M, N]; eps 1e-4; stored scale is 1/scale.
 * q_row [M, N], s_row [M, ceil(N/128)]; q_col [M, N] (NOT transposed), s_col [ceil(M/128), N].
 * Pass null for the direction that is not wanted.
 * Replaces quant_fp8_blockwise_impl / quant_fp8_blockwise_dual_impl
 * (primus_turbo/pytorch/kernels/quantization/quantization_impl.py:81-125,236-281). */
int pt_quantize_fp8_blockwise(const void *x, int x_dtype, int64_t M, int64_t N, int fmt, void *q_row, float *s_row,
                              void *q_col, float *s_col, void *stream);

/* One scale per 128 x 128 tile of w [B, M, N]; s [B, ceil(M/128), ceil(N/128)].
 * Replaces quantize_fp8_blockwise_for_weight (bindings_pytorch.cpp:40, quantization_blockwise.cu:248-346). */
int pt_quantize_fp8_blockwise_weight(const void *w, int x_dtype, int64_t B, int64_t M, int64_t N, int fmt, void *q,
                                     float *s, void *stream);

/* Grouped row + segment-padded column quantization of x [M, N] whose rows are split into G groups.
 * group_offs / padded_offs: int64 [G+1] exclusive prefix sums of the group lengths and of the lengths
 * rounded up to 128.  q_row [M, N]; s_row [ceil(N/128), M] (transposed); q_col [m_alloc, N] and
 * s_col [m_alloc/128, N] with m_alloc = M + G*128; rows at or past padded_offs[G] are not written.
 * Replaces quantize_fp8_blockwise_segment_m_row_col (bindings_pytorch.cpp:38, quantization_blockwise.cu:60-232). */
int pt_quantize_fp8_blockwise_segment_m(const void *x, int x_dtype, int64_t M, int64_t N, int G,
                                        const int64_t *group_offs, const int64_t *padded_offs, int fmt, void *q_row,
                                        float *s_row, void *q_col, float *s_col, void *stream);

/* y = float(q) * s with the block scale layouts above: kind 0 = row (s [M, ceil(N/128)]),
 * 1 = col (s [ceil(M/128), N]), 2 = weight tiles (s [ceil(M/128), ceil(N/128)]); B batches.
 * Replaces dequant_fp8_blockwise_impl / dequant_fp8_blockwise_for_weight_impl (quantization_impl.py:146-233). */
int pt_dequantize_fp8_blockwise(const void *q, int fmt, const float *s, int kind, int64_t B, int64_t M, int64_t N,
                                void *y, int y_dtype, void *stream);

/* ------------------------------------------------------------------ group offsets */

/* offs[0] = 0, offs[i+1] = sum_{j<=i} lens[j]; int64, G <= 4096.
 * Replaces grouped_gemm_compute_offs (bindings_pytorch.cpp:134, compute_group_offs.cu:15-32). */
int pt_compute_group_offs(const int64_t *lens, int G, int64_t *offs, void *stream);
/* plens[i] = ceil_to(lens[i], align); poffs = their exclusive prefix sums
 * (quantization_blockwise.cu:18-36, quantization_mxfp8.cu:2025-2039). */
int pt_compute_padded_group_offs(const int64_t *lens, int G, int64_t align, int64_t *plens, int64_t *poffs,
                                 void *stream);

/* ------------------------------------------------------------------ MX (32-element blocks, ue8m0 scales) */

/* flags for pt_quantize_mx */
#define PT_MX_ROW 1u        /* produce the row-wise copy  (blocks along N) */
#define PT_MX_COL 2u        /* produce the col-wise, transposed copy (blocks along M) */
#define PT_MX_ROW_2D 4u     /* row copy uses one scale per 32 x 32 tile */
#define PT_MX_COL_2D 8u     /* col copy uses one scale per 32 x 32 tile */
#define PT_MX_ROW_RHT 16u   /* e2m1 only: 16-point Hadamard along the quantized axis before amax */
#define PT_MX_COL_RHT 32u
#define PT_MX_ROW_SR 64u    /* e2m1 only: stochastic rounding of the row copy (a fresh seed per call; unbiased, not */
#define PT_MX_COL_SR 128u   /*            reproducible -- quantization_mxfp4.cu:59-71,241-274 of the reference)     */

/* x [G, M, N] (G = 1 for 2-D), bf16 / fp16, N % 32 == 0.  M_pad = ceil128(M), N_pad = ceil128(N).
 * fmt e4m3 / e5m2: q_row [G, M, N_pad], s_row [G, M, N_pad/32]; q_col [G, N, M_pad], s_col [G, N, M_pad/32].
 * fmt e2m1: data rows are half as long (two codes per byte).  Pad columns hold zeros (scale byte 0).
 * Replaces quantize_mxfp8 / quantize_mxfp8_dual / quantize_mxfp4 / quantize_mxfp4_dual with shuffle off
 * (bindings_pytorch.cpp:52-93; csrc/pytorch/quantization/quantization.cpp:511-969). */
int pt_quantize_mx(const void *x, int x_dtype, int64_t G, int64_t M, int64_t N, int fmt, unsigned flags,
                   void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream);

/* Grouped form for x [M, N] whose rows are split into G groups (int64 offsets [G+1] on the device).
 * The col-wise copy lives in the 128-padded row space: q_col [N, col_alloc(/2)], s_col [N, col_alloc/32] with
 * col_alloc = ceil128(M + G*128); group g occupies columns padded_offs_col[g] .. padded_offs_col[g+1], zero padded.
 * The row-wise copy puts row i of group g at row padded_offs_row[g] + i of q_row [rows_alloc, N_pad(/2)],
 * s_row [rows_alloc, N_pad/32] (fp8: groups padded to 32 rows, rows_alloc = ceil32(M + G*32); fp4: pass the tight
 * offsets, rows_alloc = M); pad rows and anything at or past the last padded offset are not written.
 * An all-zero block gets scale byte 127.  Flags as in pt_quantize_mx without the 2-D options.
 * Replaces grouped_quantize_mxfp8(_dual) / grouped_quantize_mxfp4(_dual) (bindings_pytorch.cpp:61-70,79-93;
 * csrc/pytorch/quantization/quantization.cpp:971-1378). */
int pt_grouped_quantize_mx(const void *x, int x_dtype, int64_t M, int64_t N, int G, const int64_t *group_offs,
                           const int64_t *padded_offs_row, const int64_t *padded_offs_col, int fmt, unsigned flags, void *q_row,
                           uint8_t *s_row, void *q_col, uint8_t *s_col, int64_t col_alloc, void *stream);

/* y [rows, cols] = decode(q [rows, cols_stored]) * 2^(s - 127); cols <= cols_stored (the stored row length in
 * elements, a multiple of 32); s [rows, cols_stored/32].  When transpose_out != 0 y is written as [cols, rows]
 * (col-wise inputs are returned re-transposed, quantization.cpp:332-358).
 * Replaces dequantize_mxfp8 / dequantize_mxfp4 (bindings_pytorch.cpp:58,88). */
int pt_dequantize_mx(const void *q, int fmt, const uint8_t *s, int64_t rows, int64_t cols, int64_t cols_stored,
                     int transpose_out, void *y, int y_dtype, void *stream);

/* ------------------------------------------------------------------ transpose */
/* y [N, M] = x [M, N]^T for 1-, 2- or 4-byte elements (bindings_pytorch.cpp:44, csrc/kernels/transpose/transpose_2d.cu). */
int pt_transpose_2d(const void *x, int64_t M, int64_t N, int elem_bytes, void *y, void *stream);

/* The same over a batch: y [B, N, M] = x [B, M, N] transposed per matrix (a [G, K, N] expert weight to [G, N, K]). */
int pt_transpose_batched(const void *x, int64_t B, int64_t M, int64_t N, int elem_bytes, void *y, void *stream);

/* Token-major to token-minor copy of a grouped operand (1- or 2-byte elements) for the variable-K GEMM: x [M, C] holds group g in rows
 * group_offs[g] .. group_offs[g+1]; y [C, T] receives them as columns padded_offs[g] .. padded_offs[g] + len_g.  The rest
 * of every segment (padded_offs are multiples of 128, see pt_compute_padded_group_offs) and all columns from
 * padded_offs[G] on are written as zeros, so that they add nothing to the contraction.  T is a multiple of 64 and
 * at least padded_offs[G]; both offset arrays are device int64 [G+1] (no host synchronisation).
 * The reference's tensorwise / rowwise variable-K kernels read the token-major operands in place
 * (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:936-1030); pt_grouped_gemm_fp8_variable_k takes
 * K-major operands, and this is the copy that produces them. */
int pt_grouped_transpose_pad(const void *x, int64_t M, int64_t C, int elem_bytes, const int64_t *group_offs,
                             const int64_t *padded_offs, int G, void *y, int64_t T, void *stream);

/* Zero-fills rows [*first_row, rows) of a row-major buffer with `row_bytes` bytes per row (a multiple of 4, base 4-byte
 * aligned); `first_row` is a device pointer, so no host synchronisation is needed.  The grouped GEMMs leave rows past the
 * last group untouched; the reference returns zeros there (grouped_gemm_fp8_impl.py: output tail), so the caller
 * clears that tail — and only it — with this call instead of a memset of the whole output. */
int pt_zero_rows_from(void *buf, int64_t rows, int64_t row_bytes, const int64_t *first_row, void *stream);

/* ------------------------------------------------------------------ FP8 / MXFP8 GEMM (tcgen05, TMEM accumulators) */

/* C [M, N] (row-major, c_dtype) = A [M, K] . B [N, K]^T, both operands K-major FP8 bytes ("NT").  Other
 * layouts of the reference's (trans_a, trans_b, trans_c) are reached by swapping operands (trans_c) or by
 * handing in the transposed copy (pt_transpose_2d) as the reference itself does for its NT-only back ends
 * (primus_turbo/pytorch/ops/gemm_fp8.py:44-50,126-149).
 *   granularity PT_TENSORWISE:   a_scale, b_scale = device float[1] (scale_inv);  C = acc * a_scale * b_scale
 *   granularity PT_ROWWISE:      a_scale float[M], b_scale float[N];               C = acc * a_scale[m] * b_scale[n]
 *   granularity PT_MX_BLOCKWISE: a_scale uint8 [M, K/32], b_scale uint8 [N, K/32] (ue8m0, raw row-major as the
 *                                quantizer writes them); K is the padded length (multiple of 128)
 * a_fmt / b_fmt: PT_E4M3 or PT_E5M2 (may differ: HYBRID).  beta: 0, or 1 to accumulate into C.
 * block_n: 0 = default tile width, else 128 / 240 / 256.  workspace: device scratch of at least
 * pt_gemm_fp8_workspace_bytes(...) bytes, 16-byte aligned (may be null when that is 0).  status: optional device int that receives
 * PT_ERR_TIMEOUT if a bounded wait inside the kernel expires (it is never written otherwise).
 * Replaces primus_turbo::gemm_fp8_impl / gemm_fp8_accum_impl (primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:518-593)
 * and the vendor ops hipblaslt_gemm_fp8 / ck_gemm_fp8 / turbo_gemm_fp8 (csrc/pytorch/bindings_pytorch.cpp:20-31). */
int pt_gemm_fp8(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt, void *c,
                int c_dtype, int granularity, int64_t M, int64_t N, int64_t K, float beta, int block_n, void *workspace,
                size_t workspace_bytes, int *status, void *stream);

/* pt_gemm_fp8 for PT_TENSORWISE / PT_ROWWISE with operands read in place whichever way they are stored: a_mn = 1 means
 * `a` is stored [K, M] (contraction-major: the layout of an activation or gradient that a wgrad contracts over its tokens,
 * or of a weight that a dgrad contracts over its output features), 0 means [M, K]; likewise b_mn for `b` ([K, N] / [N, K]).
 * An MN-major operand needs a row count (M or N) that is a multiple of 16.  Removes the transposed copies the reference's
 * NT-only back ends make first (primus_turbo/pytorch/ops/gemm_fp8.py:44-50 of the reference). */
int pt_gemm_fp8_mn(const void *a, const void *a_scale, int a_fmt, int a_mn, const void *b, const void *b_scale, int b_fmt, int b_mn, void *c,
                   int c_dtype, int granularity, int64_t M, int64_t N, int64_t K, float beta, int *status, void *stream);

/* Scratch bytes pt_gemm_fp8 / pt_grouped_gemm_fp8 need: 0 except for PT_MX_BLOCKWISE, where the raw scales are
 * re-tiled into the block layout of the tensor core's scale copy before the GEMM (the reference's back ends also
 * pre-shuffle the raw scales right before their kernels, primus_turbo/pytorch/ops/gemm_fp8.py:577-579).
 * c_rows: rows of C (per group for the variable-K form); grouped: 0 = pt_gemm_fp8, 1 = pt_grouped_gemm_fp8,
 * 2 = pt_grouped_gemm_fp8_variable_k; block_n as passed to the GEMM. */
size_t pt_gemm_fp8_workspace_bytes(int granularity, int64_t c_rows, int64_t N, int64_t K, int G, int grouped, int block_n);

/* Grouped form: rows are split into G groups, group g multiplies B[g] ([G, N, K] contiguous).
 * group_offs_write int64 [G+1]: first C row of each group (tight); group length = difference.
 * group_offs_read  int64 [G+1] or null: first A row of each group when A (and its scales) were written in a
 * padded layout (MX grouped quantizers); null = same as group_offs_write.
 * a_rows: rows of the A buffer; c_rows: rows of C covered by the groups.  Rows of C at or past
 * group_offs_write[G] are not written.  max_ctas: 0 = one CTA per SM, else an upper bound (the reference's num_cu).
 * Replaces primus_turbo::grouped_gemm_fp8_impl (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:888-930). */
int pt_grouped_gemm_fp8(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt,
                        void *c, int c_dtype, int granularity, int64_t a_rows, int64_t c_rows, int64_t N, int64_t K,
                        const int64_t *group_offs_read, const int64_t *group_offs_write, int G, float beta, int block_n,
                        int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream);

/* Variable-K grouped GEMM (the grouped wgrad): C [G, M, N], C[g] = A[:, k_offs[g]:k_offs[g+1]] . B[:, same range]^T with
 * A [M, K_total] and B [N, K_total] K-major and shared by all groups; k_offs int64 [G+1], multiples of 128 (the
 * 128-padded per-group token segments the grouped quantizers produce).  A group with an empty range yields zeros.
 * Scales: PT_TENSORWISE scalars; PT_ROWWISE a_scale [G, M], b_scale [G, N]; PT_MX_BLOCKWISE raw ue8m0 [rows, K_total/32].
 * Replaces primus_turbo::grouped_gemm_fp8_variable_k_impl / _accum_impl
 * (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:936-1030). */
int pt_grouped_gemm_fp8_variable_k(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt,
                                   void *c, int c_dtype, int granularity, int64_t M, int64_t N, int64_t K_total,
                                   const int64_t *k_offs, int G, float beta, int block_n, int max_ctas, void *workspace,
                                   size_t workspace_bytes, int *status, void *stream);

/* fp16 / bf16 GEMMs on the same tcgen05 kernels (kind::f16, fp32 accumulate, no scales): C [M, N] = A [M, K] . B [N, K]^T,
 * both operands K-major with K a multiple of 8; ab_dtype PT_BF16 or PT_F16; c_dtype any PT_* output type; beta 0 or 1.
 * Grouped: A [a_rows, K] split by group_offs int64 [G+1] (device), B [G, N, K], rows of C past group_offs[G] are not
 * written.  Variable-K: A [M, K_total], B [N, K_total], C [G, M, N], k_offs int64 [G+1] multiples of 64 elements.
 * Replace primus_turbo::gemm_impl / gemm_accum_impl (primus_turbo/pytorch/kernels/gemm/gemm_impl.py) and
 * primus_turbo::grouped_gemm_impl / grouped_gemm_variable_k_impl / _accum_impl
 * (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_impl.py). */
int pt_gemm(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t M, int64_t N, int64_t K, float beta, int *status,
            void *stream);
int pt_grouped_gemm(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t a_rows, int64_t N, int64_t K,
                    const int64_t *group_offs, int G, float beta, int max_ctas, int *status, void *stream);
int pt_grouped_gemm_variable_k(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t M, int64_t N, int64_t K_total,
                               const int64_t *k_offs, int G, float beta, int max_ctas, int *status, void *stream);

/* MXFP4 (packed e2m1, 32-element blocks, ue8m0 scales) forms of the three MX GEMMs above, on
 * tcgen05.mma kind::mxf4.block_scale: a [M, K/2] bytes, a_scale [M, K/32]; b [N, K/2], b_scale [N, K/32]; K is the
 * padded element count (multiple of 128).  Variable-K offsets count elements and are multiples of 256.
 * Replace primus_turbo::gemm_fp4_impl / gemm_fp4_accum_impl (primus_turbo/pytorch/kernels/gemm/gemm_fp4_impl.py:340-441)
 * and primus_turbo::grouped_gemm_fp4_impl / _variable_k_impl / _variable_k_accum_impl
 * (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp4_impl.py:430-). */
int pt_gemm_fp4(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype, int64_t M, int64_t N,
                int64_t K, float beta, int block_n, void *workspace, size_t workspace_bytes, int *status, void *stream);
int pt_grouped_gemm_fp4(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype, int64_t a_rows,
                        int64_t c_rows, int64_t N, int64_t K, const int64_t *group_offs_read, const int64_t *group_offs_write, int G,
                        float beta, int block_n, int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream);
int pt_grouped_gemm_fp4_variable_k(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype,
                                   int64_t M, int64_t N, int64_t K_total, const int64_t *k_offs, int G, float beta, int block_n,
                                   int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream);
/* Scratch bytes of the FP4 GEMMs (grouped: 0 dense, 1 grouped, 2 variable-K), cf. pt_gemm_fp8_workspace_bytes. */
size_t pt_gemm_fp4_workspace_bytes(int64_t c_rows, int64_t N, int64_t K, int G, int grouped, int block_n);

/* FP8 GEMM with fp32 128-block scales along the contraction (BLOCKWISE granularity): dense (G = 1, offsets null),
 * grouped by rows, or grouped with a per-group contraction range ("variable K", the grouped wgrad):
 *   C[m, n] = sum_kb ( sum_{k in kb} A[m, k] B[n, k] ) * sa(m, kb) * sb(n, kb),   kb = 128-wide block of k.
 * Operands are FP8 bytes, each either K-major (a_mn = 0: memory [rows, K]) or MN-major (a_mn = 1: memory [K, rows],
 * the layout of an operand whose contraction runs over its stored rows); *_mem_rows x *_mem_cols is the 2-D
 * extent of the buffer as stored (row pitch = *_mem_cols bytes, a multiple of 16).  MN-major operands make the
 * reference's NN (dgrad) and TN (wgrad) GEMMs run on the stored tensors without transposed copies.
 * Each scale operand is read in place through
 *   s(row, kb) = base[(row >> shift) * row_stride + kb * kb_stride]   (+ g * sb_group_stride for B),
 * shift 0 = one scale per row, 7 = one per 128 rows; this covers every layout the reference's quantizers emit:
 * [M, K/128] (0, K/128, 1); transposed [K/128, M] (0, 1, M); column scales [Kc/128, R] of a token-major operand
 * (0, 1, R); 128 x 128 weight tiles [N/128, K/128] (7, K/128, 1) or, read across, (7, 1, R/128).
 * Row grouping: group_offs_write / group_offs_read as in pt_grouped_gemm_fp8; B is [G, N, K] (K-major) or
 * [G, K, N] (MN-major, K % 128 == 0).
 * Variable K: k_offs int64 [G+1] (multiples of 128) gives the contraction rows of group g; both operands MN-major
 * ([total_k, c_rows] and [total_k, N]); C is [G, c_rows, N]; a group with an empty range yields zeros.
 * Replaces the BLOCKWISE branches of primus_turbo::gemm_fp8_impl, primus_turbo::grouped_gemm_fp8_impl and
 * primus_turbo::grouped_gemm_fp8_variable_k_impl (primus_turbo/triton/gemm/gemm_fp8_kernel.py:872-1013,
 * primus_turbo/triton/grouped_gemm/grouped_gemm_fp8_kernel.py:1407-1556,1661-1802). */
int pt_grouped_gemm_fp8_blockwise(const void *a, int a_fmt, int a_mn, int64_t a_mem_rows, int64_t a_mem_cols, const float *sa,
                                  int sa_shift, int64_t sa_row_stride, int64_t sa_kb_stride, const void *b, int b_fmt, int b_mn,
                                  int64_t b_mem_rows, int64_t b_mem_cols, const float *sb, int sb_shift, int64_t sb_row_stride,
                                  int64_t sb_kb_stride, int64_t sb_group_stride, void *c, int c_dtype, int64_t c_rows, int64_t N,
                                  int64_t K, const int64_t *group_offs_read, const int64_t *group_offs_write,
                                  const int64_t *k_offs, int G, float beta, int max_ctas, int *status, void *stream);

/* ------------------------------------------------------------------ MoE token permutation (mask-map form) */

/* Scratch bytes of pt_moe_make_row_id_map. */
size_t pt_moe_row_id_map_workspace_bytes(int64_t T, int E);

/* routing_map [T, E] (bool / int32 / int64 elements, map_elem_bytes = 1 / 4 / 8; non-zero = token t goes to expert e) ->
 * row_id_map int32 [T, 2E + 1]: per token the destination rows of its routed experts in ascending expert order (rows of
 * expert 0 first, tokens in order inside an expert), at column E the expert ids in the same order, in the last column
 * their number; unused slots hold -1.  tokens_per_expert int64 [E].
 * Replaces make_row_id_map (primus_turbo/triton/moe/permutation.py:143-230 of the reference). */
int pt_moe_make_row_id_map(const void *routing_map, int map_elem_bytes, int64_t T, int E, int *row_id_map, int64_t *tokens_per_expert,
                           void *workspace, size_t workspace_bytes, void *stream);

/* out[dst] = tokens[t] for every destination row of token t (rows of row_bytes bytes, a multiple of 16); with probs
 * [T, E] (elements of probs_elem_bytes bytes) also out_probs[dst] = probs[t, e].  Destinations at or past num_out_tokens
 * are dropped.  Replaces permute_with_mask_map (primus_turbo/triton/moe/permutation.py of the reference). */
int pt_moe_permute(const void *tokens, int64_t T, int64_t row_bytes, int E, const int *row_id_map, const void *probs, int probs_elem_bytes,
                   int64_t num_out_tokens, void *out, void *out_probs, void *stream);

/* out[t] = sum over the routed experts of (merging_probs[t, e] *) permuted[dst], accumulated in fp32 in expert order
 * (merging_probs optional).  With permuted_probs also unpermuted_probs[t, e] = permuted_probs[dst], zero where token t
 * does not go to expert e; `out` may then be null.  dtype / probs_dtype: pt_dtype codes.
 * Replaces unpermute_with_mask_map (primus_turbo/triton/moe/permutation.py of the reference). */
int pt_moe_unpermute(const void *permuted, int dtype, int64_t T, int64_t H, int E, const int *row_id_map, const void *merging_probs,
                     const void *permuted_probs, int probs_dtype, void *out, void *unpermuted_probs, void *stream);

/* Backward of the weighted unpermute: act_grad[dst] = grad_out[t] * merging_probs[t, e];
 * probs_grad[t, e] = <grad_out[t], fwd_in[dst]> (fp32 dot product), zero where token t does not go to expert e.
 * Replaces unpermute_with_mask_map_bwd_with_merging_probs of the reference. */
int pt_moe_unpermute_bwd_with_probs(const void *grad_out, const void *fwd_in, int dtype, int64_t T, int64_t H, int E, const int *row_id_map,
                                    const void *merging_probs, int probs_dtype, void *act_grad, void *probs_grad, void *stream);

/* ---- gated activations and RMSNorm: the element-wise steps either side of the low-precision GEMMs -------------------- */

/* out[r, :H] = act(x[r, :H]) * x[r, H:2H] * probs[r], computed in fp32 and rounded to dtype; act: 0 = SiLU (SwiGLU),
 * 1 = GELU in its erf form (GeGLU).  row_mask (int64 [rows], optional): rows with a zero entry are not computed and
 * come out as zeros.  Rows of x and out must be 16-byte multiples.
 * Replaces swiglu_fwd_with_probs / geglu_fwd_with_probs (primus_turbo/pytorch/kernels/activation/{swiglu,geglu}_impl.py,
 * kernels in primus_turbo/triton/activation/{swiglu,geglu}_kernel.py of the reference). */
int pt_glu_fwd(const void *x, int dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, void *out, void *stream);

/* grad_x[r, :H] = g * p * b * act'(a), grad_x[r, H:] = g * p * act(a), grad_probs[r] = sum_h g * act(a) * b (fp32).
 * The GELU branch uses the derivative of the forward's erf form; the reference's GeGLU backward kernel multiplies the
 * incoming gradient in twice (geglu_kernel.py, backward), which only agrees with autograd for a gradient of ones.
 * Replaces swiglu_bwd_with_probs / geglu_bwd_with_probs of the reference. */
int pt_glu_bwd(const void *grad_out, const void *x, int dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act,
               void *grad_x, float *grad_probs, void *stream);

/* y[r] = (x[r] (+ residual[r])) * rstd[r] * g, rstd[r] = rsqrt(mean(x^2) + eps) in fp32, g = gamma or 1 + gamma
 * (zero_centered).  With a residual the sum is rounded to dtype, written to x_plus_r and normalised from that rounded
 * value.  y may be null: only rstd (and x_plus_r) are produced.
 * Replaces rmsnorm_fwd_impl / rmsnorm_fwd_residual_impl (primus_turbo/pytorch/kernels/normalization/rmsnorm_impl.py,
 * kernels in primus_turbo/triton/normalization/rmsnorm_kernel.py of the reference). */
int pt_rmsnorm_fwd(const void *x, const void *residual, const void *gamma, int dtype, float eps, int zero_centered, int64_t rows, int64_t H, void *y,
                   void *x_plus_r, float *rstd, void *stream);

/* Number of partial dgamma rows pt_rmsnorm_bwd needs for this row count (dg_partial is fp32 [parts, H]). */
int pt_rmsnorm_bwd_parts(int64_t rows);

/* dx = (dy * g - x_hat * mean(dy * g * x_hat)) * rstd (+ dxpr), x_hat = x * rstd; dgamma[h] = sum_r dy * x_hat,
 * accumulated in fp32 through dg_partial and rounded to dtype.  dxpr (optional) is the gradient that reached x_plus_r.
 * Replaces rmsnorm_bwd_impl / rmsnorm_bwd_residual_impl of the reference. */
int pt_rmsnorm_bwd(const void *dy, const void *dxpr, const void *x, const void *gamma, const float *rstd, int dtype, int zero_centered, int64_t rows,
                   int64_t H, void *dx, void *dgamma, float *dg_partial, int parts, void *stream);

/* MX quantization of a gated activation in one pass: what pt_glu_fwd followed by pt_quantize_mx (flags PT_MX_ROW |
 * PT_MX_COL) writes, byte for byte, without the [rows, H] intermediate in memory.  x bf16 [rows, 2H]; H a multiple of 64;
 * fmt PT_E4M3 or PT_E2M1; outputs laid out as pt_quantize_mx's.  With fmt PT_E2M1 the flags may add PT_MX_COL_RHT (the
 * transposed copy is taken of the 16-point Hadamard transform, as the MXFP4 recipe lays out its wgrad operand); no other
 * option flags.  PT_ERR_UNSUPPORTED outside that range (the caller then runs the two kernels).  Covers the SwiGLU -> quantize step between the two grouped GEMMs of an expert MLP
 * (primus_turbo/pytorch/ops/activation.py:72-80 followed by quantize_fp8 in ops/grouped_gemm_fp8.py of the reference). */
int pt_glu_quantize_mx(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int fmt,
                       unsigned flags, void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream);

/* The same with the rows split into G groups: what pt_glu_fwd followed by pt_grouped_quantize_mx writes. */
int pt_grouped_glu_quantize_mx(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int G,
                               const int64_t *group_offs, const int64_t *padded_offs_row, const int64_t *padded_offs_col, int fmt, unsigned flags,
                               void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, int64_t col_alloc, void *stream);

/* MX quantization of RMSNorm(x) given the row statistics (pt_rmsnorm_fwd with y = null): what pt_rmsnorm_fwd followed by
 * pt_quantize_mx writes, byte for byte.  x, gamma bf16; H a multiple of 32.
 * (primus_turbo/pytorch/ops/normalization.py rmsnorm followed by quantize_fp8 of the reference.) */
int pt_rmsnorm_quantize_mx(const void *x, int x_dtype, const float *rstd, const void *gamma, int zero_centered, int64_t rows, int64_t H, int fmt,
                           unsigned flags, void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream);

/* Gated activation and the row-wise MX copy in one pass (forward-only callers: no transposed copy): what pt_glu_fwd followed
 * by pt_quantize_mx (flags PT_MX_ROW) writes, byte for byte.  x bf16 [rows, 2H]; H a multiple of 32 (else
 * PT_ERR_UNSUPPORTED); fmt PT_E4M3, PT_E5M2 or PT_E2M1; q_row [rows, ceil(H, 128)] codes, s_row [rows, ceil(H, 128) / 32].
 * (primus_turbo/pytorch/ops/activation.py:72-80 followed by quantize_fp8 of the reference.) */
int pt_glu_quantize_mx_row(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int fmt,
                           void *q_row, uint8_t *s_row, void *stream);

/* RMSNorm and the row-wise MX copy in one pass over x (forward-only callers need no transposed copy): writes rstd [rows]
 * and what pt_rmsnorm_fwd followed by pt_quantize_mx (flags PT_MX_ROW) writes, byte for byte, without y in memory.
 * x, gamma bf16; fmt PT_E4M3, PT_E5M2 or PT_E2M1; q_row [rows, ceil(H, 128)] codes (half the bytes for e2m1), s_row
 * [rows, ceil(H, 128) / 32].  PT_ERR_UNSUPPORTED when H is not a multiple of 32 or exceeds 8192 (the caller then runs
 * the two kernels).  (primus_turbo/pytorch/ops/normalization.py rmsnorm followed by quantize_fp8 of the reference.) */
int pt_rmsnorm_quantize_mx_row(const void *x, int x_dtype, const void *gamma, float eps, int zero_centered, int64_t rows, int64_t H,
                               int fmt, void *q_row, uint8_t *s_row, float *rstd, void *stream);

/* ---- pre-shuffled MX layouts (the tile orders the reference hands to its pre-shuffled GEMM back ends) ----------------
 * Replaces torch.ops.primus_turbo_cpp_extension.shuffle_scale / shuffle_weight of the reference
 * (csrc/pytorch/shuffle/shuffle.cpp:16-92, csrc/kernels/shuffle/shuffle.cu:33-118, index rules
 * csrc/include/primus_turbo/device/shuffle.cuh:39-80) and the shuffle_scale / shuffle_out options of its MX quantizers
 * (csrc/pytorch/quantization/quantization.cpp:795-830), which write the same bytes.
 *
 * pt_shuffle_e8m0_scale: scale ue8m0 [M, N] -> out [ceil(M, 256), ceil(N, 8)] bytes, padding 0; element (row, col) at
 *   ((row / 32) * (N_pad / 8) + col / 8) * 256 + (col % 4) * 64 + (row % 16) * 4 + ((col % 8) / 4) * 2 + (row % 32) / 16.
 * pt_shuffle_mx_codes: codes [M, row_bytes] (packed e2m1 pairs or fp8 bytes), M % 16 == 0, row_bytes % 32 == 0 -> out of
 *   the same size; byte (row, col) at (row / 16) * (row_bytes * 16) + (col / 32) * 512 + ((col % 32) / 16) * 256 +
 *   (row % 16) * 16 + col % 16.  Both pointers 16-byte aligned; out must not overlap the input. */
int pt_shuffle_e8m0_scale(const uint8_t *scale, int64_t M, int64_t N, uint8_t *out, void *stream);
int pt_shuffle_mx_codes(const void *codes, int64_t M, int64_t row_bytes, void *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PT_B200_H_ */
