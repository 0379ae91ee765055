/*
 * splat_b200 -- C ABI of the B200 (sm_100a) implementation of SPLAT's sparse-regular attention
 * path over the ACSR ("affine compressed sparse row") format:
 *
 *     ACSR metadata  ->  SDDMM (Q.K^T at the affine non-zeros)  ->  row softmax  ->  SpMM (P.V)
 *
 * This header is the whole boundary: plain C types, device pointers passed as void* / typed
 * pointers, sizes as int64_t, the CUDA stream as an opaque void* (a cudaStream_t).  Every function
 * returns a splat_status (0 = ok, negative = error), never throws, never allocates device memory
 * and never synchronises the device; work is enqueued on the stream the caller passes.
 *
 * Each entry point names the function of the reference project it stands in for (paths are
 * relative to the reference repository, spikerheado1234/triton-fun).
 *
 * ACSR conventions (SPLAT/acsr_helpers.py:99-160): for row i, sparse slot j < nnz_i is dense
 * column start_i + j*stride_i.  The reference hands its kernels five float32 arrays of length L:
 *     dTos_lin = 1/stride, dTos_tr = -(start/stride), sTod_lin = stride, sTod_tr = start/stride,
 *     nnzs = nnz
 * plus per-row-block span arrays.  The kernels here take the same float32 arrays (only sTod_lin,
 * sTod_tr and nnzs are read, as in the reference kernels) and recover integers as
 *     stride = rint(sTod_lin), start = rint(sTod_tr * sTod_lin), nnz = rint(nnzs).
 * Sparse operands are stored as (BH, L, trailing_dim) with trailing_dim = max_i nnz_i.
 * A problem with no work (BH * L = 0) returns SPLAT_OK without a launch; its data pointers may be
 * null (an empty torch tensor has a null data pointer).
 */
#ifndef SPLAT_B200_H
#define SPLAT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPLAT_B200_VERSION 100

/* Capacity of the fixed intermediate buffer used by splat_attention_noalloc. */
#define SPLAT_NOALLOC_SCRATCH_BYTES (64ll << 20)

typedef enum {
    SPLAT_OK = 0,
    SPLAT_ERR_BAD_ARG = -1,          /* null pointer, negative size, inconsistent sizes        */
    SPLAT_ERR_UNSUPPORTED_DTYPE = -2,
    SPLAT_ERR_MISALIGNED = -3,       /* a pointer or stride breaks an alignment the path needs  */
    SPLAT_ERR_LAUNCH = -4,           /* CUDA reported an error at launch                        */
    SPLAT_ERR_DEVICE_TIMEOUT = -5,   /* a bounded device-side wait gave up (see status words)   */
    SPLAT_ERR_UNSUPPORTED_SHAPE = -6,/* shape outside what the requested path implements        */
    SPLAT_ERR_DRIVER = -7,           /* tensor-map encoding / driver entry point failure        */
    SPLAT_ERR_NO_DEVICE = -8,
    SPLAT_ERR_SCRATCH_TOO_SMALL = -9 /* problem exceeds the fixed buffer of splat_attention_noalloc */
} splat_status;

typedef enum { SPLAT_F32 = 0, SPLAT_F16 = 1, SPLAT_BF16 = 2 } splat_dtype;

/* Mask patterns with a closed form.  0-2 are the reference generators
 * (SPLAT/acsr_helpers.py:18-55); 3-4 are the two benchmark patterns it has no generator for. */
typedef enum {
    SPLAT_PATTERN_BLOCKED = 0,          /* p0 = block size                                    */
    SPLAT_PATTERN_WINDOWED = 1,         /* p0 = half width: |i-j| <= p0                       */
    SPLAT_PATTERN_CAUSAL_WINDOWED = 2,  /* p0: i-p0 <= j <= i                                 */
    SPLAT_PATTERN_STRIDED = 3,          /* p0 = stride: j = (i mod p0) + p0*k, j <= i         */
    SPLAT_PATTERN_DILATED = 4           /* p0 = taps, p1 = dilation: j = i - p1*k, k < p0     */
} splat_pattern;

/* Which fused-attention kernel to run. */
typedef enum {
    SPLAT_PATH_AUTO = 0,     /* band kernel when the plan allows it, else generic             */
    SPLAT_PATH_GENERIC = 1,  /* CUDA-core kernel, any metadata, any dtype                     */
    SPLAT_PATH_BAND = 2      /* TMA + tcgen05 kernel; error if the shape does not qualify      */
} splat_path;

int32_t splat_version(void);
const char* splat_status_string(int32_t status);

/* ---------------------------------------------------------------------------------------------
 * ACSR metadata.
 * ------------------------------------------------------------------------------------------- */

/* Per-row summary of an L_rows x L_cols uint8 mask resident on the device (row stride ld bytes).
 * rows_i32 receives 4*L_rows int32: first set column, second set column, last set column, count
 * (-1 where absent), laid out as four arrays of length L_rows.
 * Stands in for the row scans of SPLAT/acsr_helpers.py:110-117 and SPLAT/r_sddmm.py:129-135. */
int32_t splat_mask_row_summary_u8(const uint8_t* mask, int64_t n_rows, int64_t n_cols, int64_t ld,
                                  int32_t* rows_i32, void* stream);

/* The same summary from a closed-form pattern; no mask is read.  Stands in for
 * SPLAT/acsr_helpers.py:18-55 followed by the row scans above. */
int32_t splat_pattern_row_summary(int32_t kind, int64_t n, int64_t p0, int64_t p1,
                                  int32_t* rows_i32, void* stream);

/* Write the n x n uint8 mask of a pattern (row stride ld bytes).
 * Stands in for create_blocked_mask / create_windowed_mask / create_causal_windowed_mask
 * (SPLAT/acsr_helpers.py:18-55). */
int32_t splat_pattern_mask_u8(int32_t kind, int64_t n, int64_t p0, int64_t p1, uint8_t* mask,
                              int64_t ld, void* stream);

/* Row summary -> the reference's float32 metadata.  Outputs: five arrays of n_rows floats
 * (dTos_lin, dTos_tr, sTod_lin, sTod_tr, nnzs), two arrays of ceil(n_rows/block_height) floats
 * (span_start, span_end: per row block, min start/stride and max nnz*stride + start/stride, initial
 * values n_cols and -1), and trailing_dim_dev[0] = max_i nnz_i (a device int32, cleared here).
 * Values are computed in float64 and rounded once to float32, which reproduces the reference's
 * tensors bit for bit.  Stands in for instantiate_metadata + create_acsr
 * (SPLAT/acsr_helpers.py:99-160). */
int32_t splat_acsr_from_row_summary(const int32_t* rows_i32, int64_t n_rows, int64_t n_cols,
                                    int32_t block_height, float* dTos_lin, float* dTos_tr,
                                    float* sTod_lin, float* sTod_tr, float* nnzs,
                                    float* span_start, float* span_end, int32_t* trailing_dim_dev,
                                    void* stream);

/* Classify float32 metadata for kernel selection.  plan_i32 (device, 8 ints) receives
 *   [0] max nnz              [1] min stride over rows with nnz > 1 (INT_MAX if none)
 *   [2] max stride (same rows)   [3] rows with nnz > 1 whose start mod stride != row mod stride
 *   [4] rows with nnz == 1   [5] max column + 1   [6] rows with nnz == 0   [7] rows with nnz > 1
 * The band kernel applies when [1] == [2], [3] == 0 and n_rows is a multiple of the stride.
 * No counterpart in the reference (it has a single kernel per operator). */
int32_t splat_acsr_classify(const float* sTod_lin, const float* sTod_tr, const float* nnzs,
                            int64_t n_rows, int32_t* plan_i32, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The three operators.  Layouts: Q, V, O are (BH, L, d) contiguous; K is addressed as
 * K[bh][col][k] = k_ptr[bh*k_stride_bh + col*k_stride_col + k*k_stride_k] (element strides), which
 * covers both a contiguous (BH, d, L) K^T (stride_col = 1, stride_k = L) and the transposed view
 * of a (BH, L, d) tensor (stride_col = d, stride_k = 1).  S and P are (BH, L, trailing_dim).
 * Inputs and outputs share one dtype; accumulation is fp32 (true fp32 FMA for SPLAT_F32).
 * Slots >= nnz_i of S and P rows are written as zero.
 * ------------------------------------------------------------------------------------------- */

/* S[bh,i,j] = sum_k Q[bh,i,k] * K[bh,start_i + j*stride_i,k], j < nnz_i.
 * Stands in for rsddmm_launcher -> rsddmm_kernel (SPLAT/r_sddmm.py:16-115,171-184). */
int32_t splat_sddmm(const void* q, const void* k, int64_t k_stride_bh, int64_t k_stride_col,
                    int64_t k_stride_k, void* s_out, const float* sTod_lin, const float* sTod_tr,
                    const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                    int64_t trailing_dim, int32_t dtype, void* stream);

/* P[bh,i,j] = softmax_j(scale * S[bh,i,j]) over j < nnz_i, for ALL rows.  s_in == p_out (in place)
 * is allowed.
 * Stands in for rsoftmax_launcher -> r_softmax_1d_kernel (SPLAT/r_softmax.py:17-59,126-150);
 * the reference applies no scale (scale = 1). */
int32_t splat_softmax(const void* s_in, void* p_out, const float* nnzs, int64_t bh, int64_t n_rows,
                      int64_t trailing_dim, float scale, int32_t dtype, void* stream);

/* O[bh,i,c] = sum_{j<nnz_i} P[bh,i,j] * V[bh,start_i + j*stride_i,c].
 * Stands in for rspmm_launcher -> r_spmm_kernel_row_maj_row_comp (SPLAT/r_spmm.py:14-126,148-164). */
int32_t splat_spmm(const void* p, const void* v, void* o, const float* sTod_lin,
                   const float* sTod_tr, const float* nnzs, int64_t bh, int64_t n_rows,
                   int64_t n_cols, int64_t d, int64_t trailing_dim, int32_t dtype, void* stream);

/* O = softmax(scale * Q.K^T restricted to the ACSR non-zeros) . V in one kernel; scores never
 * reach global memory.  Stands in for the three launches of RegularAttention.forward
 * (SPLAT/r_attention.py:77-100).
 *   path ........ a splat_path value
 *   plan_i32 .... HOST pointer to a copy of the 8 ints of splat_acsr_classify, or NULL (then only
 *                 the generic kernel can run)
 *   status_word . device int32 the band kernel sets non-zero if one of its bounded waits gives up;
 *                 may be NULL for the generic path.  The caller clears and reads it.  WHILE THE WORD
 *                 IS NON-ZERO EVERY TENSOR-CORE KERNEL THAT IS GIVEN IT RETURNS AT ENTRY WITHOUT
 *                 WRITING ITS OUTPUT (the entry point still returns SPLAT_OK: nothing is known at
 *                 enqueue time).  Read the word wherever the stream is synchronised anyway; a
 *                 non-zero value means the outputs of that launch and of every later one are not
 *                 valid until the word is cleared.
 * Under SPLAT_PATH_AUTO a band path that does not apply (shape, pattern, operand alignment, no
 * tensor-map support in the driver) falls through to the generic kernel. */
int32_t splat_attention_fused(const void* q, const void* k, int64_t k_stride_bh,
                              int64_t k_stride_col, int64_t k_stride_k, const void* v, void* o,
                              const float* sTod_lin, const float* sTod_tr, const float* nnzs,
                              int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d, float scale,
                              int32_t dtype, int32_t path, const int32_t* plan_i32,
                              int32_t* status_word, void* stream);

/* The same call with one more output: *path_ran (HOST int32, may be NULL) receives SPLAT_PATH_BAND or
 * SPLAT_PATH_GENERIC according to the kernel that was enqueued (SPLAT_PATH_AUTO: none).  A caller
 * uses it to know whether status_word can have been touched.  Same reference counterpart as
 * splat_attention_fused. */
int32_t splat_attention_fused_ex(const void* q, const void* k, int64_t k_stride_bh,
                                 int64_t k_stride_col, int64_t k_stride_k, const void* v, void* o,
                                 const float* sTod_lin, const float* sTod_tr, const float* nnzs,
                                 int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d, float scale,
                                 int32_t dtype, int32_t path, const int32_t* plan_i32,
                                 int32_t* status_word, int32_t* path_ran, void* stream);

/* splat_attention_fused_ex with the softmax normaliser as a second output: lse (DEVICE fp32,
 * (BH, n_rows), may be NULL = off) receives, per row, log(sum_j exp(scale * q_i . k_j)) over the
 * row's non-zeros (natural logarithm; -inf for a row without non-zeros), from either kernel.  It is
 * what a backward pass over the same tiles recomputes the probabilities from.  Counterpart in the
 * reference: none -- its module has no gradient path (SPLAT/r_attention.py:12-100) and its softmax
 * kernel keeps the row maximum and sum in registers only (SPLAT/r_softmax.py:17-58). */
int32_t splat_attention_fused_lse(const void* q, const void* k, int64_t k_stride_bh,
                                  int64_t k_stride_col, int64_t k_stride_k, const void* v, void* o,
                                  float* lse, const float* sTod_lin, const float* sTod_tr,
                                  const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols,
                                  int64_t d, float scale, int32_t dtype, int32_t path,
                                  const int32_t* plan_i32, int32_t* status_word, int32_t* path_ran,
                                  void* stream);

/* The three-launch chain (SDDMM, softmax in place, SpMM) for callers that cannot allocate device
 * memory -- code running after its host application froze its memory pool, plug-ins that receive
 * input/output buffers but own no allocator, callers that must avoid cudaMalloc's device-wide
 * synchronisation.  The (bh, n_rows, trailing_dim) intermediate lives in a fixed 64 MiB array inside
 * the library (held by every GPU that uses the library, until the process exits), so this entry
 * point allocates nothing.  bh*n_rows*trailing_dim*sizeof(element) above
 * SPLAT_NOALLOC_SCRATCH_BYTES returns SPLAT_ERR_SCRATCH_TOO_SMALL and launches nothing.  The first
 * call on a device resolves the array's address there: make it before any stream capture.  All calls
 * on a device share the array: calls that can overlap on the GPU race; the array keeps the last
 * call's contents and nothing in it needs clearing.  Arguments as in splat_sddmm / splat_spmm.
 * This entry point has no counterpart in the reference. */
int32_t splat_attention_noalloc(const void* q, const void* k, int64_t k_stride_bh,
                                int64_t k_stride_col, int64_t k_stride_k, const void* v, void* o,
                                const float* sTod_lin, const float* sTod_tr, const float* nnzs,
                                int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                                int64_t trailing_dim, float scale, int32_t dtype, void* stream);

/* Tensor-core SDDMM and SpMM for ACSR patterns whose rows are contiguous bands after regrouping by
 * residue class (the condition of SPLAT_PATH_BAND above): same operands and results as splat_sddmm /
 * splat_spmm (replacing SPLAT/r_sddmm.py:171-184 and SPLAT/r_spmm.py:148-164 for such patterns),
 * 16-bit dtypes, d = 64 or 128, K given as the transposed view of a contiguous (BH, L, d) array.
 * plan_i32 = the 8 host integers of splat_acsr_classify, status_word as in splat_attention_fused.
 * SPLAT_ERR_UNSUPPORTED_SHAPE means "use splat_sddmm / splat_spmm"; nothing was launched. */
int32_t splat_sddmm_band(const void* q, const void* k, int64_t k_stride_bh, int64_t k_stride_col,
                         int64_t k_stride_k, void* s_out, const float* sTod_lin, const float* sTod_tr,
                         const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                         int64_t trailing_dim, int32_t dtype, const int32_t* plan_i32,
                         int32_t* status_word, void* stream);
int32_t splat_spmm_band(const void* p, const void* v, void* o, const float* sTod_lin,
                        const float* sTod_tr, const float* nnzs, int64_t bh, int64_t n_rows,
                        int64_t n_cols, int64_t d, int64_t trailing_dim, int32_t dtype,
                        const int32_t* plan_i32, int32_t* status_word, void* stream);

/* Self-test of the bounded device-side wait used by the tensor-core kernels: one CTA waits on an
 * mbarrier that nothing arrives on, gives up after limit_cycles SM clocks (1 .. 2e9), stores code
 * 99 in *status_word (device int32, cleared by the caller) and ends normally; the context stays
 * usable.  No counterpart in the reference. */
int32_t splat_selftest_bounded_wait(int32_t* status_word, int64_t limit_cycles, void* stream);

/* Checked-index mode of the CUDA-core kernels (splat_sddmm, splat_spmm and the CUDA-core path of
 * splat_attention_fused).  While a device int32 is registered, every dense column the kernels
 * derive from the row metadata (start + j * stride) is compared with [0, n_cols) before it is
 * dereferenced; a column outside the range is clamped to the nearest valid one and the kernel's
 * code is stored in the word if it still holds 0 (71 = SDDMM, 72 = SpMM, 73 = fused).  Null (the
 * default) switches the comparison off.  The setting is process-wide and is read at each launch;
 * the word must stay valid until the launches that saw it have completed.  Counterpart in the
 * reference: none (its kernels index K and V by raw pointer arithmetic,
 * SPLAT/r_sddmm.py:24-37, SPLAT/r_spmm.py:24-38). */
int32_t splat_debug_check_indices(int32_t* status_word);

#ifdef __cplusplus
}
#endif
#endif /* SPLAT_B200_H */
