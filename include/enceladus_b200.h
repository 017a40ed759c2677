/*
 * enceladus_b200 — C ABI of the sm_100a kernel library (libenc_b200.so).
 *
 * This is the boundary a binding generator (ctypes, cffi, nanobind, cgo ...) binds.  It replaces, for
 * the kernel set, what the reference reaches through its generic Metal runtime:
 *   fr_stream_dispatch(stream, pso, name, plan, bufs, offsets, scalar_bytes, grid, tg)
 *                                                     src/enceladus/_C/enceladus_rt.h:137-139
 *   Stream.dispatch(...) in the nanobind module       src/enceladus/_C/bindings.mm:479-490
 *   CompiledKernel.launch(grid, values)               src/enceladus/runtime/launcher.py:457-512
 * The reference dispatches a JIT-compiled pipeline with an untyped binding plan; here every kernel of
 * the set is a typed entry point.  Conventions shared by all entry points:
 *
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer on the current CUDA device
 *     unless the parameter name ends in `_host`;
 *   - the caller owns all buffers.  The library itself owns, per device: a 256-byte status block (bounded
 *     device-side waits report there) and the tile-descriptor scratch of enc_cumsum / enc_sum (see
 *     enc_cumsum); both are allocated on first use and freed at exit.  No other entry point allocates;
 *   - `stream` is a cudaStream_t / CUstream passed as void* (NULL = the legacy default stream); work
 *     is enqueued and the call returns without synchronising, like fr_stream_dispatch;
 *   - the return value is an enc_status; on failure enc_last_error() holds a message for the calling
 *     thread (the reference returns nonzero plus a message buffer, enceladus_rt.h:78-83,143-145);
 *   - sizes and strides are in ELEMENTS, 64-bit;
 *   - `variant` selects one of the hand-written tile variants of a kernel (0 .. enc_num_variants-1),
 *     or ENC_VARIANT_AUTO for the built-in choice; the autotuner iterates over them.
 */
#ifndef ENCELADUS_B200_H
#define ENCELADUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ENC_OK = 0,
    ENC_ERR_BAD_ARG = 1,      /* NULL pointer, negative size, unknown dtype/variant            */
    ENC_ERR_UNSUPPORTED = 2,  /* valid request this build has no kernel for                    */
    ENC_ERR_LAUNCH = 3,       /* CUDA reported an error at launch / in an earlier async launch */
    ENC_ERR_DEVICE_WAIT = 4,  /* a bounded device-side wait ran out (reported at sync)         */
    ENC_ERR_NO_MEMORY = 5     /* scratch allocation failed                                     */
} enc_status;

typedef enum {
    ENC_F32 = 0,
    ENC_F16 = 1,
    ENC_BF16 = 2,
    ENC_I32 = 3,
    ENC_I8 = 4,
    ENC_I16 = 5,
    ENC_I64 = 6,
    ENC_U8 = 7
} enc_dtype;

typedef enum {
    ENC_K_SOFTMAX = 0,
    ENC_K_LAYERNORM = 1,
    ENC_K_RMSNORM = 2,
    ENC_K_GELU = 3,
    ENC_K_MATMUL = 4,
    ENC_K_ATTENTION = 5,
    ENC_K_HISTOGRAM = 6,
    ENC_K_CUMSUM = 7,
    ENC_K_ADD = 8,
    ENC_K_MATMUL_INT = 9,
    ENC_K_COUNT = 10
} enc_kernel;

#define ENC_VARIANT_AUTO (-1)

/* ---- library / device -------------------------------------------------------------------- */

/* Message for the last failure on the calling thread ("" if none).  Replaces the `char *err`
 * out-parameters of fr_library_new / fr_stream_sync (enceladus_rt.h:78-83,143-145). */
const char *enc_last_error(void);

typedef struct {
    int device;               /* current CUDA device ordinal                         */
    int sm_count;             /* multiprocessors                                     */
    int cc_major, cc_minor;   /* compute capability                                  */
    int max_smem_per_block;   /* opt-in shared memory per block, bytes               */
    int l2_bytes;
    uint64_t global_mem;      /* bytes                                               */
    char name[128];
} enc_device_info_t;

/* Replaces fr_device_query / fr_device_name (enceladus_rt.h:29-33). */
int enc_device_info(enc_device_info_t *out);

/* Number of hand-written tile variants of a kernel, and a one-line description of one
 * ("rows_per_cta=8 threads_per_row=32", "tile=128x256x64 stages=4", ...).  The autotuner uses
 * these in place of the reference's (BM, BN, BK, num_warps) config lists (src/enceladus/configs.py:19-44). */
int enc_num_variants(int kernel);
int enc_variant_info(int kernel, int variant, char *out, size_t n);

/* Waits for `stream` and reports errors of earlier asynchronous launches, including a bounded
 * device-side wait that ran out (ENC_ERR_DEVICE_WAIT).  Replaces fr_stream_sync (enceladus_rt.h:143-145). */
int enc_synchronize(void *stream);

/* ---- bandwidth-bound kernels -------------------------------------------------------------- */

/* Row softmax over the last axis, float32 math, output in the input dtype.
 * Replaces softmax_kernel[(rows,)](out, in, stride_in, stride_out, n_cols, BLOCK)   examples/02_softmax.py:15-38
 * dtype: ENC_F32 | ENC_F16 | ENC_BF16.  Rows may be strided; elements of a row are contiguous. */
int enc_softmax(const void *in, void *out, int64_t rows, int64_t cols, int64_t stride_in,
                int64_t stride_out, int dtype, int variant, void *stream);

/* LayerNorm forward: y = (x-mean)*rstd*w + b, mean/rstd float32 per row (biased variance: one pass of sum and
 * sum of squares, the centred second pass of the reference for rows with mean^2 > 16 var).
 * Replaces layernorm_kernel[(rows,)](x, y, w, b, mean, rstd, stride_x, stride_y, n_cols, eps, BLOCK)
 *                                                                                    examples/03_layernorm.py:15-57
 * x, y, w, b share `dtype`.  mean / rstd may be NULL (not written). */
int enc_layernorm(const void *x, void *y, const void *w, const void *b, float *mean, float *rstd,
                  int64_t rows, int64_t cols, int64_t stride_x, int64_t stride_y, float eps,
                  int dtype, int variant, void *stream);

/* RMSNorm forward: y = x * (1/sqrt(mean(x^2)+eps)) * w.
 * Replaces rmsnorm_kernel[(rows,)](x, w, out, stride_x, stride_out, n_cols, eps, BLOCK)  examples/06_rmsnorm.py:15-37 */
int enc_rmsnorm(const void *x, const void *w, void *y, int64_t rows, int64_t cols,
                int64_t stride_x, int64_t stride_y, float eps, int dtype, int variant, void *stream);

/* Fused elementwise GELU: t = x*scale + bias[i % n_cols]; out = gelu(t).
 * mode 0 = erf form (0.5*t*(1+erf(t*0.70710677f))), mode 1 = tanh form
 * (0.5*t*(1+tanh(0.7978846f*(t+0.044715f*t^3)))).  bias may be NULL (then no bias is added and
 * n_cols is ignored); scale is applied only when has_scale != 0.
 * Replaces fused_gelu_kernel[(cdiv(n,BLOCK),)](x, bias, out, n, n_cols, scale, BLOCK)    examples/05_fused_gelu.py:17-33 */
int enc_gelu(const void *x, const void *bias, void *out, int64_t n, int64_t n_cols, float scale,
             int has_scale, int mode, int dtype, int variant, void *stream);

/* out = x + y.  Replaces add_kernel  examples/01_vector_add.py:15-22 */
int enc_add(const void *x, const void *y, void *out, int64_t n, int dtype, int variant, void *stream);

/* ---- integer kernels ---------------------------------------------------------------------- */

/* hist[b] += #{ i : floor((float(x[i]) - lo) * inv_width) == b, 0 <= b < num_bins }, int32 counts.
 * `hist` is accumulated into (the caller zero-fills it, as enceladus.new_zeros does).
 * Replaces histogram_kernel[(cdiv(n,BLOCK),)](x, hist, n, lo, inv_width, NUM_BINS, BLOCK)  examples/09_histogram.py:17-34
 * dtype: ENC_F32 | ENC_F16 | ENC_BF16 | ENC_I32. */
int enc_histogram(const void *x, int32_t *hist, int64_t n, float lo, float inv_width,
                  int64_t num_bins, int dtype, int variant, void *stream);

/* Inclusive scan along rows: out[r, c] = sum_{c' <= c} in[r, c'] (or c' >= c when reverse != 0).
 * Integers narrower than 32 bits accumulate and are written as int32; int32 wraps modulo 2^32;
 * float16/bfloat16 accumulate in float32 and are rounded on store; out dtype = enc_cumsum_out_dtype.
 * rows == 1 is the flat form (any length, single-pass decoupled look-back over tiles).
 * `seed` (device pointer to ONE accumulator-typed value, or NULL) is added to every output of the
 * flat form: the exclusive offset of this shard when one array is split across GPUs.
 * Scratch: the flat form keeps 8 bytes per 4096-element tile plus a 64-byte header in a per-device
 * buffer the library allocates on first use and grows on demand (cudaMalloc; freed at exit).
 * Replaces cumsum_kernel[(cdiv(rows,BLOCK_M),)](out, in, n_rows, n_cols, stride_in, stride_out, REVERSE, ...)
 *                                                                                    examples/10_cumsum.py:17-42 */
int enc_cumsum(const void *in, void *out, int64_t rows, int64_t cols, int64_t stride_in,
               int64_t stride_out, int reverse, int dtype, const void *seed, int variant,
               void *stream);
int enc_cumsum_out_dtype(int dtype);

/* The flat form of enc_cumsum (rows == 1, forward) for callers that must not allocate device memory:
 * a framework that owns the whole device through its own pool, a serving loop that cannot take the
 * device-wide stall of an allocation, code under a "nothing is allocated after start-up" rule.  This
 * entry point has no counterpart in the reference.  It calls no cudaMalloc/cudaFree or other allocating
 * routine; the look-back descriptors live in a 1 MiB array inside the library image (held by every GPU
 * that loads the library until the process exits), which limits n to 2^30 elements — longer inputs are
 * refused with ENC_ERR_UNSUPPORTED.  The first call on a device resolves the array's device address;
 * make that call before any stream capture.  Every call on a device shares the array: calls on one
 * stream are safe, calls that overlap on the GPU race.  `status` (device pointer owned by the caller, or
 * NULL) is set non-zero if a bounded device-side wait ran out, in which case the output is invalid.  With
 * status == NULL that timeout is recorded only in a spare word of the array that nothing reads, so the
 * failure is SILENT (enc_synchronize does not report it either): pass a status word unless a wrong output
 * would be caught downstream.  Same dtypes and results as enc_cumsum except ENC_I64. */
int enc_cumsum_noalloc(const void *in, void *out, int64_t n, int dtype, const void *seed,
                       unsigned *status, void *stream);

/* total[0] = sum of n elements in the accumulator type of enc_cumsum (int32 wrap / float32).
 * Pass 1 of the multi-GPU flat scan (local total -> all-gather -> seed).  No counterpart in the
 * reference, which has no multi-device path. */
int enc_sum(const void *in, void *total, int64_t n, int dtype, void *stream);

/* offset[0] = totals[0] + ... + totals[index-1] (0 for index 0) in the accumulator type of enc_cumsum for
 * `dtype` (32-bit wrap, float32 or int64 adds in shard order): the `seed` of shard `index` once the per-shard
 * totals of enc_sum have been all-gathered into `totals` (device, `count` values).  A one-thread kernel on
 * `stream`, so that the two passes of the multi-GPU scan and the collective between them stay stream-ordered
 * with no host round trip.  No counterpart in the reference (single device). */
int enc_scan_offset(const void *totals, int count, int index, void *offset, int dtype, void *stream);

/* ---- tensor-core kernels ------------------------------------------------------------------ */

/* C = epilogue(A @ B): A [M,K] (lda), B [K,N] (ldb), C [M,N] (ldc), all row-major with unit inner
 * stride, float32 accumulation on tcgen05 tensor cores (float32 operands: CUDA cores), C in the operand dtype.
 * epilogue 0: identity.  epilogue 1: t = acc + bias[n]; 0.5*t*(1+erf(t*0.70710677f)).
 * Out-of-range tile elements read as zero and are not stored (descriptor semantics,
 * src/enceladus/language/ops.py:495-514).  dtype: ENC_F16 | ENC_BF16 | ENC_F32.  Operands need no alignment:
 * 16-byte aligned bases and leading dimensions that are multiples of 8 are fetched by TMA, anything else (the
 * reference's 513^3 shape, benchmarks/bench_matmul.py:30) by loader warps inside the same tensor-core kernel;
 * nothing is copied or allocated.
 * Replaces matmul_bias_gelu_kernel[(cdiv(N,BN),cdiv(M,BM))](a, b, bias, c, M, N, K, lda, ldb, ldc, BM, BN, BK)
 *                                                                                    examples/07_matmul_fused.py:17-48
 * and matmul_desc_kernel                                                             examples/04_matmul.py:21-63 */
int enc_matmul(const void *a, const void *b, const void *bias, void *c, int64_t M, int64_t N,
               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int epilogue, int dtype,
               int variant, void *stream);

/* C = A @ B for integer operands: A [M,K] (lda), B [K,N] (ldb), both of `dtype`, C [M,N] int32 (ldc), row-major
 * with unit inner stride.  int32 accumulation, exact: products and sums wrap modulo 2^32
 * (integer tl.dot, src/enceladus/language/ops.py:1255-1259).  ENC_I8 and ENC_U8 run on the tcgen05 tensor cores
 * (kind::i8) when A and B are 16-byte aligned with leading dimensions that are multiples of 16, otherwise and for
 * ENC_I16 / ENC_I32 on CUDA cores.  Out-of-range tile elements read as zero and are not stored.
 * Replaces int8_matmul_kernel[(cdiv(N,BN),cdiv(M,BM))](a, b, c, M, N, K, BM, BN, BK)   benchmarks/bench_matmul.py:100-131
 * and the integer tl.dot kernels of                                                   tests/test_interpreter.py:808-835 */
int enc_matmul_int(const void *a, const void *b, void *c, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                   int64_t ldc, int dtype, int variant, void *stream);

/* Flash-attention forward over `bh` independent (batch, head) slices of shape [seq, head_dim]:
 * O = softmax(Q K^T * sm_scale [causal]) V, base-2 online softmax in float32, P rounded to the input
 * dtype before P@V, O in the input dtype.  lse (float32 [bh, seq], may be NULL) receives
 * ln2*(m + log2 l) of the running statistics.  stride_h = elements between slices, stride_m =
 * elements between rows (head_dim contiguous).  dtype: ENC_F16 | ENC_BF16 | ENC_F32; head_dim <= 128.
 * float16 / bfloat16 with head_dim 64 or 128, 16-byte aligned tensors and strides that are multiples of 8
 * run on the tcgen05 tensor cores; every other accepted shape runs on a CUDA-core kernel with the same
 * arithmetic.
 * Replaces attention_kernel[(cdiv(S,BLOCK_M), B*H)](q, k, v, o, sm_scale, N_CTX, stride_h, stride_m, HEAD_DIM, ...)
 *                                                                                    examples/08_flash_attention.py:30-103 */
int enc_attention_fwd(const void *q, const void *k, const void *v, void *o, float *lse, int64_t bh,
                      int64_t seq, int64_t head_dim, int64_t stride_h, int64_t stride_m,
                      float sm_scale, int causal, int dtype, int variant, void *stream);

/* ---- test hook ---------------------------------------------------------------------------- */

/* Forces the NEXT entry-point call on this thread to return `status` without launching anything
 * (host-side failure injection for the binding's error path; the reference injects failures with a
 * proxy around its native stream, tests/test_runtime.py:460-514).  0 clears it. */
void enc_test_fail_next(int status);

/* Launches one thread that polls a flag nothing sets, `polls` times at most (1 us apart, polls <=
 * 1000000), then gives up exactly as the library's bounded device-side waits do: it raises the device
 * status word and returns, so the next enc_synchronize reports ENC_ERR_DEVICE_WAIT and the context stays
 * usable.  Exercises the timeout path without hanging or faulting the GPU (the reference tests its
 * lost-sentinel timeout the same way, with a bounded wait: src/enceladus/runtime/stream.py:153-168). */
int enc_test_device_wait(unsigned int polls, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ENCELADUS_B200_H */
