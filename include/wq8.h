/* C ABI of libwgp_int8.so, the B200 (sm_100a) INT8 weight-linear library.
 *
 * Every entry point below replaces the entry point of the same name in the reference library
 * (wgpkernels/int8/int8_gemm.cu of WGPKernels, ABI 11); the reference's Python module binds them with
 * ctypes (wgpkernels/int8/__init__.py:73-89) and this library keeps names, argument order, argument
 * meaning and error codes, so that module can load this file unchanged.
 *
 * Conventions (same as the reference):
 *   - all pointers are device pointers owned by the caller unless stated; nothing is allocated here except
 *     the private buffer of wq8_l2_flush();
 *   - `stream` is a raw cudaStream_t of the CURRENT device; calls launch asynchronously and never synchronize;
 *   - return value: 0 = launched, > 0 = a cudaError_t, -1 = bad dtype / act / group, -2 = bad operands (shape, alignment, NULL),
 *     -3 = unknown variant, -4 = bad segments;
 *   - dtype: 0 = fp16, 1 = bf16, 2 = fp32 (quantizer inputs only, no input operation);
 *   - act: 0 none, 1 rms_norm (act_weight: K values of x's dtype or NULL; eps), 2 swiglu (x rows hold
 *     [gate (K) | value (K)]), 3 gelu (tanh approximation);
 *   - group: ConvRot rotation group, one of 0 (none), 16, 64, 256;
 *   - ldx: row stride of x in elements; rows of x are 16-byte aligned (8-byte for wq8_gemv_lines).
 */
#ifndef WQ8_H
#define WQ8_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* wq8_stream_t; /* cudaStream_t */

/* ABI version (11) and feature bits (bit 0: per-(n, 128-block of K) weight scales, variants 12-14).
 * Replaces int8_gemm.cu:1349-1352. */
int wq8_abi(void);
int wq8_features(void);

/* q (M, K) int8 and scale (M, ceil(K / 128)) fp32 of op(x): one scale per row and 128-element block of K.
 * K multiple of 8; M at most 65535 per call is NOT required here (any M).  inv_rms: M floats of scratch, only
 * read/written for rms_norm with K > 16384 (else may be NULL).  Replaces int8_gemm.cu:1936-1943. */
int wq8_quantize_blocks(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                        const void* act_weight, float eps, float* inv_rms, wq8_stream_t stream);

/* Row-wise INT8 of op(x): hi (M, K), scale (M) and, when lo is not NULL, the exact split
 * op(x) ~= scale * (hi + lo / 254).  Replaces int8_gemm.cu:1404-1414. */
int wq8_quantize(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                 const void* act_weight, float eps, wq8_stream_t stream);

/* out (M, K) = op(x), rotated, rounded once to x's dtype (fp16 / bf16): the activation of the few-token
 * paths.  Replaces int8_gemm.cu:1971-1977. */
int wq8_transform_rows(const void* x, void* out, int m, int k, int64_t ldx, int dtype, int group, int act, const void* act_weight,
                       float eps, wq8_stream_t stream);

/* out (M, K) = ConvRot rotation of x in groups of 16 / 64 / 256, normalised, rounded once.
 * Replaces int8_gemm.cu:1871-1876. */
int wq8_rotate_groups(const void* x, void* out, int m, int k, int64_t ldx, int dtype, int group, wq8_stream_t stream);

/* Y (M, N) = (A (M, K) * sa) @ (B (N, K) * sb).T + bias, or residual + rscale * (...), FP32 epilogue, one
 * rounding to dtype (fp16 / bf16); y may be the residual.  K multiple of 16; A, B, residual, y contiguous.
 * variant selects the mode (tile shapes are this library's own):
 *   0, 2, 6  'row'      sa (M)               sb (N)
 *   1, 7     'exact'    sa (M), a_lo given   sb (N)
 *   10, 11, 15, 16, 20  'block'  sa (M, ceil(K/128))  sb (N)      (15, 16: tiles of 128 output channels; 20: eight drain warps)
 *   12, 13, 22   'block+g'  sa (M, ceil(K/128))  sb (N, ceil(K/128))   (13: tiles of 128 output channels; 22: eight drain warps)
 *   14       'exact+g'  sa (M), a_lo given   sb (N, ceil(K/128))
 * a_lo must be non-NULL exactly for variants 1, 7, 14 (else -2).  split: accepted, tiles are never split along K
 * here.  workspace / counters: sizes from wq8_gemm_workspace(); variants 12-14 and 22 regroup the weight scales by
 * block of K into the workspace (16-byte aligned; NULL is -2), the other variants use neither.  sms: SM count
 * of the device.  Replaces int8_gemm.cu:1648-1656. */
int wq8_gemm(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias,
             const void* residual, const void* rscale, void* y, int m, int n, int k, int dtype, int variant, int sms, int split,
             int* workspace, int* counters, wq8_stream_t stream);

/* sizes[0] = workspace bytes, sizes[1] = counter bytes of wq8_gemm with these arguments.
 * Replaces int8_gemm.cu:1506-1528. */
void wq8_gemm_workspace(int m, int n, int k, int variant, int sms, int split, int64_t* sizes);

/* Default variant of the 'row' (hilo = 0) or 'exact' (hilo = 1) mode for a shape.  Replaces int8_gemm.cu:1564-1568. */
int wq8_gemm_select(int m, int n, int k, int hilo, int sms);

/* wq8_gemm of `count` (1 to 4) weights bs[s] (rows, K) of one input in ONE launch that reads the input once, outputs
 * ys[s] (M, rows) contiguous, rows a multiple of 8; per-channel weight scales only; biases[s] may be NULL; no residual.
 * A column tile never straddles two weights, so every output equals wq8_gemm's on that weight bit for bit.  -4 for bad
 * segments (count, rows, NULL entries, group-scaled variants).  Replaces int8_gemm.cu:1663-1676. */
int wq8_gemm_segments(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* const* bs, const float* const* sbs,
                      const void* const* biases, void* const* ys, int count, int rows, int m, int k, int dtype, int variant, int sms,
                      int split, int* workspace, int* counters, wq8_stream_t stream);

/* The CUDA-graph-loop forms: the same kernels on a window of rows whose position is read ON THE GPU when the kernel runs
 * (counter: device pointer to one int64 that a graph's loop body advances), so one captured launch serves every iteration.
 *   wq8_quantize_at / wq8_quantize_blocks_at: the INPUT rows are rows first + counter[0] * step ... of x; outputs start at row 0.
 *   wq8_gemm_at: the OUTPUT rows (and the residual's) are rows first + counter[0] * step ... of y; when in_first or in_step is
 *   non-zero the INPUT rows (a, a_lo and their scales) are rows in_first + counter[0] * in_step ...; span > 0: rscale holds
 *   scale_step values per span of output rows (a gate per frame), row r reads rscale[(shift + r) / span * scale_step + n].
 * counter == NULL: exactly the plain entry point.  The buffers must hold every row a counter value can address (rows past the
 * window are never read or written).  Replace int8_gemm.cu:1396-1402, :1926-1932, :1637-1645 (RowOffset, :238-244). */
int wq8_quantize_at(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                    const void* act_weight, float eps, const long long* counter, long long first, long long step, wq8_stream_t stream);
int wq8_quantize_blocks_at(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                           const void* act_weight, float eps, float* inv_rms, const long long* counter, long long first, long long step,
                           wq8_stream_t stream);
int wq8_gemm_at(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias,
                const void* residual, const void* rscale, void* y, int m, int n, int k, int dtype, int variant, int sms, int split,
                int* workspace, int* counters, const long long* counter, long long first, long long step, long long span,
                long long scale_step, long long in_first, long long in_step, wq8_stream_t stream);

/* Weight-only INT8 for at most 32 unquantized tokens: Y = X @ (W * sw).T + bias (+ residual), FP32
 * accumulation of exact products.  K multiple of 64; x and w 16-byte aligned, ldx a multiple of 8 (-2 otherwise).
 * slots / counters: scratch of the sizes wq8_small_workspace() reports (slots 256-byte aligned); counters zero on entry,
 * left zero.  With scratch and K a multiple of 128 the linear runs on tcgen05 (the activations as INT8 digit planes --
 * see wq8_stream_planes for their accuracy --, K ranges shared over all SMs, partial sums added in a fixed order);
 * without scratch (NULL) on the kernels that need none.  The digit split and the stream kernel of a call are launched with
 * programmatic stream serialization: each may start under the tail of the kernel before it on the stream (wq8_transform_rows lets
 * them) and waits for that kernel to finish before it reads what it wrote; callers need to do nothing.
 * Replaces int8_gemm.cu:1752-1759 and :1693-1697. */
int wq8_small(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
              void* y, int m, int n, int k, int dtype, int sms, float* slots, int* counters, wq8_stream_t stream);
void wq8_small_workspace(int m, int n, int k, int sms, int64_t* sizes);

/* The same linear for one to four tokens, K multiple of 4, no workspace; x 8-byte aligned, ldx a multiple of 4, w 4-byte
 * aligned (-2 otherwise).  Replaces int8_gemm.cu:1851-1858. */
int wq8_gemv_lines(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual,
                   const void* rscale, void* y, int m, int n, int k, int dtype, wq8_stream_t stream);

/* Reads `bytes` from a private cudaMalloc buffer on `stream` so that the next launch finds a cold L2 (tuner
 * timing).  Returns nonzero when the buffer cannot be allocated.  wq8_l2_flush_release() frees it.
 * Replaces int8_gemm.cu:1997-2016. */
int wq8_l2_flush(int device, int64_t bytes, wq8_stream_t stream);
void wq8_l2_flush_release(void);

/* ---- additions of this library (no counterpart in the reference) -------------------------------------- */

/* Exact INT32 block dot products S[b][m][n] = sum over block b of a[m, k] * b[n, k], written to
 * sums (ceil(K/128), M, N) int32 by the same tensor-core pipeline as wq8_gemm: the debug hook the parity
 * tests use to check the INT32 sums bit for bit. */
int wq8_debug_block_sums(const int8_t* a, const int8_t* b, int32_t* sums, int m, int n, int k, int sms, wq8_stream_t stream);

/* wq8_gemm with `count` (1 to 8) destinations of the same output: ys is a HOST array of device pointers, each to the first element
 * of an (M, N) block with row stride ld_y (elements) inside a wider matrix; the residual has row stride ld_residual.  The rank of an
 * N-sharded layer passes the position of its output columns in the full-width (M, N_total) buffers of all ranks (its own first;
 * the others peer-mapped), and the all-gather of the output happens inside the GEMM: the tile epilogue issues one TMA store per
 * destination.  Needs N, ld_y, ld_residual multiples of 8 and 16-byte aligned pointers when count > 1 (-2 otherwise).  The caller
 * orders the launch against the readers of the destinations (a barrier over the ranks before and after).  No split, no counters. */
int wq8_gemm_multi(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias,
                   const void* residual, int64_t ld_residual, const void* rscale, void* const* ys, int count, int64_t ld_y, int m, int n, int k,
                   int dtype, int variant, int sms, int* workspace, wq8_stream_t stream);

/* The few-token linear (at most 8 tokens, K multiple of 128) on INT8 tensor cores with the weights as they are: the activations are
 * first split into three planes of signed 7-bit digits per 128 values with one power of two (exact for every value within 2^14 of the
 * largest of its 128; smaller ones are rounded to nearest with an absolute error of at most 2^-21 of that largest value, unbiased),
 * into `workspace` (wq8_stream_planes_workspace() bytes, 16-byte aligned; 0 = the shape is not supported, use
 * wq8_gemv_lines / wq8_small).  Same arguments and error codes as wq8_small otherwise.  The reference has no counterpart: its few-token
 * kernels (and wq8_gemv_lines / wq8_small here) convert every weight byte to BF16 / FP16 instead, which bounds them below the HBM rate. */
int64_t wq8_stream_planes_workspace(int m, int n, int k, int sms);
int wq8_stream_planes(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                      void* y, int m, int n, int k, int dtype, int sms, void* workspace, wq8_stream_t stream);

/* wq8_small for callers that cannot allocate device memory (no counterpart in the reference, which always takes caller scratch).
 * A host that reaches this library through a bare FFI with buffers it was handed, a serving loop under a fixed memory budget, code
 * running during CUDA graph capture or in a section where cudaMalloc is not allowed: none of them can supply the K-split scratch
 * wq8_small asks for.  Here the scratch is a static device buffer inside the library (8 MiB + 4 KiB per GPU that loads it, held until
 * the process exits); nothing is allocated or freed.  The first call on a device looks up the buffer's device address and should come
 * before any stream capture.  Same arguments and error codes as wq8_small without `slots` / `counters`, the same kernel choice and so
 * the same values bit for bit; -5 when the shape's scratch exceeds the buffer.  All calls on a device share the buffer: calls whose
 * kernels can overlap on the GPU race. */
int wq8_small_static(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                     void* y, int m, int n, int k, int dtype, int sms, wq8_stream_t stream);

/* One bounded wait on a barrier that nothing ever completes, with a limit of `clocks` SM clocks (at most 2e9): the kernel writes
 * 2 to *returned (device int) when the wait gave up (1 if it completed), leaves `code` in the status word that
 * wq8_debug_status() reads, and returns.  The give-up path that every wait of this library shares, for tests: no fault, no trap. */
int wq8_debug_wait_probe(long long clocks, int code, int* returned, wq8_stream_t stream);

/* Device-side status word of the GEMM pipeline on the current device: 0, or a code left by a bounded wait
 * that gave up (the kernel then returned early with unspecified output).  Synchronizes the device; clears
 * the word.  For tests and diagnostics only. */
int wq8_debug_status(void);

#ifdef __cplusplus
}
#endif
#endif /* WQ8_H */
