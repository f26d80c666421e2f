/* C ABI of the Blackwell (sm_100a) build of Flint's GPT-2 training kernels.
 *
 * Every entry point below has the name, argument list, status codes and error
 * behaviour of the function of the same name in the reference's
 * include/flint/flint.h, so a program or ctypes binding written against the
 * reference library loads this one unchanged. Each declaration cites the
 * reference declaration it replaces as "ref: flint.h:<lines>".
 *
 * Conventions shared by all functions:
 *   - pointers are raw device addresses unless stated otherwise, matrices are
 *     row-major and contiguous, sizes are size_t, flags are int (non-zero =
 *     true);
 *   - work is enqueued on the caller's stream and the call returns at once;
 *     a null stream is the legacy default stream;
 *   - a failing call returns a non-zero status and records a message that
 *     flint_last_error() returns on the same thread;
 *   - the library allocates no device memory except inside flint_gpt2_create.
 *
 * Plain C, no CUDA headers needed. */
#ifndef FLINT_FLINT_H
#define FLINT_FLINT_H

#include <stddef.h>

#if defined(_WIN32)
#  if defined(FLINT_BUILD)
#    define FLINT_API __declspec(dllexport)
#  else
#    define FLINT_API __declspec(dllimport)
#  endif
#else
#  define FLINT_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ref: flint.h:26-32 */
typedef int flint_status;
enum {
    FLINT_OK = 0,
    FLINT_ERROR_INVALID_ARGUMENT = 1,
    FLINT_ERROR_CUDA = 2
};

/* "major.minor.patch". ref: flint.h:34-35 */
FLINT_API const char* flint_version(void);

/* "ok", "invalid argument", "CUDA error", or "unknown status".
 * ref: flint.h:37-38 */
FLINT_API const char* flint_status_string(flint_status status);

/* Message of the most recent failed call made by the calling thread ("" before
 * any failure). A successful call does not clear it. ref: flint.h:40-42 */
FLINT_API const char* flint_last_error(void);

/* cudaStream_t without the CUDA headers. ref: flint.h:44-46 */
typedef struct CUstream_st* flint_stream;

/* Device-to-device byte copy; ranges must be disjoint; any size or alignment.
 * bytes == 0 is a no-op. ref: flint.h:48-51 */
FLINT_API flint_status flint_copy(void* dst, const void* src, size_t bytes, flint_stream stream);

/* ---- GEMMs: FP16 operands, FP32 accumulation on the tensor cores ----------
 *
 * Shared limits (ref: flint.h:59-62): all pointers 16-byte aligned, m and n at
 * most 8,388,480, k at most 65,536, outputs disjoint from inputs, and m == 0
 * or n == 0 succeeds without touching anything. Outputs that are FP16 round
 * once, to nearest even, from the FP32 value (overflow gives inf). */

/* y[m,n] = x[m,k] * w[n,k]^T, FP16 out. k a positive multiple of 8.
 * ref: flint.h:53-64 */
FLINT_API flint_status flint_gemm_nt(void* y, const void* x, const void* w, size_t m, size_t n,
                                     size_t k, flint_stream stream);

/* As flint_gemm_nt with bias[n] (FP32) added to the FP32 sums before the one
 * rounding. ref: flint.h:66-72 */
FLINT_API flint_status flint_gemm_nt_bias(void* y, const void* x, const void* w, const void* bias,
                                          size_t m, size_t n, size_t k, flint_stream stream);

/* s = x w^T + bias in FP32; pre = half(s); y = half(gelu_tanh(s)) evaluated
 * on the unrounded s. pre is disjoint from y, x, w and bias.
 * ref: flint.h:74-83 */
FLINT_API flint_status flint_gemm_nt_bias_gelu(void* y, void* pre, const void* x, const void* w,
                                               const void* bias, size_t m, size_t n, size_t k,
                                               flint_stream stream);

/* y32[m,n] = residual32[m,n] + (x w^T + bias): bias added first, then the
 * residual, one FP32 add each; nothing rounds to FP16. n even.
 * ref: flint.h:85-95 */
FLINT_API flint_status flint_gemm_nt_bias_residual(void* y, const void* x, const void* w,
                                                   const void* bias, const void* residual,
                                                   size_t m, size_t n, size_t k,
                                                   flint_stream stream);

/* y[m,n] = x[m,k] * w[k,n], FP16 out. k and n multiples of 8.
 * ref: flint.h:97-102 */
FLINT_API flint_status flint_gemm_nn(void* y, const void* x, const void* w, size_t m, size_t n,
                                     size_t k, flint_stream stream);

/* y = half((x w) * gelu_tanh'(pre)), pre[m,n] FP16 as flint_gemm_nt_bias_gelu
 * stored it. pre = -inf gives derivative 0, +inf gives 1, NaN gives NaN.
 * ref: flint.h:104-114 */
FLINT_API flint_status flint_gemm_nn_dgelu(void* y, const void* x, const void* w,
                                           const void* pre, size_t m, size_t n, size_t k,
                                           flint_stream stream);

/* y32[m,n] = x[k,m]^T * w[k,n], or y32 += with accumulate (old + sum, one FP32
 * add). m and n multiples of 8, k from 1. When flint_gemm_tn_workspace reports
 * a non-zero size the call splits k over several CTAs, stores their FP32
 * partial tiles in the workspace and adds them in split order, so the result
 * is deterministic on a given GPU. ref: flint.h:116-134 */
FLINT_API flint_status flint_gemm_tn(void* y, const void* x, const void* w, size_t m, size_t n,
                                     size_t k, int accumulate, void* workspace,
                                     size_t workspace_bytes, flint_stream stream);

/* Bytes of workspace flint_gemm_tn needs for this shape on the current GPU
 * (depends on its SM count); 0 when k is not split. ref: flint.h:136-138 */
FLINT_API flint_status flint_gemm_tn_workspace(size_t m, size_t n, size_t k, size_t* bytes);

/* dbias32[cols] = column sums of dy16[rows,cols] (or += with accumulate).
 * Compensated (TwoSum) FP32 sums over 256-row chunks in a fixed order that
 * depends only on rows and cols; no atomics. cols a multiple of 8 up to
 * 16,776,960 (0 is a no-op), rows from 1 to 549,755,813,632.
 * ref: flint.h:140-155 */
FLINT_API flint_status flint_bias_gradient(void* dbias, const void* dy, size_t rows, size_t cols,
                                           int accumulate, void* workspace,
                                           size_t workspace_bytes, flint_stream stream);

/* ceil(rows / 256) * cols * 8 bytes. ref: flint.h:157-159 */
FLINT_API flint_status flint_bias_gradient_workspace(size_t rows, size_t cols, size_t* bytes);

/* Batched forms: batch j's matrices follow batch j-1's directly. batches up
 * to 65,535, m up to 1,024; any of batches, m, n zero is a no-op. Per batch
 * the bits equal the unbatched function's (NT at scale 1; TN where k is not
 * split, rounded to FP16). */

/* y[j] = half(scale * x[j] w[j]^T); scale finite, applied in FP32.
 * ref: flint.h:161-175 */
FLINT_API flint_status flint_gemm_nt_batched(void* y, const void* x, const void* w, size_t batches,
                                             size_t m, size_t n, size_t k, float scale,
                                             flint_stream stream);

/* y[j] = x[j] w[j], w[j] is k x n. ref: flint.h:177-182 */
FLINT_API flint_status flint_gemm_nn_batched(void* y, const void* x, const void* w, size_t batches,
                                             size_t m, size_t n, size_t k, flint_stream stream);

/* y[j] = half(x[j]^T w[j]), x[j] is k x m, w[j] is k x n; k is never split.
 * ref: flint.h:184-191 */
FLINT_API flint_status flint_gemm_tn_batched(void* y, const void* x, const void* w, size_t batches,
                                             size_t m, size_t n, size_t k, flint_stream stream);

/* ---- Row-wise kernels ------------------------------------------------------ */

/* Per row of x32[rows,cols]: mean, rstd = 1/sqrt(biased variance + eps), and
 * y16 = (x - mean) * rstd * gamma32 + beta32. mean and rstd (rows FP32 each)
 * are kept for the backward pass. cols 1..2^24, rows up to 17,179,869,176,
 * eps finite and >= 0; rows == 0 is a no-op. ref: flint.h:193-213 */
FLINT_API flint_status flint_layernorm_forward(void* y, void* mean, void* rstd, const void* x,
                                               const void* gamma, const void* beta, size_t rows,
                                               size_t cols, float eps, flint_stream stream);

/* With xhat = (x - mean) * rstd and g = dy * gamma:
 *   dx32 = rstd * ((g - mean(g)) - xhat * mean(g * xhat))   (or += with accumulate_dx)
 *   dgamma32 = column sums of dy * xhat, dbeta32 = column sums of dy
 *                                                 (or += with accumulate_params)
 * All FP32 with individually rounded operations; dgamma/dbeta use the
 * bias-gradient's compensated chunked order, so dbeta equals
 * flint_bias_gradient(dy) bit for bit. cols a multiple of 8 from 8 to
 * 16,776,960; rows from 1. ref: flint.h:215-241 */
FLINT_API flint_status flint_layernorm_backward(void* dx, void* dgamma, void* dbeta,
                                                const void* dy, const void* x, const void* mean,
                                                const void* rstd, const void* gamma, size_t rows,
                                                size_t cols, int accumulate_dx,
                                                int accumulate_params, void* workspace,
                                                size_t workspace_bytes, flint_stream stream);

/* Same size as flint_bias_gradient_workspace(rows, cols). ref: flint.h:243-246 */
FLINT_API flint_status flint_layernorm_backward_workspace(size_t rows, size_t cols,
                                                          size_t* bytes);

/* x32[s*length+t, :] = wte32[tokens[s*length+t], :] + wpe32[t, :]. tokens are
 * uint16 and are not range-checked. width a positive multiple of 8 up to 2^24,
 * vocab 1..65,536. ref: flint.h:248-268 */
FLINT_API flint_status flint_embedding_forward(void* x, const void* tokens, const void* wte,
                                               const void* wpe, size_t sequences, size_t length,
                                               size_t vocab, size_t width, flint_stream stream);

/* dwte32[v,:] = sum of dx32[r,:] over rows r with tokens[r] == v, in ascending
 * r (every row written, +0 for unused v; with accumulate_wte only the used
 * rows get old + sum). dwpe32[t,:] = sum over sequences of dx[s*length+t,:]
 * in the bias-gradient order for dx viewed as sequences x (length*width).
 * Compensated FP32 sums, no atomics; tokens are bucketed by a stable sort in
 * the workspace. Tokens >= vocab reach no dwte row. ref: flint.h:270-303 */
FLINT_API flint_status flint_embedding_backward(void* dwte, void* dwpe, const void* dx,
                                                const void* tokens, size_t sequences,
                                                size_t length, size_t vocab, size_t width,
                                                int accumulate_wte, int accumulate_wpe,
                                                void* workspace, size_t workspace_bytes,
                                                flint_stream stream);

/* ref: flint.h:305-310 */
FLINT_API flint_status flint_embedding_backward_workspace(size_t sequences, size_t length,
                                                          size_t vocab, size_t width,
                                                          size_t* bytes);

/* y16[i] = round-to-nearest-even(x32[i]) for i < count; overflow gives inf.
 * ref: flint.h:312-318 */
FLINT_API flint_status flint_fp32_to_fp16(void* y, const void* x, size_t count,
                                          flint_stream stream);

/* y[b,h,t,c] = x[b*length+t, first + h*head_width + c], moved as bits.
 * x: batches*length rows of row_width FP16; y: batches x heads x length x
 * head_width. head_width, row_width, first multiples of 8.
 * ref: flint.h:320-338 */
FLINT_API flint_status flint_heads_split(void* y, const void* x, size_t batches, size_t length,
                                         size_t heads, size_t head_width, size_t row_width,
                                         size_t first, flint_stream stream);

/* Inverse of flint_heads_split; only columns [first, first + heads*head_width)
 * of each row of y are written. ref: flint.h:340-348 */
FLINT_API flint_status flint_heads_merge(void* y, const void* x, size_t batches, size_t length,
                                         size_t heads, size_t head_width, size_t row_width,
                                         size_t first, flint_stream stream);

/* p16[b,t,c] = softmax over c <= t of s16[b,t,:], +0 for c > t (masked inputs
 * ignored even if NaN). length a multiple of 8 up to 1,024, batches up to
 * 65,535. ref: flint.h:350-369 */
FLINT_API flint_status flint_causal_softmax_forward(void* p, const void* s, size_t batches,
                                                    size_t length, flint_stream stream);

/* ds16[b,t,c] = scale * p * (dp - D) for c <= t, +0 above the diagonal, with
 * D the compensated FP32 sum of p*dp over the visible columns. ds may alias
 * dp. ref: flint.h:371-392 */
FLINT_API flint_status flint_causal_softmax_backward(void* ds, const void* p, const void* dp,
                                                     size_t batches, size_t length, float scale,
                                                     flint_stream stream);

/* Over the first vocab columns of each row of logits16[rows,cols]:
 *   row_loss32[r] = log(sum exp(l - max)) - (l[target] - max)
 *   dlogits16[r,c] = scale * (softmax[c] - [c == target]); +0 for c >= vocab.
 * targets are uint16. cols a multiple of 8 from 8 to 65,536.
 * ref: flint.h:394-433 */
FLINT_API flint_status flint_softmax_cross_entropy(void* dlogits, void* row_loss,
                                                   const void* logits, const void* targets,
                                                   float scale, size_t rows, size_t vocab,
                                                   size_t cols, flint_stream stream);

/* ---- GPT-2 model object ------------------------------------------------------ */

/* ref: flint.h:435-438 */
typedef struct flint_gpt2 flint_gpt2;

/* Model shape; limits as in the reference. ref: flint.h:440-466 */
typedef struct {
    size_t layers;
    size_t heads;
    size_t width;
    size_t block_size;
    size_t vocab;
    size_t padded_vocab;
    size_t sequences;
    size_t length;
    int separate_buffers;
    int backward;
} flint_gpt2_config;

/* One FP32 master weight (or its gradient). ref: flint.h:468-475 */
typedef struct {
    const char* name;
    void* data;
    size_t rows;
    size_t cols;
} flint_gpt2_parameter_info;

/* Device bytes flint_gpt2_create would allocate. ref: flint.h:477-482 */
FLINT_API flint_status flint_gpt2_bytes(const flint_gpt2_config* config, size_t* bytes);

/* ref: flint.h:484-491 */
FLINT_API flint_status flint_gpt2_create(const flint_gpt2_config* config, flint_gpt2** model);

/* ref: flint.h:493-495 */
FLINT_API void flint_gpt2_destroy(flint_gpt2* model);

/* ref: flint.h:497-498 */
FLINT_API size_t flint_gpt2_parameter_count(const flint_gpt2* model);

/* Parameters in PyTorch named_parameters order. ref: flint.h:500-504 */
FLINT_API flint_status flint_gpt2_parameter(const flint_gpt2* model, size_t index,
                                            flint_gpt2_parameter_info* info);

/* FP32 masters -> FP16 compute copies. ref: flint.h:506-509 */
FLINT_API flint_status flint_gpt2_sync_weights(flint_gpt2* model, flint_stream stream);

/* tokens -> logits, row_loss, dlogits. ref: flint.h:511-523 */
FLINT_API flint_status flint_gpt2_forward(flint_gpt2* model, const void* tokens,
                                          const void* targets, float scale, flint_stream stream);

/* dlogits -> every parameter gradient. ref: flint.h:525-553 */
FLINT_API flint_status flint_gpt2_backward(flint_gpt2* model, const void* tokens, int accumulate,
                                           flint_stream stream);

/* ref: flint.h:555-560 */
FLINT_API flint_status flint_gpt2_gradient(const flint_gpt2* model, size_t index,
                                           flint_gpt2_parameter_info* info);

/* ref: flint.h:562-567 */
FLINT_API flint_status flint_gpt2_outputs(const flint_gpt2* model, const void** logits,
                                          const void** dlogits, const void** row_loss);

/* Synchronises stream, reads row_loss and returns its FP64 mean in *loss (a
 * host pointer). ref: flint.h:569-573 */
FLINT_API flint_status flint_gpt2_mean_loss(flint_gpt2* model, flint_stream stream, double* loss);

#ifdef __cplusplus
}
#endif

#endif /* FLINT_FLINT_H */
