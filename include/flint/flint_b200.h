/* Extensions of the Blackwell build that the reference library does not have:
 * fused (flash) causal attention, the optimizer and loss-scaling kernels, a
 * model variant that uses them, and hooks for data-parallel training. None of
 * these has a counterpart in the reference's include/flint/flint.h; they follow
 * the same conventions (device pointers, caller's stream, flint_status,
 * flint_last_error). The PyTorch oracle they are checked against is the
 * reference's scripts/gpt2_torch.py (attention: :52-60, AdamW groups: :161-175,
 * train_step: :178-192). */
#ifndef FLINT_FLINT_B200_H
#define FLINT_FLINT_B200_H

#include "flint/flint.h"

#ifdef __cplusplus
extern "C" {
#endif

/* 1 if a kernel (GEMM, attention, column sums, cross-entropy) gave up on a
 * bounded barrier wait since the last call (the flag is cleared), 0 otherwise.
 * Synchronises the device; meant for tests. */
FLINT_API flint_status flint_b200_kernel_fault(int* raised);

/* Kernels this library has launched in this process so far (host counter). */
FLINT_API flint_status flint_b200_launch_count(unsigned long long* launches);

/* Diagnostic (no counterpart in the reference): the rate of the tensor pipe for
 * the small MMAs that attention with head width 64 is made of. One CTA on an
 * otherwise idle GPU issues `count` (1 to 4,096) tcgen05.mma of kind::f16 with
 * M = 128, K = 16 and N = `n` (64 or 128) back to back from one elected thread,
 * the A operand read from shared memory or, when a_in_tmem is not 0, from tensor
 * memory; operands are zeros. *issue_clocks receives the SM clocks until the last
 * one was accepted, *complete_clocks until all had completed. Waits for the
 * stream; meant for `python -m flint_b200.kernel_bench --group mma`. */
FLINT_API flint_status flint_b200_mma_clocks(int n, int a_in_tmem, int count,
                                             long long* issue_clocks, long long* complete_clocks,
                                             flint_stream stream);

/* Causal attention without materialising scores or probabilities:
 * o[b] = softmax(scale * q[b] k[b]^T + causal mask) v[b] for `batches`
 * (sequence, head) pairs, all FP16 [batches, length, head_width] contiguous;
 * lse[batches, length] FP32 receives log-sum-exp of the scaled scores (natural
 * log), which the backward pass needs. head_width must be 64, length a
 * multiple of 8 up to 1,024, scale finite and positive. */
FLINT_API flint_status flint_b200_attention_forward(void* o, void* lse, const void* q,
                                                    const void* k, const void* v, size_t batches,
                                                    size_t length, size_t head_width, float scale,
                                                    flint_stream stream);

/* Gradients of the above: dq, dk, dv from d_o, o, lse and q, k, v (layouts as
 * above). delta is an FP32 scratch [batches, length] the call overwrites. */
FLINT_API flint_status flint_b200_attention_backward(void* dq, void* dk, void* dv, const void* d_o,
                                                     const void* o, const void* lse, void* delta,
                                                     const void* q, const void* k, const void* v,
                                                     size_t batches, size_t length,
                                                     size_t head_width, float scale,
                                                     flint_stream stream);

/* flint_gpt2_create with a choice of attention: flash_attention non-zero builds
 * the model on the fused kernels above (no T x T buffers, so far less memory);
 * zero is flint_gpt2_create. */
FLINT_API flint_status flint_b200_gpt2_create(const flint_gpt2_config* config, int flash_attention,
                                              flint_gpt2** model);

/* Called on the launching host thread from inside
 * flint_b200_gpt2_backward_buckets each time every kernel that writes one
 * contiguous range of the gradient arena has been enqueued: bucket 0 is ln_f,
 * buckets 1..layers are the blocks from last to first, and the final bucket is
 * wte + wpe. A data-parallel trainer records an event there and starts that
 * range's all-reduce on another stream. */
typedef void (*flint_b200_bucket_callback)(void* user, int bucket, void* gradients, size_t bytes);

/* flint_gpt2_backward plus the callback above (which may be null). */
FLINT_API flint_status flint_b200_gpt2_backward_buckets(flint_gpt2* model, const void* tokens,
                                                        int accumulate, flint_stream stream,
                                                        flint_b200_bucket_callback callback,
                                                        void* user);

/* Called on the launching host thread from inside flint_b200_gpt2_forward_stages
 * before the kernels of each stage are enqueued: stage 0 is the embedding,
 * stages 1..layers the transformer blocks in order, stage layers + 1 the final
 * LayerNorm with the output layer and the loss. A trainer whose weights arrive
 * bucket by bucket (a sharded optimizer's all-gather) makes the stream wait
 * there for that stage's weights only. */
typedef void (*flint_b200_stage_callback)(void* user, int stage);

/* flint_gpt2_forward plus the callback above (which may be null). */
FLINT_API flint_status flint_b200_gpt2_forward_stages(flint_gpt2* model, const void* tokens,
                                                      const void* targets, float scale,
                                                      flint_stream stream,
                                                      flint_b200_stage_callback callback,
                                                      void* user);

/* The contiguous FP32 range that holds every gradient, in parameter order. */
FLINT_API flint_status flint_b200_gpt2_gradient_arena(const flint_gpt2* model, void** base,
                                                      size_t* bytes);

/* The FP16 compute copy of the index-th master weight (what the GEMMs read), or
 * null for biases and LayerNorm parameters, which have none. An optimizer that
 * writes it together with the master weight saves flint_gpt2_sync_weights. */
FLINT_API flint_status flint_b200_gpt2_compute_copy(const flint_gpt2* model, size_t index,
                                                    void** address);

/* Fused AdamW over `count` FP32 values (PyTorch semantics, decoupled decay):
 *   g = grad * grad_scale;  m = b1 m + (1 - b1) g;  v = b2 v + (1 - b2) g^2
 *   p = p - lr * (weight_decay * p + (m / (1 - b1^step)) / (sqrt(v / (1 - b2^step)) + eps))
 * and, when half_copy is not null, half_copy = half(p). When *skip (a device
 * int, may be null) is non-zero the call changes nothing: a step whose
 * gradients overflowed is dropped. */
FLINT_API flint_status flint_b200_adamw(void* param, void* m, void* v, const void* grad,
                                        void* half_copy, size_t count, float lr, float beta1,
                                        float beta2, float eps, float weight_decay,
                                        float grad_scale, int step, const int* skip,
                                        flint_stream stream);

/* One tensor of a multi-tensor AdamW plan; half_copy may be null. */
typedef struct {
    void* param;
    void* m;
    void* v;
    const void* grad;
    void* half_copy;
    size_t count;
    float weight_decay;
} flint_b200_adamw_tensor;

/* A plan lets one launch update every tensor of a model. tensors is a host
 * array; *bytes is the device memory the plan needs; *items is what
 * flint_b200_adamw_run takes. */
FLINT_API flint_status flint_b200_adamw_plan_bytes(const flint_b200_adamw_tensor* tensors,
                                                   size_t count, size_t* bytes);
FLINT_API flint_status flint_b200_adamw_plan_items(const flint_b200_adamw_tensor* tensors,
                                                   size_t count, size_t* items);

/* Writes the plan into device memory `plan` (16-byte aligned, plan_bytes long)
 * and waits for the copy, so tensors may be freed on return. */
FLINT_API flint_status flint_b200_adamw_plan(void* plan, size_t plan_bytes,
                                             const flint_b200_adamw_tensor* tensors, size_t count,
                                             flint_stream stream);

/* flint_b200_adamw over every tensor of the plan, each with its own weight
 * decay, in one launch. */
FLINT_API flint_status flint_b200_adamw_run(const void* plan, size_t items, float lr, float beta1,
                                            float beta2, float eps, float grad_scale, int step,
                                            const int* skip, flint_stream stream);

/* flint_bias_gradient for callers that cannot supply a workspace. It has no
 * counterpart in the reference. The result is flint_bias_gradient's bit for bit;
 * the partial sums live in a 4 MiB array built into the library instead of a
 * caller buffer, and the call allocates nothing (no cudaMalloc, no cudaFree).
 * It exists for hosts that may not allocate device memory once they are running:
 * a plug-in inside an application that owns the whole memory budget, or a loop
 * that cannot afford the device-wide synchronisation cudaMalloc implies.
 *
 * Limit: ceil(rows / 256) * cols * 8 bytes must fit in 4 MiB (for example 16,384
 * rows x 3,072 cols needs 1.5 MiB); larger shapes fail with
 * FLINT_ERROR_INVALID_ARGUMENT and should use flint_bias_gradient. Every GPU
 * that loads the library holds the 4 MiB until the process exits.
 *
 * The first call on each device looks up the array's device address; make that
 * call before starting any stream capture. All calls share the one array, so two
 * calls that can overlap on the GPU (different streams, no ordering between
 * them) race on it; calls ordered on one stream are fine, and nothing has to be
 * cleared between them. */
FLINT_API flint_status flint_b200_bias_gradient_static(void* dbias, const void* dy, size_t rows,
                                                       size_t cols, int accumulate,
                                                       flint_stream stream);

/* ---- decoding with a KV cache (the reference's inference milestone, README.md:148; it has
 * no code for it, so nothing here has a counterpart in its header) ----
 *
 * A generator decodes with the weights of `model` (whose FP16 copies must be in
 * sync): `sequences` sequences (1..64) side by side, each up to `max_length`
 * positions (a multiple of 8, at most min(block_size, 1024)). It owns the cache
 * [layer][K|V][sequence][head][position][64] in FP16 and its scratch; with
 * int8_weights it also owns an int8 copy of every matrix with one FP32 scale per
 * output row (w[n, :] ~ q[n, :] * scale[n], q = round(w / scale), scale = max|w| / 127),
 * halving the bytes a decode step reads. Heads must be 64 wide. */
typedef struct flint_b200_generator flint_b200_generator;

FLINT_API flint_status flint_b200_generator_create(const flint_gpt2* model, size_t sequences,
                                                   size_t max_length, int int8_weights,
                                                   flint_b200_generator** generator);
FLINT_API void flint_b200_generator_destroy(flint_b200_generator* generator);

/* Re-derives the int8 copies after the model's weights changed. */
FLINT_API flint_status flint_b200_generator_refresh(flint_b200_generator* generator,
                                                    flint_stream stream);

/* Starts over: tokens is uint16 [sequences, length], length a multiple of 8 up
 * to max_length. Runs the prompt through the tensor-core GEMMs and the fused
 * causal attention kernel, stores every position's keys and values in the
 * cache and leaves the logits of each sequence's last position. */
FLINT_API flint_status flint_b200_generator_prefill(flint_b200_generator* generator,
                                                    const void* tokens, size_t length,
                                                    flint_stream stream);

/* Appends one token per sequence (uint16 [sequences]) at the next position:
 * leaves its logits and writes each sequence's most likely next token (lowest
 * index among equals, padded columns excluded) to next_tokens (uint16
 * [sequences] on the device; null keeps it internal). With use_graph non-zero
 * the step's launches are captured into a CUDA graph on the first call and
 * replayed afterwards (the position lives in device memory); tokens and
 * next_tokens must then be the same buffers on every call. */
FLINT_API flint_status flint_b200_generator_step(flint_b200_generator* generator,
                                                 const void* tokens, void* next_tokens,
                                                 int use_graph, flint_stream stream);

/* FP32 logits [sequences, padded_vocab] of the last position processed, and how
 * many positions each sequence holds. */
FLINT_API flint_status flint_b200_generator_logits(const flint_b200_generator* generator,
                                                   const void** logits, size_t* position);

/* Bytes the next decode step must read from HBM: the weights (each matrix once;
 * the output layer once per group of eight sequences) and the cache. */
FLINT_API flint_status flint_b200_generator_bytes_per_step(const flint_b200_generator* generator,
                                                           size_t* weight_bytes,
                                                           size_t* cache_bytes);

/* Sets *found_nonfinite (device int) to 1 if any of the count FP32 values is
 * inf or NaN; leaves it unchanged otherwise, so several calls can share it.
 * When sum_squares (device double, may be null) is given, adds the sum of
 * squares of the values times scale^2 to it (for gradient-norm clipping). */
FLINT_API flint_status flint_b200_check_gradients(const void* grad, size_t count, float scale,
                                                  int* found_nonfinite, double* sum_squares,
                                                  flint_stream stream);

#ifdef __cplusplus
}
#endif

#endif /* FLINT_FLINT_B200_H */
