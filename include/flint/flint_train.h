/* libflint_train.so: the data-parallel GPT-2 training step behind a C ABI.
 *
 * The reference has no trainer in C++ (its README lists the optimizer, loss
 * scaling and multi-GPU as planned); what a step must do is fixed by its PyTorch
 * oracle, scripts/gpt2_torch.py:161-192: forward and backward in FP16 with FP32
 * accumulation under a dynamic loss scale (GradScaler's policy: start at 2^16,
 * halve on a non-finite gradient and skip that step, double after
 * growth_interval good steps), optional clipping of the global gradient norm
 * (:187-188) and AdamW with two parameter groups (:150-175). None of the
 * functions below has a counterpart in the reference's include/flint/flint.h.
 *
 * This library is a client of libflint.so's C ABI (flint.h, flint_b200.h) and
 * adds the host-side step around it: one process per GPU, a second stream for
 * collectives, NCCL loaded at run time with dlopen (so neither library links
 * it; FLINT_NCCL_LIBRARY names the file, default libnccl.so.2) and used only
 * when world > 1; NCCL_NVLS_ENABLE is set to 0 unless the environment already
 * sets it (the configuration every multi-rank figure was measured in). Two ways
 * to share the work across ranks:
 *   replicated  every gradient bucket is summed with ncclAllReduce while the
 *               backward pass continues; every rank runs the whole AdamW
 *   sharded     (shard_optimizer) every bucket is summed with ncclReduceScatter,
 *               each rank keeps AdamW moments for, and updates, only its 1/world
 *               slice of each bucket, and the updated FP32 weights are gathered
 *               with ncclAllGather bucket by bucket in forward order while the
 *               next step's forward pass starts (each layer waits only for its
 *               own bucket)
 * Each rank scales its loss by loss_scale / (rows_per_rank * world *
 * micro_batches), so the plain sum over ranks is loss_scale times the gradient
 * of the global mean loss and every rank takes the same skip decision.
 *
 * Conventions are libflint's: device pointers, the caller's stream, flint_status
 * return codes; flint_train_last_error() is this library's per-thread message. */
#ifndef FLINT_FLINT_TRAIN_H
#define FLINT_FLINT_TRAIN_H

#include "flint/flint_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct flint_trainer flint_trainer;

typedef struct {
    flint_gpt2_config model;  /* sequences and length are per rank and micro-batch;
                                 backward and separate_buffers are set by the trainer */
    int flash_attention;      /* build the model on the fused attention kernels */
    float lr, beta1, beta2, eps;
    float weight_decay;       /* on parameters with two or more dimensions */
    float loss_scale;         /* initial dynamic loss scale */
    int growth_interval;
    float max_grad_norm;      /* 0 disables clipping */
    int world, rank;          /* data-parallel job; world 1 needs no NCCL */
    int shard_optimizer;      /* world > 1: reduce-scatter + per-rank AdamW + all-gather */
    int overlap_update;       /* replicated, world > 1, no clipping: update most of the model
                                 while the last bucket's all-reduce is in flight */
} flint_trainer_config;

typedef struct {
    float loss_scale;
    int good_steps;           /* consecutive finite steps since the scale last changed */
    long long step_count;     /* optimizer steps attempted */
    long long skipped;        /* of which skipped for a non-finite gradient */
    double grad_norm;         /* global norm of the unscaled gradient, last clipped step */
} flint_trainer_status;

/* One contiguous FP32 range of the gradient arena that this rank's optimizer
 * owns: `first` floats from the arena's start, `count` floats, stored from
 * `storage` floats into the moment arrays. `shared` is 1 when every rank owns
 * this same range (a replicated trainer's one range, the whole arena; or a
 * bucket too ragged to split), 0 when the other ranks own the rest of it. */
typedef struct {
    size_t first, count, storage;
    int shared;
} flint_trainer_range;

#define FLINT_TRAIN_NCCL_ID_BYTES 128

FLINT_API const char* flint_train_last_error(void);

/* GradScaler's update as a pure function (no GPU): the next scale and good-step count. */
FLINT_API flint_status flint_train_scale_policy(float scale, int good_steps, int growth_interval,
                                                int found_nonfinite, float* next_scale,
                                                int* next_good_steps);

/* ncclGetUniqueId into id[128]: call on one rank and hand the bytes to the
 * others by any host channel before flint_trainer_create. */
FLINT_API flint_status flint_train_nccl_id(void* id);

/* Builds the model, the optimizer state and, for world > 1, the NCCL
 * communicator (collective: every rank must call it, nccl_id identical). The
 * current device is the trainer's. On failure *trainer is NULL. */
FLINT_API flint_status flint_trainer_create(const flint_trainer_config* config, const void* nccl_id,
                                            flint_trainer** trainer);
FLINT_API void flint_trainer_destroy(flint_trainer* trainer);

/* The model inside (owned by the trainer): load FP32 weights through
 * flint_gpt2_parameter, then call flint_trainer_weights_changed. */
FLINT_API flint_status flint_trainer_model(flint_trainer* trainer, flint_gpt2** model);
FLINT_API flint_status flint_trainer_weights_changed(flint_trainer* trainer, flint_stream stream);

/* One optimizer step over `micro_batches` (tokens[i], targets[i]) pairs of
 * uint16 device arrays, accumulated into one gradient as the reference's
 * train_step does: enqueues forward, backward with overlapped collectives, the
 * non-finite check, the optional clip and AdamW. Returns without waiting. */
FLINT_API flint_status flint_trainer_step(flint_trainer* trainer, const void* const* tokens,
                                          const void* const* targets, size_t micro_batches,
                                          flint_stream stream);

/* The optimizer's half of a step on whatever the gradient arena holds (world 1):
 * check, optional clip, AdamW. */
FLINT_API flint_status flint_trainer_update(flint_trainer* trainer, flint_stream stream);

/* Waits for the step, applies the loss-scale policy and returns this rank's mean
 * loss over the step's micro-batches and whether the step was skipped. */
FLINT_API flint_status flint_trainer_finish(flint_trainer* trainer, flint_stream stream,
                                            double* mean_loss, int* skipped);

/* Waits for `stream` and for the trainer's collective stream: after a sharded
 * step the updated weights of other ranks' slices may still be arriving when
 * flint_trainer_finish returns (the next step waits for them layer by layer);
 * call this before reading weights from the host. */
FLINT_API flint_status flint_trainer_synchronize(flint_trainer* trainer, flint_stream stream);

FLINT_API flint_status flint_trainer_get_status(const flint_trainer* trainer,
                                                flint_trainer_status* status);
/* For resuming from a checkpoint: scale, good_steps, step_count and skipped are taken. */
FLINT_API flint_status flint_trainer_set_status(flint_trainer* trainer,
                                                const flint_trainer_status* status);

/* AdamW's moments (device FP32 arrays of `count` floats each) and the ranges of
 * the gradient arena they belong to. */
FLINT_API flint_status flint_trainer_moments(flint_trainer* trainer, void** m, void** v,
                                             size_t* count);
FLINT_API size_t flint_trainer_shard_count(const flint_trainer* trainer);
FLINT_API flint_status flint_trainer_shard(const flint_trainer* trainer, size_t index,
                                           flint_trainer_range* shard);

/* The device int that is 1 when the last step's gradients were not finite and
 * the device double holding the squared norm of the last clipped step. */
FLINT_API flint_status flint_trainer_flags(flint_trainer* trainer, int** found_nonfinite,
                                           double** norm_squared);

/* Called on the launching thread for each gradient bucket of the last
 * micro-batch, after its producers are enqueued and before its collective is:
 * a test can enqueue work on `stream` there (for instance write a non-finite
 * value into one rank's gradient). Null removes the hook. */
typedef void (*flint_trainer_bucket_hook)(void* user, int bucket, void* gradients, size_t bytes,
                                          flint_stream stream);
FLINT_API flint_status flint_trainer_set_bucket_hook(flint_trainer* trainer,
                                                     flint_trainer_bucket_hook hook, void* user);

#ifdef __cplusplus
}
#endif

#endif /* FLINT_FLINT_TRAIN_H */
