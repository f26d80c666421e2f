// libflint_train.so: the data-parallel GPT-2 training step (see include/flint/flint_train.h).
//
// Host code only: every kernel is libflint.so's, reached through its C ABI. What this
// file adds is the step's choreography: two streams, events at the gradient buckets the
// backward pass reports, NCCL collectives on the second stream (the library is opened at
// run time, nothing links it), GradScaler's loss-scale policy, gradient clipping and the
// AdamW launches. What a step must compute follows the reference's PyTorch oracle,
// scripts/gpt2_torch.py:161-192.
//
// Gradient buckets, in the order the backward pass completes them: ln_f, the transformer
// blocks from last to first, then wte + wpe. The FP32 masters and the FP32 gradients lie
// in two arenas with identical offsets, so a float range of the gradient arena names the
// same parameters in the master arena.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nccl.h>  // types and enumerators only; the functions come from dlopen

#include "flint/flint_train.h"

namespace {

constexpr flint_status kInvalid = FLINT_ERROR_INVALID_ARGUMENT;
thread_local std::string g_error;

flint_status fail(flint_status status, const char* format, ...) {
    char buffer[512];
    va_list args;
    va_start(args, format);
    std::vsnprintf(buffer, sizeof buffer, format, args);
    va_end(args);
    g_error = buffer;
    return status;
}

// A failed libflint call: its message becomes ours.
flint_status forward_error(flint_status status) {
    g_error = flint_last_error();
    return status;
}

flint_status cuda_error(cudaError_t e, const char* what) {
    cudaGetLastError();
    return fail(FLINT_ERROR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TRY(call)                            \
    do {                                     \
        const flint_status try_status = (call); \
        if (try_status != FLINT_OK) {        \
            return try_status;               \
        }                                    \
    } while (0)
#define FLINT(call)                              \
    do {                                         \
        const flint_status lib_status = (call);  \
        if (lib_status != FLINT_OK) {            \
            return forward_error(lib_status);    \
        }                                        \
    } while (0)
#define CUDA(call)                               \
    do {                                         \
        const cudaError_t cuda_status = (call);  \
        if (cuda_status != cudaSuccess) {        \
            return cuda_error(cuda_status, #call); \
        }                                        \
    } while (0)

// ---- NCCL through dlopen ------------------------------------------------------------------

struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t,
                                  ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

flint_status load_nccl(Nccl** out) {
    static Nccl nccl;
    static bool loaded = false;
    if (loaded) {
        *out = &nccl;
        return FLINT_OK;
    }
    const char* name = std::getenv("FLINT_NCCL_LIBRARY");
    if (name == nullptr || name[0] == '\0') {
        name = "libnccl.so.2";
    }
    // In-switch reductions (NVLS) stay off unless the caller's environment asks for them: every
    // multi-rank number of this library was measured that way (two, four and eight ranks), and
    // the one eight-rank run with NVLS on did not get through communicator set-up in ten
    // minutes. NCCL reads the variable when the first communicator is created.
    setenv("NCCL_NVLS_ENABLE", "0", 0);
    void* handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) {
        return fail(FLINT_ERROR_CUDA, "flint_train: cannot open %s (%s); set FLINT_NCCL_LIBRARY",
                    name, dlerror());
    }
    struct {
        const char* symbol;
        void** slot;
    } const wanted[] = {
        {"ncclGetUniqueId", reinterpret_cast<void**>(&nccl.GetUniqueId)},
        {"ncclCommInitRank", reinterpret_cast<void**>(&nccl.CommInitRank)},
        {"ncclCommDestroy", reinterpret_cast<void**>(&nccl.CommDestroy)},
        {"ncclAllReduce", reinterpret_cast<void**>(&nccl.AllReduce)},
        {"ncclReduceScatter", reinterpret_cast<void**>(&nccl.ReduceScatter)},
        {"ncclAllGather", reinterpret_cast<void**>(&nccl.AllGather)},
        {"ncclGetErrorString", reinterpret_cast<void**>(&nccl.GetErrorString)},
    };
    for (const auto& w : wanted) {
        *w.slot = dlsym(handle, w.symbol);
        if (*w.slot == nullptr) {
            return fail(FLINT_ERROR_CUDA, "flint_train: %s lacks %s", name, w.symbol);
        }
    }
    nccl.handle = handle;
    loaded = true;
    *out = &nccl;
    return FLINT_OK;
}

// ---- the trainer ----------------------------------------------------------------------------

struct Tensor {
    std::string name;
    float* master;
    float* gradient;
    void* half;     // FP16 compute copy or null
    size_t first;   // floats from the arenas' start
    size_t count;
    float decay;
};

struct Bucket {
    size_t first, count;     // float range of the arenas (whole tensors)
    size_t tensor_lo, tensor_hi;  // tensors [lo, hi) in parameter order
    bool sharded;            // sharded mode and count divisible by world
    cudaEvent_t ready = nullptr;     // producers enqueued (main stream)
    cudaEvent_t gathered = nullptr;  // sharded: updated weights have arrived (comm stream)
};

struct Plan {
    void* device = nullptr;
    size_t items = 0;
};

}  // namespace

struct flint_trainer {
    flint_trainer_config config{};
    flint_gpt2* model = nullptr;
    size_t rows = 0;
    size_t layers = 0;
    std::vector<Tensor> tensors;
    std::vector<Bucket> buckets;        // completion order: ln_f, blocks last..first, embeddings
    float* gradient_arena = nullptr;
    float* master_arena = nullptr;
    size_t arena_count = 0;             // floats
    std::vector<flint_trainer_range> shards;  // what this rank's optimizer owns
    float* m = nullptr;
    float* v = nullptr;
    size_t moment_count = 0;
    Plan whole, body, embeddings;       // AdamW plans: all owned ranges; replicated split
    int* found = nullptr;               // device
    double* norm_squared = nullptr;     // device
    float* losses = nullptr;            // device [capacity][rows]
    size_t loss_capacity = 0;
    std::vector<float> host_losses;
    size_t micro_batches = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t comm_done = nullptr, flag_ready = nullptr, updated = nullptr, checked = nullptr;
    bool gather_pending = false;        // sharded: the next forward waits for the all-gathers
    Nccl* nccl = nullptr;
    ncclComm_t comm = nullptr;
    flint_trainer_status status{};
    flint_trainer_bucket_hook hook = nullptr;
    void* hook_user = nullptr;
    // Per-step context for the callbacks.
    cudaStream_t stream = nullptr;
    flint_status callback_status = FLINT_OK;
    bool reduce_now = false;

    ~flint_trainer();
};

flint_trainer::~flint_trainer() {
    if (comm_stream != nullptr) {
        cudaStreamSynchronize(comm_stream);
    }
    if (comm != nullptr && nccl != nullptr) {
        nccl->CommDestroy(comm);
    }
    for (Bucket& b : buckets) {
        if (b.ready != nullptr) cudaEventDestroy(b.ready);
        if (b.gathered != nullptr) cudaEventDestroy(b.gathered);
    }
    for (cudaEvent_t e : {comm_done, flag_ready, updated, checked}) {
        if (e != nullptr) cudaEventDestroy(e);
    }
    if (comm_stream != nullptr) cudaStreamDestroy(comm_stream);
    for (void* p : {static_cast<void*>(m), static_cast<void*>(v), static_cast<void*>(found),
                    static_cast<void*>(norm_squared), static_cast<void*>(losses), whole.device,
                    body.device, embeddings.device}) {
        if (p != nullptr) cudaFree(p);
    }
    if (model != nullptr) {
        flint_gpt2_destroy(model);
    }
    cudaGetLastError();
}

namespace {

flint_status nccl_check(flint_trainer& t, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) {
        return FLINT_OK;
    }
    return fail(FLINT_ERROR_CUDA, "%s: NCCL error: %s", what, t.nccl->GetErrorString(r));
}

flint_status check_config(const flint_trainer_config* c) {
    constexpr const char* name = "flint_trainer_create";
    if (c == nullptr) {
        return fail(kInvalid, "%s: config is null", name);
    }
    if (c->world < 1 || c->rank < 0 || c->rank >= c->world) {
        return fail(kInvalid, "%s: rank (%d) must be from 0 to world (%d) - 1", name, c->rank,
                    c->world);
    }
    if (!(c->lr >= 0.0f) || !std::isfinite(c->lr) || !(c->beta1 >= 0.0f && c->beta1 < 1.0f) ||
        !(c->beta2 >= 0.0f && c->beta2 < 1.0f) || !(c->eps >= 0.0f) ||
        !std::isfinite(c->weight_decay)) {
        return fail(kInvalid, "%s: hyper-parameters must be finite, with betas in [0, 1)", name);
    }
    if (!(c->loss_scale > 0.0f) || !std::isfinite(c->loss_scale)) {
        return fail(kInvalid, "%s: loss_scale (%g) must be positive and finite", name,
                    static_cast<double>(c->loss_scale));
    }
    if (c->growth_interval < 1) {
        return fail(kInvalid, "%s: growth_interval (%d) must be at least 1", name,
                    c->growth_interval);
    }
    if (!(c->max_grad_norm >= 0.0f) || !std::isfinite(c->max_grad_norm)) {
        return fail(kInvalid, "%s: max_grad_norm (%g) must be finite and non-negative", name,
                    static_cast<double>(c->max_grad_norm));
    }
    return FLINT_OK;
}

// A device-resident AdamW plan over the pieces of `tensors` inside the owned ranges
// [lo, hi) of `shards` (all of them, or those with first inside [from, to)).
flint_status build_plan(flint_trainer& t, size_t from, size_t to, Plan* plan) {
    std::vector<flint_b200_adamw_tensor> pieces;
    for (const flint_trainer_range& s : t.shards) {
        for (const Tensor& x : t.tensors) {
            const size_t lo = std::max({s.first, x.first, from});
            const size_t hi = std::min({s.first + s.count, x.first + x.count, to});
            if (lo >= hi) {
                continue;
            }
            flint_b200_adamw_tensor piece;
            piece.param = t.master_arena + lo;
            piece.grad = t.gradient_arena + lo;
            piece.m = t.m + s.storage + (lo - s.first);
            piece.v = t.v + s.storage + (lo - s.first);
            piece.half_copy =
                x.half == nullptr ? nullptr : static_cast<char*>(x.half) + (lo - x.first) * 2;
            piece.count = hi - lo;
            piece.weight_decay = x.decay;
            pieces.push_back(piece);
        }
    }
    plan->items = 0;
    if (pieces.empty()) {
        return FLINT_OK;
    }
    size_t bytes = 0;
    FLINT(flint_b200_adamw_plan_bytes(pieces.data(), pieces.size(), &bytes));
    FLINT(flint_b200_adamw_plan_items(pieces.data(), pieces.size(), &plan->items));
    CUDA(cudaMalloc(&plan->device, bytes + 16));
    FLINT(flint_b200_adamw_plan(plan->device, bytes, pieces.data(), pieces.size(), nullptr));
    return FLINT_OK;
}

flint_status build(flint_trainer& t, const void* nccl_id) {
    const flint_trainer_config& c = t.config;
    flint_gpt2_config mc = c.model;
    mc.backward = 1;
    mc.separate_buffers = 0;
    FLINT(flint_b200_gpt2_create(&mc, c.flash_attention, &t.model));
    t.rows = mc.sequences * mc.length;
    t.layers = mc.layers;

    void* arena = nullptr;
    size_t arena_bytes = 0;
    FLINT(flint_b200_gpt2_gradient_arena(t.model, &arena, &arena_bytes));
    t.gradient_arena = static_cast<float*>(arena);
    t.arena_count = arena_bytes / 4;
    const size_t count = flint_gpt2_parameter_count(t.model);
    for (size_t i = 0; i < count; ++i) {
        flint_gpt2_parameter_info p{}, g{};
        FLINT(flint_gpt2_parameter(t.model, i, &p));
        FLINT(flint_gpt2_gradient(t.model, i, &g));
        void* half = nullptr;
        FLINT(flint_b200_gpt2_compute_copy(t.model, i, &half));
        if (i == 0) {
            t.master_arena = static_cast<float*>(p.data);
        }
        Tensor x;
        x.name = p.name;
        x.master = static_cast<float*>(p.data);
        x.gradient = static_cast<float*>(g.data);
        x.half = half;
        x.first = static_cast<size_t>(x.gradient - t.gradient_arena);
        x.count = p.rows * p.cols;
        x.decay = p.rows > 1 ? c.weight_decay : 0.0f;
        if (static_cast<size_t>(x.master - t.master_arena) != x.first) {
            return fail(FLINT_ERROR_CUDA,
                        "flint_trainer_create: the master and gradient arenas differ in layout at %s",
                        p.name);
        }
        t.tensors.push_back(x);
    }
    if (count != 4 + 12 * t.layers) {
        return fail(FLINT_ERROR_CUDA, "flint_trainer_create: unexpected parameter count %zu", count);
    }

    const bool many = c.world > 1;
    const bool sharded = many && c.shard_optimizer != 0;
    auto add_bucket = [&](size_t lo, size_t hi) {
        Bucket b;
        b.tensor_lo = lo;
        b.tensor_hi = hi;
        b.first = t.tensors[lo].first;
        b.count = t.tensors[hi - 1].first + t.tensors[hi - 1].count - b.first;
        b.sharded = sharded && b.count % static_cast<size_t>(c.world) == 0 &&
                    (b.count / c.world) % 4 == 0;
        t.buckets.push_back(b);
    };
    add_bucket(count - 2, count);                     // ln_f
    for (size_t i = t.layers; i-- > 0;) {
        add_bucket(2 + 12 * i, 2 + 12 * i + 12);      // block i
    }
    add_bucket(0, 2);                                 // wte, wpe

    // What this rank's optimizer owns.
    size_t storage = 0;
    if (!sharded) {
        t.shards.push_back({0, t.arena_count, 0, 1});
        storage = t.arena_count;
    } else {
        for (const Bucket& b : t.buckets) {
            flint_trainer_range s;
            if (b.sharded) {
                const size_t chunk = b.count / c.world;
                s = {b.first + chunk * c.rank, chunk, storage, 0};
            } else {
                s = {b.first, b.count, storage, 1};  // too ragged to split: summed and updated everywhere
            }
            storage += s.count;
            t.shards.push_back(s);
        }
    }
    t.moment_count = storage;
    CUDA(cudaMalloc(reinterpret_cast<void**>(&t.m), storage * 4));
    CUDA(cudaMalloc(reinterpret_cast<void**>(&t.v), storage * 4));
    CUDA(cudaMemset(t.m, 0, storage * 4));
    CUDA(cudaMemset(t.v, 0, storage * 4));
    CUDA(cudaMalloc(reinterpret_cast<void**>(&t.found), 16));
    CUDA(cudaMemset(t.found, 0, 16));
    CUDA(cudaMalloc(reinterpret_cast<void**>(&t.norm_squared), 16));
    CUDA(cudaMemset(t.norm_squared, 0, 16));

    TRY(build_plan(t, 0, t.arena_count, &t.whole));
    if (many && !sharded) {
        // Replicated ranks can update everything but the embeddings while the embeddings'
        // all-reduce, the last and largest, is still in flight.
        const size_t body_first = t.tensors[2].first;
        TRY(build_plan(t, 0, body_first, &t.embeddings));
        TRY(build_plan(t, body_first, t.arena_count, &t.body));
    }

    if (many) {
        if (nccl_id == nullptr) {
            return fail(kInvalid, "flint_trainer_create: nccl_id is null with world (%d) > 1",
                        c.world);
        }
        TRY(load_nccl(&t.nccl));
        CUDA(cudaStreamCreateWithFlags(&t.comm_stream, cudaStreamNonBlocking));
        for (cudaEvent_t* e : {&t.comm_done, &t.flag_ready, &t.updated, &t.checked}) {
            CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        }
        for (Bucket& b : t.buckets) {
            CUDA(cudaEventCreateWithFlags(&b.ready, cudaEventDisableTiming));
            CUDA(cudaEventCreateWithFlags(&b.gathered, cudaEventDisableTiming));
        }
        ncclUniqueId id;
        std::memcpy(&id, nccl_id, sizeof id);
        TRY(nccl_check(t, t.nccl->CommInitRank(&t.comm, c.world, id, c.rank), "ncclCommInitRank"));
    }
    t.status.loss_scale = c.loss_scale;
    CUDA(cudaDeviceSynchronize());
    return FLINT_OK;
}

// ---- one step -----------------------------------------------------------------------------------

bool pipelined(const flint_trainer& t) {
    return t.config.world > 1 && t.config.shard_optimizer == 0 && t.config.overlap_update != 0 &&
           t.config.max_grad_norm <= 0.0f;
}

float inverse_scale(const flint_trainer& t) { return 1.0f / t.status.loss_scale; }

// The backward pass reports bucket `index` complete (its producers are enqueued on the main
// stream): start its collective on the second stream.
void on_bucket(void* user, int index, void* gradients, size_t bytes) {
    flint_trainer& t = *static_cast<flint_trainer*>(user);
    if (!t.reduce_now || t.callback_status != FLINT_OK) {
        return;
    }
    Bucket& b = t.buckets[static_cast<size_t>(index)];
    float* base = t.gradient_arena + b.first;
    auto run = [&]() -> flint_status {
        if (gradients != base || bytes != b.count * 4) {
            return fail(FLINT_ERROR_CUDA, "flint_trainer_step: bucket %d is not where it was planned",
                        index);
        }
        if (t.hook != nullptr) {
            t.hook(t.hook_user, index, gradients, bytes, t.stream);
        }
        const bool last = static_cast<size_t>(index) + 1 == t.buckets.size();
        if (last && pipelined(t)) {
            // This rank's embedding gradients are checked before they are summed: a non-finite
            // value on any rank makes the sum non-finite, so the maximum of the ranks' flags is
            // the flag the summed gradients would raise.
            FLINT(flint_b200_check_gradients(base, b.count, inverse_scale(t), t.found, nullptr,
                                             t.stream));
        }
        CUDA(cudaEventRecord(b.ready, t.stream));
        CUDA(cudaStreamWaitEvent(t.comm_stream, b.ready, 0));
        if (last && pipelined(t)) {
            TRY(nccl_check(t, t.nccl->AllReduce(t.found, t.found, 1, ncclInt32, ncclMax, t.comm,
                                                t.comm_stream), "ncclAllReduce"));
            CUDA(cudaEventRecord(t.flag_ready, t.comm_stream));
        }
        if (b.sharded) {
            const size_t chunk = b.count / t.config.world;
            TRY(nccl_check(t, t.nccl->ReduceScatter(base, base + chunk * t.config.rank, chunk,
                                                    ncclFloat32, ncclSum, t.comm, t.comm_stream),
                           "ncclReduceScatter"));
        } else {
            TRY(nccl_check(t, t.nccl->AllReduce(base, base, b.count, ncclFloat32, ncclSum, t.comm,
                                                t.comm_stream), "ncclAllReduce"));
        }
        return FLINT_OK;
    };
    t.callback_status = run();
}

// Sharded: stage `stage` of the forward pass needs the weights of its bucket, which the
// previous step's all-gather may still be delivering.
void on_stage(void* user, int stage) {
    flint_trainer& t = *static_cast<flint_trainer*>(user);
    if (!t.gather_pending || t.callback_status != FLINT_OK) {
        return;
    }
    const size_t blocks = t.layers;
    size_t bucket;
    if (stage == 0) {
        bucket = t.buckets.size() - 1;                     // embeddings
    } else if (static_cast<size_t>(stage) <= blocks) {
        bucket = 1 + (blocks - static_cast<size_t>(stage));  // block stage - 1
    } else {
        bucket = 0;                                        // ln_f (wte was awaited at stage 0)
    }
    const cudaError_t e = cudaStreamWaitEvent(t.stream, t.buckets[bucket].gathered, 0);
    if (e != cudaSuccess) {
        t.callback_status = cuda_error(e, "cudaStreamWaitEvent");
    }
}

flint_status adamw(flint_trainer& t, const Plan& plan, float grad_scale, cudaStream_t stream) {
    if (plan.items == 0) {
        return FLINT_OK;
    }
    const flint_trainer_config& c = t.config;
    const int step = static_cast<int>(t.status.step_count - t.status.skipped);
    FLINT(flint_b200_adamw_run(plan.device, plan.items, c.lr, c.beta1, c.beta2, c.eps, grad_scale,
                               step, t.found, stream));
    return FLINT_OK;
}

// The optimizer's half of a step once every gradient this rank owns is summed: the
// non-finite check over the owned ranges (combined across ranks when they differ), the
// optional clip, AdamW.
flint_status update(flint_trainer& t, cudaStream_t stream) {
    const flint_trainer_config& c = t.config;
    const bool many = c.world > 1;
    const bool sharded = many && c.shard_optimizer != 0;
    const bool clip = c.max_grad_norm > 0.0f;
    const float inverse = inverse_scale(t);
    CUDA(cudaMemsetAsync(t.found, 0, 4, stream));
    if (clip) {
        CUDA(cudaMemsetAsync(t.norm_squared, 0, 8, stream));
    }
    for (size_t i = 0; i < t.shards.size(); ++i) {
        const flint_trainer_range& s = t.shards[i];
        // Ranges every rank holds in full are counted once towards the norm: by rank 0.
        const bool counted_elsewhere = sharded && s.shared != 0 && c.rank != 0;
        double* norm = clip && !counted_elsewhere ? t.norm_squared : nullptr;
        FLINT(flint_b200_check_gradients(t.gradient_arena + s.first, s.count, inverse, t.found, norm,
                                         stream));
    }
    if (sharded) {
        // Each rank saw only its slices: combine the flags (and the squared norms).
        CUDA(cudaEventRecord(t.checked, stream));
        CUDA(cudaStreamWaitEvent(t.comm_stream, t.checked, 0));
        TRY(nccl_check(t, t.nccl->AllReduce(t.found, t.found, 1, ncclInt32, ncclMax, t.comm,
                                            t.comm_stream), "ncclAllReduce"));
        if (clip) {
            TRY(nccl_check(t, t.nccl->AllReduce(t.norm_squared, t.norm_squared, 1, ncclFloat64,
                                                ncclSum, t.comm, t.comm_stream), "ncclAllReduce"));
        }
        CUDA(cudaEventRecord(t.flag_ready, t.comm_stream));
        CUDA(cudaStreamWaitEvent(stream, t.flag_ready, 0));
    }
    float grad_scale = inverse;
    if (clip) {
        // The clip coefficient needs the norm on the host; clipping is off by default.
        double squared = 0.0;
        CUDA(cudaMemcpyAsync(&squared, t.norm_squared, 8, cudaMemcpyDeviceToHost, stream));
        CUDA(cudaStreamSynchronize(stream));
        const double norm = std::sqrt(squared);
        t.status.grad_norm = norm;
        if (std::isfinite(norm) && norm > c.max_grad_norm) {
            grad_scale *= static_cast<float>(c.max_grad_norm / (norm + 1e-6));
        }
    }
    t.status.step_count += 1;
    TRY(adamw(t, t.whole, grad_scale, stream));
    if (sharded) {
        // Hand the updated weights round, bucket by bucket in the order the next forward
        // pass needs them; each bucket's FP16 copies are refreshed behind its gather.
        CUDA(cudaEventRecord(t.updated, stream));
        CUDA(cudaStreamWaitEvent(t.comm_stream, t.updated, 0));
        std::vector<size_t> order;
        order.push_back(t.buckets.size() - 1);               // embeddings
        for (size_t k = t.buckets.size() - 1; k-- > 1;) {
            order.push_back(k);                               // blocks 0 .. layers-1
        }
        order.push_back(0);                                   // ln_f
        for (const size_t k : order) {
            Bucket& b = t.buckets[k];
            if (b.sharded) {
                const size_t chunk = b.count / c.world;
                float* base = t.master_arena + b.first;
                TRY(nccl_check(t, t.nccl->AllGather(base + chunk * c.rank, base, chunk, ncclFloat32,
                                                    t.comm, t.comm_stream), "ncclAllGather"));
                for (size_t i = b.tensor_lo; i < b.tensor_hi; ++i) {
                    const Tensor& x = t.tensors[i];
                    if (x.half != nullptr) {
                        FLINT(flint_fp32_to_fp16(x.half, x.master, x.count, t.comm_stream));
                    }
                }
            }
            CUDA(cudaEventRecord(b.gathered, t.comm_stream));
        }
        t.gather_pending = true;
    }
    return FLINT_OK;
}

flint_status ensure_loss_buffer(flint_trainer& t, size_t micro_batches) {
    if (micro_batches <= t.loss_capacity) {
        return FLINT_OK;
    }
    if (t.losses != nullptr) {
        CUDA(cudaDeviceSynchronize());
        CUDA(cudaFree(t.losses));
        t.losses = nullptr;
    }
    CUDA(cudaMalloc(reinterpret_cast<void**>(&t.losses), micro_batches * t.rows * 4));
    t.loss_capacity = micro_batches;
    t.host_losses.resize(micro_batches * t.rows);
    return FLINT_OK;
}

}  // namespace

extern "C" {

const char* flint_train_last_error(void) { return g_error.c_str(); }

flint_status flint_train_scale_policy(float scale, int good_steps, int growth_interval,
                                      int found_nonfinite, float* next_scale, int* next_good_steps) {
    if (next_scale == nullptr || next_good_steps == nullptr) {
        return fail(kInvalid, "flint_train_scale_policy: outputs must not be null");
    }
    if (found_nonfinite != 0) {
        *next_scale = scale * 0.5f;
        *next_good_steps = 0;
        return FLINT_OK;
    }
    good_steps += 1;
    if (good_steps >= growth_interval) {
        *next_scale = scale * 2.0f;
        *next_good_steps = 0;
    } else {
        *next_scale = scale;
        *next_good_steps = good_steps;
    }
    return FLINT_OK;
}

flint_status flint_train_nccl_id(void* id) {
    if (id == nullptr) {
        return fail(kInvalid, "flint_train_nccl_id: id is null");
    }
    Nccl* nccl = nullptr;
    TRY(load_nccl(&nccl));
    ncclUniqueId unique;
    const ncclResult_t r = nccl->GetUniqueId(&unique);
    if (r != ncclSuccess) {
        return fail(FLINT_ERROR_CUDA, "ncclGetUniqueId: %s", nccl->GetErrorString(r));
    }
    static_assert(sizeof unique == FLINT_TRAIN_NCCL_ID_BYTES, "ncclUniqueId is 128 bytes");
    std::memcpy(id, &unique, sizeof unique);
    return FLINT_OK;
}

flint_status flint_trainer_create(const flint_trainer_config* config, const void* nccl_id,
                                  flint_trainer** trainer) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_create: trainer is null");
    }
    *trainer = nullptr;
    TRY(check_config(config));
    std::unique_ptr<flint_trainer> t(new (std::nothrow) flint_trainer);
    if (!t) {
        return fail(FLINT_ERROR_CUDA, "flint_trainer_create: out of host memory");
    }
    t->config = *config;
    TRY(build(*t, nccl_id));
    *trainer = t.release();
    return FLINT_OK;
}

void flint_trainer_destroy(flint_trainer* trainer) { delete trainer; }

flint_status flint_trainer_model(flint_trainer* trainer, flint_gpt2** model) {
    if (trainer == nullptr || model == nullptr) {
        return fail(kInvalid, "flint_trainer_model: trainer and model must not be null");
    }
    *model = trainer->model;
    return FLINT_OK;
}

flint_status flint_trainer_weights_changed(flint_trainer* trainer, flint_stream stream) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_weights_changed: trainer is null");
    }
    FLINT(flint_gpt2_sync_weights(trainer->model, stream));
    return FLINT_OK;
}

flint_status flint_trainer_step(flint_trainer* trainer, const void* const* tokens,
                                const void* const* targets, size_t micro_batches,
                                flint_stream stream) {
    constexpr const char* name = "flint_trainer_step";
    if (trainer == nullptr || tokens == nullptr || targets == nullptr) {
        return fail(kInvalid, "%s: trainer, tokens and targets must not be null", name);
    }
    if (micro_batches == 0) {
        return fail(kInvalid, "%s: a step needs at least one micro-batch", name);
    }
    flint_trainer& t = *trainer;
    const flint_trainer_config& c = t.config;
    const bool many = c.world > 1;
    TRY(ensure_loss_buffer(t, micro_batches));
    t.micro_batches = micro_batches;
    t.stream = stream;
    t.callback_status = FLINT_OK;
    const float scale = t.status.loss_scale /
                        (static_cast<float>(t.rows) * static_cast<float>(c.world) *
                         static_cast<float>(micro_batches));
    const bool pipe = pipelined(t);
    if (pipe) {
        CUDA(cudaMemsetAsync(t.found, 0, 4, stream));
    }
    const void* row_loss = nullptr;
    FLINT(flint_gpt2_outputs(t.model, nullptr, nullptr, &row_loss));
    for (size_t i = 0; i < micro_batches; ++i) {
        FLINT(flint_b200_gpt2_forward_stages(t.model, tokens[i], targets[i], scale, stream, on_stage,
                                             &t));
        TRY(t.callback_status);
        t.gather_pending = false;  // this forward pass waited for every bucket
        FLINT(flint_copy(t.losses + i * t.rows, row_loss, t.rows * 4, stream));
        t.reduce_now = many && i + 1 == micro_batches;
        FLINT(flint_b200_gpt2_backward_buckets(t.model, tokens[i], i > 0 ? 1 : 0, stream,
                                               many ? on_bucket : nullptr, &t));
        t.reduce_now = false;
        TRY(t.callback_status);
    }
    if (pipe) {
        // Every bucket but the last is summed while backward runs; the last one (the
        // embeddings, a third of the bytes) would otherwise be waited for with nothing to do.
        // Its non-finite flag is settled early (see on_bucket), so the rest of the model is
        // checked and updated while that all-reduce is in flight.
        const float inverse = inverse_scale(t);
        CUDA(cudaEventRecord(t.comm_done, t.comm_stream));
        CUDA(cudaStreamWaitEvent(stream, t.flag_ready, 0));
        const size_t body_first = t.tensors[2].first;
        FLINT(flint_b200_check_gradients(t.gradient_arena + body_first, t.arena_count - body_first,
                                         inverse, t.found, nullptr, stream));
        t.status.step_count += 1;
        TRY(adamw(t, t.body, inverse, stream));
        CUDA(cudaStreamWaitEvent(stream, t.comm_done, 0));
        TRY(adamw(t, t.embeddings, inverse, stream));
        return FLINT_OK;
    }
    if (many) {
        CUDA(cudaEventRecord(t.comm_done, t.comm_stream));
        CUDA(cudaStreamWaitEvent(stream, t.comm_done, 0));
    }
    return update(t, stream);
}

flint_status flint_trainer_update(flint_trainer* trainer, flint_stream stream) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_update: trainer is null");
    }
    if (trainer->config.world > 1) {
        return fail(kInvalid, "flint_trainer_update: only for world 1 (collectives belong to a step)");
    }
    trainer->stream = stream;
    return update(*trainer, stream);
}

flint_status flint_trainer_finish(flint_trainer* trainer, flint_stream stream, double* mean_loss,
                                  int* skipped) {
    constexpr const char* name = "flint_trainer_finish";
    if (trainer == nullptr) {
        return fail(kInvalid, "%s: trainer is null", name);
    }
    flint_trainer& t = *trainer;
    int found = 0;
    const size_t values = t.micro_batches * t.rows;
    if (t.losses != nullptr && values <= t.host_losses.size()) {
        CUDA(cudaMemcpyAsync(t.host_losses.data(), t.losses, values * 4, cudaMemcpyDeviceToHost,
                             stream));
    }
    CUDA(cudaMemcpyAsync(&found, t.found, 4, cudaMemcpyDeviceToHost, stream));
    CUDA(cudaStreamSynchronize(stream));
    if (mean_loss != nullptr) {
        double sum = 0.0;
        for (size_t i = 0; i < values && i < t.host_losses.size(); ++i) {
            sum += static_cast<double>(t.host_losses[i]);
        }
        *mean_loss = values == 0 ? 0.0 : sum / static_cast<double>(values);
    }
    if (found != 0) {
        t.status.skipped += 1;
    }
    TRY(flint_train_scale_policy(t.status.loss_scale, t.status.good_steps, t.config.growth_interval,
                                 found, &t.status.loss_scale, &t.status.good_steps));
    if (skipped != nullptr) {
        *skipped = found != 0 ? 1 : 0;
    }
    return FLINT_OK;
}

flint_status flint_trainer_synchronize(flint_trainer* trainer, flint_stream stream) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_synchronize: trainer is null");
    }
    CUDA(cudaStreamSynchronize(stream));
    if (trainer->comm_stream != nullptr) {
        CUDA(cudaStreamSynchronize(trainer->comm_stream));
    }
    return FLINT_OK;
}

flint_status flint_trainer_get_status(const flint_trainer* trainer, flint_trainer_status* status) {
    if (trainer == nullptr || status == nullptr) {
        return fail(kInvalid, "flint_trainer_get_status: trainer and status must not be null");
    }
    *status = trainer->status;
    return FLINT_OK;
}

flint_status flint_trainer_set_status(flint_trainer* trainer, const flint_trainer_status* status) {
    if (trainer == nullptr || status == nullptr) {
        return fail(kInvalid, "flint_trainer_set_status: trainer and status must not be null");
    }
    if (!(status->loss_scale > 0.0f) || !std::isfinite(status->loss_scale) ||
        status->step_count < status->skipped || status->skipped < 0 || status->good_steps < 0) {
        return fail(kInvalid, "flint_trainer_set_status: inconsistent status");
    }
    trainer->status.loss_scale = status->loss_scale;
    trainer->status.good_steps = status->good_steps;
    trainer->status.step_count = status->step_count;
    trainer->status.skipped = status->skipped;
    return FLINT_OK;
}

flint_status flint_trainer_moments(flint_trainer* trainer, void** m, void** v, size_t* count) {
    if (trainer == nullptr || m == nullptr || v == nullptr || count == nullptr) {
        return fail(kInvalid, "flint_trainer_moments: arguments must not be null");
    }
    *m = trainer->m;
    *v = trainer->v;
    *count = trainer->moment_count;
    return FLINT_OK;
}

size_t flint_trainer_shard_count(const flint_trainer* trainer) {
    return trainer == nullptr ? 0 : trainer->shards.size();
}

flint_status flint_trainer_shard(const flint_trainer* trainer, size_t index,
                                 flint_trainer_range* shard) {
    if (trainer == nullptr || shard == nullptr) {
        return fail(kInvalid, "flint_trainer_shard: trainer and shard must not be null");
    }
    if (index >= trainer->shards.size()) {
        return fail(kInvalid, "flint_trainer_shard: index (%zu) must be below %zu", index,
                    trainer->shards.size());
    }
    *shard = trainer->shards[index];
    return FLINT_OK;
}

flint_status flint_trainer_flags(flint_trainer* trainer, int** found_nonfinite,
                                 double** norm_squared) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_flags: trainer is null");
    }
    if (found_nonfinite != nullptr) {
        *found_nonfinite = trainer->found;
    }
    if (norm_squared != nullptr) {
        *norm_squared = trainer->norm_squared;
    }
    return FLINT_OK;
}

flint_status flint_trainer_set_bucket_hook(flint_trainer* trainer, flint_trainer_bucket_hook hook,
                                           void* user) {
    if (trainer == nullptr) {
        return fail(kInvalid, "flint_trainer_set_bucket_hook: trainer is null");
    }
    trainer->hook = hook;
    trainer->hook_user = user;
    return FLINT_OK;
}

}  // extern "C"
