// Shared host-side plumbing of the C ABI: the per-thread error message, the
// pointer checks every entry point performs, and small device helpers.
//
// The check order and message texts follow the reference's validation layer
// (src/common/checks.cpp:7-34, src/common/error.cpp:9-21), because callers
// match on them.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>

#include <cuda_runtime_api.h>

#include "flint/flint.h"

namespace fb {

// Stores a printf-style message for flint_last_error() and returns status.
flint_status fail(flint_status status, const char* format, ...)
    __attribute__((__format__(__printf__, 2, 3)));

// Reports a CUDA runtime error as FLINT_ERROR_CUDA and clears the sticky
// last-error slot so the next launch does not inherit it.
flint_status cuda_fail(cudaError_t error, const char* file, int line);

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

inline bool fits(const void* p, size_t bytes) {
    return bytes <= UINTPTR_MAX - reinterpret_cast<uintptr_t>(p);
}

inline bool overlap(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a);
    const uintptr_t b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + b_bytes && b0 < a0 + a_bytes;
}

struct Span {
    const char* name;
    const void* pointer;
    size_t bytes;
};

// In list order: null, then alignment, then address-space fit for every span;
// only then each of the first `outputs` spans against every later span.
flint_status check_spans(const char* function, const Span* spans, size_t count, size_t outputs);

template <size_t N>
flint_status check_spans(const char* function, const Span (&spans)[N], size_t outputs) {
    return check_spans(function, spans, N, outputs);
}

// cudaGetLastError() for the line after a kernel launch; also counts the launch
// (flint_b200_launch_count reports the total).
cudaError_t after_launch();
unsigned long long launch_count();

// Launches `kernel` so that it may begin while the kernel before it in the stream
// is still draining (programmatic dependent launch): its CTAs become resident as the
// earlier kernel's CTAs retire, and its set-up (barrier initialisation, tensor-memory
// allocation, index arithmetic) overlaps that tail. Every kernel launched this way
// calls fb::dependency_wait() before its first access to global memory; the earlier
// kernel allows the early start with fb::dependency_release(). FLINT_B200_PDL=0 in the
// environment turns the attribute off (plain stream order). Counts the launch.
bool dependent_launch_enabled();

template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launch_enabled() ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
    const cudaError_t last = after_launch();
    return e != cudaSuccess ? e : last;
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute belongs
// to the device's copy of the function); `done` is the caller's static per-kernel table.
// Host threads may race on a first call: the slots are atomics and the attribute call is
// idempotent, so two threads that both miss simply set it twice.
template <typename Kernel>
cudaError_t allow_shared_memory(Kernel kernel, int bytes, std::atomic<bool> (&done)[64]) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        return e;
    }
    if (device >= 0 && device < 64 && done[device].load(std::memory_order_relaxed)) {
        return cudaSuccess;
    }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && device >= 0 && device < 64) {
        done[device].store(true, std::memory_order_relaxed);
    }
    return e;
}

// Number of SMs of the current device (cached per device index).
cudaError_t sm_count(int* sms);

// Tensor map over a row-major matrix [rows, cols] of 2- or 4-byte elements (zero
// fill outside; swizzle_bytes 0 or 64), for boxes of box_cols x box_rows. The row
// pitch must be a multiple of 16 bytes and both extents below 2^32.
cudaError_t encode_rows_map(void* map, const void* base, size_t rows, size_t cols,
                            int element_bytes, unsigned box_cols, unsigned box_rows,
                            int swizzle_bytes = 0);

// LayerNorm forward whose row sums use plain FP32 adds (see rowwise.cu); returns false, having
// launched nothing, for shapes it does not cover.
bool launch_layernorm_forward_plain(void* y, void* mean, void* rstd, const void* x,
                                    const void* gamma, const void* beta, size_t rows, size_t cols,
                                    float eps, cudaStream_t stream, cudaError_t* error);

// Second passes of column sums that are put off and then run as one launch: the model on the
// fused attention kernels collects a block's eight (four bias gradients, two LayerNorms'
// gain and bias gradients) and finishes them together, which takes seven short dependent
// launches per block off the stream. Each job's partial sums need their own workspace
// region until then; an output is computed exactly as its own second pass would.
struct ColumnFinishList {
    static constexpr int kMost = 8;
    struct Job {
        void* out;
        const void* partial;
        size_t cols;
        bool accumulate;
    };
    Job jobs[kMost];
    int count = 0;
    bool add(void* out, const void* partial, size_t cols, bool accumulate) {
        if (count == kMost) {
            return false;
        }
        jobs[count++] = Job{out, partial, cols, accumulate};
        return true;
    }
};
// Bytes of partial sums one column-sum job over [rows, cols] writes.
size_t column_partial_bytes(size_t rows, size_t cols);
cudaError_t launch_column_finishes(const ColumnFinishList& list, size_t rows, cudaStream_t stream);

// flint_layernorm_backward's kernels without the argument checks, for the model
// assembly; dx_half, when not null, also receives dx rounded to FP16 (the next
// GEMM's operand), which saves a separate conversion pass over dx.
cudaError_t launch_layernorm_backward(void* dx, void* dgamma, void* dbeta, const void* dy,
                                      const void* x, const void* mean, const void* rstd,
                                      const void* gamma, size_t rows, size_t cols,
                                      bool accumulate_dx, bool accumulate_params, void* workspace,
                                      cudaStream_t stream, void* dx_half, bool plain,
                                      ColumnFinishList* later = nullptr);

// flint_bias_gradient's kernels without the argument checks. `plain` (here and above)
// selects column sums whose row streams use ordinary FP32 adds, merged by compensated
// adds in the same fixed order: deterministic, within a few 2^-24 of the pinned
// arithmetic's result, about seven times less FP32 work. The public entry points pass
// false; the model built on the fused attention kernels passes true.
// With `later` (both launchers) the second passes are appended to the list instead of being
// launched; the workspace must then stay untouched until launch_column_finishes has run.
cudaError_t launch_bias_gradient(void* dbias, const void* dy, size_t rows, size_t cols,
                                 bool accumulate, void* workspace, cudaStream_t stream,
                                 bool plain, ColumnFinishList* later = nullptr);

// Device error word of the column-sum kernels: set when a bounded wait for a
// staged row gave up (read, and cleared if asked, by flint_b200_kernel_fault).
cudaError_t reductions_error_flag(int* value, bool reset);
// The same for the cross-entropy kernel that stages whole rows by bulk copy.
cudaError_t rowwise_error_flag(int* value, bool reset);

}  // namespace fb

#define FB_CUDA(call)                                                  \
    do {                                                               \
        const cudaError_t fb_cuda_error_ = (call);                     \
        if (fb_cuda_error_ != cudaSuccess) {                           \
            return ::fb::cuda_fail(fb_cuda_error_, __FILE__, __LINE__); \
        }                                                              \
    } while (0)

#define FB_TRY(call)                               \
    do {                                           \
        const flint_status fb_status_ = (call);    \
        if (fb_status_ != FLINT_OK) {              \
            return fb_status_;                     \
        }                                          \
    } while (0)
