// Internal launchers of the tensor-core GEMM, shared by the C ABI layer, the
// GPT-2 assembly and the trainer. They expect arguments that already passed
// the ABI's checks.
#pragma once

#include <cstddef>

#include <cuda_runtime_api.h>

namespace fb {

enum class Layout { kNT, kNN, kTN };

enum class Epilogue {
    kNone,          // FP16 store
    kBias,          // + bias[n]
    kBiasGelu,      // + bias, store pre-activation and GELU
    kDGelu,         // * GELU'(pre)
    kBiasResidual,  // FP32: residual + (acc + bias)
    kScale,         // * scale
    kTnStore,       // FP32 store or old + acc
    kTnPartial      // FP32 store into the split's slice of the workspace
};

// How flint_gemm_tn divides k: `count` CTAs per output tile, each taking
// `len` (a multiple of 64) consecutive rows of k. count == 1 needs no workspace.
struct TnSplit {
    int count;
    int len;
};

TnSplit tn_split(size_t m, size_t n, size_t k, int sms);

cudaError_t gemm_nt(Epilogue e, void* y, void* pre, const void* x, const void* w,
                    const void* bias, const void* residual, size_t m, size_t n, size_t k,
                    cudaStream_t stream);

cudaError_t gemm_nn(Epilogue e, void* y, const void* x, const void* w, const void* pre, size_t m,
                    size_t n, size_t k, cudaStream_t stream);

cudaError_t gemm_tn(void* y, const void* x, const void* w, size_t m, size_t n, size_t k,
                    bool accumulate, void* workspace, cudaStream_t stream);

// NT applies `scale`; NN and TN ignore it. TN writes FP16 and never splits k.
cudaError_t gemm_batched(Layout l, void* y, const void* x, const void* w, size_t batches,
                         size_t m, size_t n, size_t k, float scale, cudaStream_t stream);

// Reads (and optionally clears) the flag a kernel raises when one of its
// bounded barrier waits ran out. Synchronises the device.
cudaError_t gemm_error_flag(int* value, bool reset);

}  // namespace fb
