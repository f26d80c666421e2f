// Error slot, span checks, version and status strings (the GPU-free part of the ABI).
#include "common.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include <cuda.h>

#ifndef FLINT_VERSION
#define FLINT_VERSION "0.1.0"
#endif

namespace {

// One message per thread; longer messages are truncated.
thread_local char g_last_error[512] = "";

}  // namespace

namespace fb {

flint_status fail(flint_status status, const char* format, ...) {
    va_list args;
    va_start(args, format);
    std::vsnprintf(g_last_error, sizeof g_last_error, format, args);
    va_end(args);
    return status;
}

flint_status cuda_fail(cudaError_t error, const char* file, int line) {
    cudaGetLastError();
    return fail(FLINT_ERROR_CUDA, "%s: %s (%s:%d)", cudaGetErrorName(error),
                cudaGetErrorString(error), file, line);
}

flint_status check_spans(const char* function, const Span* spans, size_t count, size_t outputs) {
    for (size_t i = 0; i < count; ++i) {
        const Span& s = spans[i];
        if (s.pointer == nullptr) {
            return fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: %s is null", function, s.name);
        }
        if (!aligned16(s.pointer)) {
            return fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: %s is not 16-byte aligned", function,
                        s.name);
        }
        if (!fits(s.pointer, s.bytes)) {
            return fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: %s runs past the end of the address space", function, s.name);
        }
    }
    for (size_t i = 0; i < outputs && i < count; ++i) {
        for (size_t j = i + 1; j < count; ++j) {
            if (overlap(spans[i].pointer, spans[i].bytes, spans[j].pointer, spans[j].bytes)) {
                return fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: %s and %s overlap", function,
                            spans[i].name, spans[j].name);
            }
        }
    }
    return FLINT_OK;
}

namespace {
std::atomic<unsigned long long> g_launches{0};
}

bool dependent_launch_enabled() {
    static const bool enabled = [] {
        const char* v = std::getenv("FLINT_B200_PDL");
        return !(v != nullptr && v[0] == '0');
    }();
    return enabled;
}

cudaError_t after_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

cudaError_t sm_count(int* sms) {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices] = {};
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) {
        return error;
    }
    if (device >= 0 && device < kMaxDevices && cached[device] > 0) {
        *sms = cached[device];
        return cudaSuccess;
    }
    int value = 0;
    error = cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device);
    if (error != cudaSuccess) {
        return error;
    }
    if (device >= 0 && device < kMaxDevices) {
        cached[device] = value;
    }
    *sms = value;
    return cudaSuccess;
}

cudaError_t encode_rows_map(void* map, const void* base, size_t rows, size_t cols,
                            int element_bytes, unsigned box_cols, unsigned box_rows,
                            int swizzle_bytes) {
    using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        const cudaError_t e =
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
        if (e != cudaSuccess) {
            return e;
        }
        if (status != cudaDriverEntryPointSuccess || fn == nullptr) {
            return cudaErrorNotSupported;
        }
        encode = reinterpret_cast<Encode>(fn);
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * static_cast<cuuint64_t>(element_bytes)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUtensorMapDataType type =
        element_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = encode(static_cast<CUtensorMap*>(map), type, 2, const_cast<void*>(base), dims,
                              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}


}  // namespace fb

extern "C" {

const char* flint_version(void) { return FLINT_VERSION; }

const char* flint_status_string(flint_status status) {
    switch (status) {
    case FLINT_OK:
        return "ok";
    case FLINT_ERROR_INVALID_ARGUMENT:
        return "invalid argument";
    case FLINT_ERROR_CUDA:
        return "CUDA error";
    default:
        return "unknown status";
    }
}

const char* flint_last_error(void) { return g_last_error; }

}  // extern "C"
