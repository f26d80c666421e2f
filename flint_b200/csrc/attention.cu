// Placeholder: the fused attention kernels are built in a later step.
#include "common.h"
#include "flint/flint_b200.h"

extern "C" {

flint_status flint_b200_attention_forward(void*, void*, const void*, const void*, const void*,
                                          size_t, size_t, size_t, float, flint_stream) {
    return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                    "flint_b200_attention_forward: not available in this build");
}

flint_status flint_b200_attention_backward(void*, void*, void*, const void*, const void*,
                                           const void*, void*, const void*, const void*,
                                           const void*, size_t, size_t, size_t, float,
                                           flint_stream) {
    return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                    "flint_b200_attention_backward: not available in this build");
}

}  // extern "C"
