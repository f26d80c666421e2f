// Internal launchers of the fused attention kernels, shared by the C ABI and
// the GPT-2 assembly. Tensors are FP16 with a head width of 64 and are
// addressed as (column, row, head, sequence) through element strides, so both
// the heads layout [B, H, T, 64] and packed qkv rows [B*T, 3*H*64] work.
#pragma once

#include <cstddef>

#include <cuda_runtime_api.h>

namespace fb {

struct AttentionView {
    const void* base;
    long long row_stride;       // elements between consecutive positions
    long long head_stride;      // elements between heads
    long long sequence_stride;  // elements between sequences
};

struct AttentionShape {
    size_t sequences;
    size_t heads;
    size_t length;
};

// lse: FP32 [sequences * heads, length].
cudaError_t attention_forward(const AttentionView& o, float* lse, const AttentionView& q,
                              const AttentionView& k, const AttentionView& v,
                              const AttentionShape& shape, float scale, cudaStream_t stream);

// delta: FP32 scratch [sequences * heads, length]. dk and dv must share strides.
cudaError_t attention_backward(const AttentionView& dq, const AttentionView& dk,
                               const AttentionView& dv, const AttentionView& d_o,
                               const AttentionView& o, const float* lse, float* delta,
                               const AttentionView& q, const AttentionView& k,
                               const AttentionView& v, const AttentionShape& shape, float scale,
                               cudaStream_t stream);

// Clocks one CTA needs to get `count` small MMAs accepted and completed (a diagnostic).
cudaError_t mma_clocks(int n, int a_in_tmem, int count, long long* issue, long long* complete,
                       cudaStream_t stream);

cudaError_t attention_error_flag(int* value, bool reset);

}  // namespace fb
