// The GPT-2 model object behind flint_gpt2_* and the trainer extension.
#pragma once

#include <cstddef>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "flint/flint.h"

namespace fb {

struct Tensor {
    std::string name;
    size_t rows = 0;
    size_t cols = 0;
    void* data = nullptr;      // FP32 master
    void* gradient = nullptr;  // FP32 gradient (backward models)
    void* half = nullptr;      // FP16 compute copy (matrices only)
    size_t count() const { return rows * cols; }
};

// Saved activations of one transformer block (pointers into the arena).
struct BlockBuffers {
    void* x_in = nullptr;    // FP32 residual entering the block
    void* x_mid = nullptr;   // FP32 residual after attention
    void* x_out = nullptr;   // FP32 residual leaving the block
    void* h1 = nullptr;      // FP16 LayerNorm-1 output
    void* mean1 = nullptr;
    void* rstd1 = nullptr;
    void* q = nullptr;       // FP16 heads layout [B, H, T, hw]
    void* k = nullptr;
    void* v = nullptr;
    void* qkv = nullptr;     // FP16 packed qkv rows [rows, 3 width] (flash attention only)
    void* p = nullptr;       // FP16 probabilities [B*H, T, T] (unfused attention only)
    void* lse = nullptr;     // FP32 log-sum-exp [B*H, T] (flash attention only)
    void* attn = nullptr;    // FP16 merged attention output [rows, width]
    void* h2 = nullptr;
    void* mean2 = nullptr;
    void* rstd2 = nullptr;
    void* gelu = nullptr;    // FP16 [rows, 4 width]
    void* pre = nullptr;     // FP16 [rows, 4 width]
};

struct BlockWeights {
    Tensor* ln1_w;
    Tensor* ln1_b;
    Tensor* attn_w;   // [3w, w]
    Tensor* attn_b;
    Tensor* proj_w;   // [w, w]
    Tensor* proj_b;
    Tensor* ln2_w;
    Tensor* ln2_b;
    Tensor* fc_w;     // [4w, w]
    Tensor* fc_b;
    Tensor* fcproj_w; // [w, 4w]
    Tensor* fcproj_b;
};

}  // namespace fb

struct flint_gpt2 {
    flint_gpt2_config config{};
    bool flash = false;          // fused attention (extension); no T x T buffers
    size_t rows = 0;
    size_t head_width = 0;
    size_t head_batches = 0;

    std::vector<fb::Tensor> tensors;  // PyTorch named_parameters order
    std::vector<fb::BlockWeights> weights;
    std::vector<fb::BlockBuffers> blocks;
    fb::Tensor* wte = nullptr;
    fb::Tensor* wpe = nullptr;
    fb::Tensor* lnf_w = nullptr;
    fb::Tensor* lnf_b = nullptr;

    void* x_final = nullptr;
    void* h_f = nullptr;
    void* mean_f = nullptr;
    void* rstd_f = nullptr;
    void* qkv = nullptr;
    void* scores = nullptr;
    void* heads_out = nullptr;
    void* logits = nullptr;
    void* dlogits = nullptr;
    void* row_loss = nullptr;
    void* dres = nullptr;
    void* dres_half = nullptr;
    void* dh = nullptr;
    void* dpre = nullptr;
    void* dq = nullptr;
    void* dk = nullptr;
    void* dv = nullptr;
    void* delta = nullptr;       // flash attention backward: rowsum(dO * O), FP32 [B*H, T]
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    void* tn_workspace = nullptr;
    size_t tn_workspace_bytes = 0;
    // The fused-attention model puts a block's column-sum second passes off to one launch:
    // six regions of partial sums, in the order backward_block produces them.
    void* column_workspace = nullptr;
    size_t column_workspace_bytes = 0;
    size_t column_offsets[6] = {};

    struct Slot {
        void** target;
        size_t bytes;
    };
    std::vector<Slot> slots;
    std::vector<void*> allocations;
    std::vector<float> host_row_loss;

    // Gradient byte ranges, for collectives: the whole gradient arena and one
    // range per bucket in the order the backward pass completes them
    // (ln_f, blocks last to first, then wpe+wte). Valid in single-arena mode.
    void* gradient_base = nullptr;
    size_t gradient_bytes = 0;

    flint_gpt2() = default;
    flint_gpt2(const flint_gpt2&) = delete;
    flint_gpt2& operator=(const flint_gpt2&) = delete;
    ~flint_gpt2();
};
