// flint_gpt2_*: GPT-2's memory plan, forward pass and backward pass, composed
// from the library's own entry points on one stream (host code only).
//
// The buffer list, parameter order and names, the order of operations and the
// accumulate semantics are those of the reference's src/api/gpt2.cpp:187-848:
// flint_gpt2_bytes is the sum of the same buffers rounded to 256 bytes, the
// residual stream and its gradient are FP32, a linear layer's output gradient
// is the residual gradient rounded to FP16, attention is unfused (scores and
// probabilities materialised per head), and wte's gradient is
// (old + output layer) + embedding.
//
// Models created through flint_b200_gpt2_create with flash attention replace
// the T x T score/probability buffers by the fused attention kernels; that
// path is an extension and not part of the drop-in contract.
#include <algorithm>
#include <cmath>
#include <memory>
#include <new>
#include <string>

#include <cuda_fp16.h>

#include "attention.h"
#include "common.h"
#include "flint/flint_b200.h"
#include "gpt2.h"

namespace {

using fb::BlockBuffers;
using fb::BlockWeights;
using fb::Tensor;

constexpr size_t kAlign = 256;  // cudaMalloc's granularity, so one arena lays out like many
constexpr size_t kMaxLayers = 1024;
constexpr size_t kMaxWidth = 16384;
constexpr size_t kMaxLength = 1024;
constexpr size_t kMaxHeadBatches = 65535;
constexpr size_t kMaxPaddedVocab = 65536;
constexpr size_t kMaxRows = size_t{65535} * 128;
constexpr size_t kMaxBackwardRows = 65536;
constexpr size_t kMaxPositionValues = 16776960;
constexpr float kEps = 1e-5f;
constexpr flint_status kInvalid = FLINT_ERROR_INVALID_ARGUMENT;

size_t round_up(size_t bytes) { return (bytes + kAlign - 1) / kAlign * kAlign; }

flint_status check_config(const char* name, const flint_gpt2_config* config) {
    if (config == nullptr) {
        return fb::fail(kInvalid, "%s: config is null", name);
    }
    const flint_gpt2_config& c = *config;
    if (c.layers == 0 || c.layers > kMaxLayers) {
        return fb::fail(kInvalid, "%s: layers (%zu) must be from 1 to %zu", name, c.layers,
                        kMaxLayers);
    }
    if (c.width == 0 || c.width % 8 != 0 || c.width > kMaxWidth) {
        return fb::fail(kInvalid, "%s: width (%zu) must be a multiple of 8 from 8 to %zu", name,
                        c.width, kMaxWidth);
    }
    if (c.heads == 0 || c.width % c.heads != 0 || (c.width / c.heads) % 8 != 0) {
        return fb::fail(kInvalid, "%s: heads (%zu) must split width (%zu) into multiples of 8",
                        name, c.heads, c.width);
    }
    if (c.length == 0 || c.length % 8 != 0 || c.length > kMaxLength) {
        return fb::fail(kInvalid, "%s: length (%zu) must be a multiple of 8 from 8 to %zu", name,
                        c.length, kMaxLength);
    }
    if (c.block_size < c.length || c.block_size > kMaxLength) {
        return fb::fail(kInvalid, "%s: block_size (%zu) must be from length (%zu) to %zu", name,
                        c.block_size, c.length, kMaxLength);
    }
    if (c.padded_vocab == 0 || c.padded_vocab % 8 != 0 || c.padded_vocab > kMaxPaddedVocab) {
        return fb::fail(kInvalid, "%s: padded_vocab (%zu) must be a multiple of 8 from 8 to %zu",
                        name, c.padded_vocab, kMaxPaddedVocab);
    }
    if (c.vocab == 0 || c.vocab > c.padded_vocab) {
        return fb::fail(kInvalid, "%s: vocab (%zu) must be from 1 to padded_vocab (%zu)", name,
                        c.vocab, c.padded_vocab);
    }
    if (c.sequences == 0 || c.sequences > kMaxHeadBatches / c.heads) {
        return fb::fail(kInvalid, "%s: sequences (%zu) x heads (%zu) must be from 1 to %zu", name,
                        c.sequences, c.heads, kMaxHeadBatches);
    }
    if (c.sequences > kMaxRows / c.length) {
        return fb::fail(kInvalid, "%s: sequences (%zu) x length (%zu) can be up to %zu rows", name,
                        c.sequences, c.length, kMaxRows);
    }
    if (c.backward != 0) {
        if (c.sequences > kMaxBackwardRows / c.length) {
            return fb::fail(kInvalid,
                            "%s: sequences (%zu) x length (%zu) can be up to %zu rows with "
                            "backward",
                            name, c.sequences, c.length, kMaxBackwardRows);
        }
        if (c.length > kMaxPositionValues / c.width) {
            return fb::fail(kInvalid,
                            "%s: length (%zu) x width (%zu) can be up to %zu with backward", name,
                            c.length, c.width, kMaxPositionValues);
        }
    }
    return FLINT_OK;
}

Tensor* add_tensor(flint_gpt2& m, std::string name, size_t rows, size_t cols) {
    m.tensors.push_back(Tensor{std::move(name), rows, cols});
    return &m.tensors.back();
}

void want(flint_gpt2& m, void** target, size_t bytes) { m.slots.push_back({target, bytes}); }

flint_status size_workspaces(flint_gpt2& m) {
    const flint_gpt2_config& c = m.config;
    const size_t w = c.width;
    size_t bytes = 0;
    size_t most = 0;
    for (const size_t cols : {w, 3 * w, 4 * w}) {
        FB_TRY(flint_bias_gradient_workspace(m.rows, cols, &bytes));
        most = std::max(most, bytes);
    }
    FB_TRY(flint_layernorm_backward_workspace(m.rows, w, &bytes));
    // The fused-attention model's LayerNorm backward writes dgamma's and dbeta's partial
    // sums as two blocks of the public size, one behind the other.
    most = std::max(most, m.flash ? 2 * bytes : bytes);
    FB_TRY(flint_embedding_backward_workspace(c.sequences, c.length, c.padded_vocab, w, &bytes));
    m.workspace_bytes = std::max(most, bytes);

    const size_t shapes[][2] = {
        {c.padded_vocab, w}, {3 * w, w}, {w, w}, {4 * w, w}, {w, 4 * w}};
    most = 0;
    for (const auto& s : shapes) {
        FB_TRY(flint_gemm_tn_workspace(s[0], s[1], m.rows, &bytes));
        most = std::max(most, bytes);
    }
    m.tn_workspace_bytes = most;
    // fcproj bias, fc bias, LayerNorm 2 (gain then bias), proj bias, qkv bias, LayerNorm 1.
    const size_t region_cols[6] = {w, 4 * w, 2 * w, w, 3 * w, 2 * w};
    size_t at = 0;
    for (int r = 0; r < 6; ++r) {
        m.column_offsets[r] = at;
        at += (fb::column_partial_bytes(m.rows, region_cols[r]) + 255) / 256 * 256;
    }
    m.column_workspace_bytes = at;
    return FLINT_OK;
}

// Registers every tensor and buffer; allocates nothing.
flint_status plan(flint_gpt2& m) {
    const flint_gpt2_config& c = m.config;
    const bool backward = c.backward != 0;
    const size_t w = c.width;
    m.rows = c.sequences * c.length;
    m.head_width = w / c.heads;
    m.head_batches = c.sequences * c.heads;

    m.tensors.reserve(4 + 12 * c.layers);
    m.wte = add_tensor(m, "wte.weight", c.padded_vocab, w);
    m.wpe = add_tensor(m, "wpe.weight", c.block_size, w);
    m.weights.resize(c.layers);
    m.blocks.resize(c.layers);
    for (size_t i = 0; i < c.layers; ++i) {
        const std::string prefix = "blocks." + std::to_string(i) + ".";
        BlockWeights& b = m.weights[i];
        b.ln1_w = add_tensor(m, prefix + "ln_1.weight", 1, w);
        b.ln1_b = add_tensor(m, prefix + "ln_1.bias", 1, w);
        b.attn_w = add_tensor(m, prefix + "attn.c_attn.weight", 3 * w, w);
        b.attn_b = add_tensor(m, prefix + "attn.c_attn.bias", 1, 3 * w);
        b.proj_w = add_tensor(m, prefix + "attn.c_proj.weight", w, w);
        b.proj_b = add_tensor(m, prefix + "attn.c_proj.bias", 1, w);
        b.ln2_w = add_tensor(m, prefix + "ln_2.weight", 1, w);
        b.ln2_b = add_tensor(m, prefix + "ln_2.bias", 1, w);
        b.fc_w = add_tensor(m, prefix + "mlp.c_fc.weight", 4 * w, w);
        b.fc_b = add_tensor(m, prefix + "mlp.c_fc.bias", 1, 4 * w);
        b.fcproj_w = add_tensor(m, prefix + "mlp.c_proj.weight", w, 4 * w);
        b.fcproj_b = add_tensor(m, prefix + "mlp.c_proj.bias", 1, w);
    }
    m.lnf_w = add_tensor(m, "ln_f.weight", 1, w);
    m.lnf_b = add_tensor(m, "ln_f.bias", 1, w);

    for (Tensor& t : m.tensors) {
        want(m, &t.data, t.count() * 4);
    }
    if (backward) {
        for (Tensor& t : m.tensors) {
            want(m, &t.gradient, t.count() * 4);
        }
    }
    want(m, &m.wte->half, m.wte->count() * 2);
    for (BlockWeights& b : m.weights) {
        for (Tensor* t : {b.attn_w, b.proj_w, b.fc_w, b.fcproj_w}) {
            want(m, &t->half, t->count() * 2);
        }
    }

    const size_t rows = m.rows;
    const size_t residual = rows * w * 4;
    const size_t rows16 = rows * w * 2;
    const size_t heads16 = rows * w * 2;
    const size_t matrix16 = m.head_batches * c.length * c.length * 2;
    const size_t stats = m.head_batches * c.length * 4;
    const size_t wide16 = rows * 4 * w * 2;

    auto want_block = [&](BlockBuffers& a) {
        want(m, &a.h1, rows16);
        want(m, &a.mean1, rows * 4);
        want(m, &a.rstd1, rows * 4);
        if (m.flash) {
            // The fused kernels read Q, K and V straight from the packed qkv rows.
            if (backward) {
                want(m, &a.qkv, rows * 3 * w * 2);
            }
            want(m, &a.lse, stats);
        } else {
            want(m, &a.q, heads16);
            want(m, &a.k, heads16);
            want(m, &a.v, heads16);
            want(m, &a.p, matrix16);
        }
        want(m, &a.attn, rows16);
    };

    if (backward) {
        for (BlockBuffers& a : m.blocks) {
            want(m, &a.x_in, residual);
            want(m, &a.x_mid, residual);
        }
        want(m, &m.x_final, residual);
        for (BlockBuffers& a : m.blocks) {
            want_block(a);
            want(m, &a.h2, rows16);
            want(m, &a.mean2, rows * 4);
            want(m, &a.rstd2, rows * 4);
            want(m, &a.gelu, wide16);
            want(m, &a.pre, wide16);
        }
        want(m, &m.h_f, rows16);
        want(m, &m.mean_f, rows * 4);
        want(m, &m.rstd_f, rows * 4);
        want(m, &m.qkv, rows * 3 * w * 2);
        if (!m.flash) {
            want(m, &m.scores, matrix16);
        } else {
            want(m, &m.delta, stats);
        }
        if (!m.flash) {
            want(m, &m.heads_out, heads16);
        }
        FB_TRY(size_workspaces(m));
        want(m, &m.dres, residual);
        want(m, &m.dres_half, rows16);
        want(m, &m.dh, rows16);
        want(m, &m.dpre, wide16);
        if (!m.flash) {
            want(m, &m.dq, heads16);
            want(m, &m.dk, heads16);
            want(m, &m.dv, heads16);
        }
        want(m, &m.workspace, m.workspace_bytes);
        want(m, &m.tn_workspace, m.tn_workspace_bytes);
        if (m.flash) {
            want(m, &m.column_workspace, m.column_workspace_bytes);
        }
    } else {
        // One set of activations shared by every block; the residual stream
        // ping-pongs between x_in and x_mid.
        BlockBuffers& a = m.blocks[0];
        want(m, &a.x_in, residual);
        want(m, &a.x_mid, residual);
        want_block(a);
        want(m, &m.qkv, rows * 3 * w * 2);
        if (!m.flash) {
            want(m, &m.scores, matrix16);
            want(m, &m.heads_out, heads16);
        }
        want(m, &a.gelu, wide16);
        want(m, &a.pre, wide16);
    }
    want(m, &m.logits, rows * c.padded_vocab * 2);
    want(m, &m.dlogits, rows * c.padded_vocab * 2);
    want(m, &m.row_loss, rows * 4);
    return FLINT_OK;
}

size_t planned_bytes(const flint_gpt2& m) {
    size_t total = 0;
    for (const flint_gpt2::Slot& s : m.slots) {
        total += round_up(s.bytes);
    }
    return total;
}

flint_status allocate(flint_gpt2& m) {
    m.allocations.reserve(m.slots.size());
    if (m.config.separate_buffers != 0) {
        for (const flint_gpt2::Slot& s : m.slots) {
            void* p = nullptr;
            FB_CUDA(cudaMalloc(&p, s.bytes));
            m.allocations.push_back(p);
            *s.target = p;
        }
        return FLINT_OK;
    }
    void* base = nullptr;
    FB_CUDA(cudaMalloc(&base, planned_bytes(m)));
    m.allocations.push_back(base);
    char* at = static_cast<char*>(base);
    for (const flint_gpt2::Slot& s : m.slots) {
        *s.target = at;
        at += round_up(s.bytes);
    }
    if (m.config.backward != 0) {
        m.gradient_base = m.tensors.front().gradient;
        const Tensor& last = m.tensors.back();
        m.gradient_bytes = static_cast<size_t>(static_cast<char*>(last.gradient) -
                                               static_cast<char*>(m.gradient_base)) +
                           round_up(last.count() * 4);
        // A trainer treats the arena as one FP32 array (non-finite check, all-reduce). The
        // 256-byte rounding gaps between tensors are never written by backward, so they
        // start as zeros rather than as whatever the allocation held.
        FB_CUDA(cudaMemset(m.gradient_base, 0, m.gradient_bytes));
    }
    return FLINT_OK;
}

void link(flint_gpt2& m) {
    if (m.config.backward != 0) {
        for (size_t i = 0; i < m.blocks.size(); ++i) {
            m.blocks[i].x_out = i + 1 < m.blocks.size() ? m.blocks[i + 1].x_in : m.x_final;
        }
        return;
    }
    BlockBuffers& shared = m.blocks[0];
    shared.qkv = m.qkv;
    shared.x_out = shared.x_in;
    shared.h2 = shared.h1;
    shared.mean2 = shared.mean1;
    shared.rstd2 = shared.rstd1;
    for (BlockBuffers& b : m.blocks) {
        b = shared;
    }
    m.x_final = shared.x_in;
    m.h_f = shared.h1;
    m.mean_f = shared.mean1;
    m.rstd_f = shared.rstd1;
}

// Heads of 64 columns inside rows of `row_width` FP16 values, starting at column `first`.
fb::AttentionView rows_view(const void* base, size_t first, size_t row_width, size_t length) {
    return fb::AttentionView{static_cast<const __half*>(base) + first,
                             static_cast<long long>(row_width), 64,
                             static_cast<long long>(length * row_width)};
}

float score_scale(size_t head_width) { return 1.0f / std::sqrt(static_cast<float>(head_width)); }

flint_status layernorm(const flint_gpt2& m, const Tensor* gain, const Tensor* bias, const void* x,
                       void* y, void* mean, void* rstd, flint_stream s) {
    if (m.flash) {
        // The extension model is not bound to the reference's bit pattern: plain row sums.
        cudaError_t e = cudaSuccess;
        if (fb::launch_layernorm_forward_plain(y, mean, rstd, x, gain->data, bias->data, m.rows,
                                               m.config.width, kEps, s, &e)) {
            FB_CUDA(e);
            return FLINT_OK;
        }
    }
    return flint_layernorm_forward(y, mean, rstd, x, gain->data, bias->data, m.rows,
                                   m.config.width, kEps, s);
}

flint_status forward_block(const flint_gpt2& m, size_t i, flint_stream s) {
    const flint_gpt2_config& c = m.config;
    const BlockWeights& wt = m.weights[i];
    const BlockBuffers& a = m.blocks[i];
    const size_t rows = m.rows;
    const size_t w = c.width;
    const size_t hw = m.head_width;

    FB_TRY(layernorm(m, wt.ln1_w, wt.ln1_b, a.x_in, a.h1, a.mean1, a.rstd1, s));
    if (m.flash) {
        FB_TRY(flint_gemm_nt_bias(a.qkv, a.h1, wt.attn_w->half, wt.attn_b->data, rows, 3 * w, w, s));
        FB_CUDA(fb::attention_forward(rows_view(a.attn, 0, w, c.length), static_cast<float*>(a.lse),
                                      rows_view(a.qkv, 0, 3 * w, c.length),
                                      rows_view(a.qkv, w, 3 * w, c.length),
                                      rows_view(a.qkv, 2 * w, 3 * w, c.length),
                                      fb::AttentionShape{c.sequences, c.heads, c.length},
                                      score_scale(hw), s));
    } else {
        FB_TRY(flint_gemm_nt_bias(m.qkv, a.h1, wt.attn_w->half, wt.attn_b->data, rows, 3 * w, w, s));
        void* const parts[] = {a.q, a.k, a.v};
        for (size_t j = 0; j < 3; ++j) {
            FB_TRY(flint_heads_split(parts[j], m.qkv, c.sequences, c.length, c.heads, hw, 3 * w,
                                     j * w, s));
        }
        FB_TRY(flint_gemm_nt_batched(m.scores, a.q, a.k, m.head_batches, c.length, c.length, hw,
                                     score_scale(hw), s));
        FB_TRY(flint_causal_softmax_forward(a.p, m.scores, m.head_batches, c.length, s));
        FB_TRY(flint_gemm_nn_batched(m.heads_out, a.p, a.v, m.head_batches, c.length, hw, c.length,
                                     s));
        FB_TRY(flint_heads_merge(a.attn, m.heads_out, c.sequences, c.length, c.heads, hw, w, 0, s));
    }
    FB_TRY(flint_gemm_nt_bias_residual(a.x_mid, a.attn, wt.proj_w->half, wt.proj_b->data, a.x_in,
                                       rows, w, w, s));
    FB_TRY(layernorm(m, wt.ln2_w, wt.ln2_b, a.x_mid, a.h2, a.mean2, a.rstd2, s));
    FB_TRY(flint_gemm_nt_bias_gelu(a.gelu, a.pre, a.h2, wt.fc_w->half, wt.fc_b->data, rows, 4 * w,
                                   w, s));
    return flint_gemm_nt_bias_residual(a.x_out, a.gelu, wt.fcproj_w->half, wt.fcproj_b->data,
                                       a.x_mid, rows, w, 4 * w, s);
}

void* region_of(const flint_gpt2& m, int region) {
    return static_cast<unsigned char*>(m.column_workspace) + m.column_offsets[region];
}

flint_status weight_gradient(const flint_gpt2& m, const Tensor* weight, const void* dy,
                             const void* input, int accumulate, flint_stream s) {
    return flint_gemm_tn(weight->gradient, dy, input, weight->rows, weight->cols, m.rows,
                         accumulate, m.tn_workspace, m.tn_workspace_bytes, s);
}

// `later` and `region` (which of the block's six partial-sum regions) are used by the model on
// the fused attention kernels, whose second passes run together at the end of the block.
flint_status bias_gradient(const flint_gpt2& m, const Tensor* bias, const void* dy, int accumulate,
                           flint_stream s, fb::ColumnFinishList* later = nullptr, int region = 0) {
    if (m.flash) {
        // The extension model: bandwidth-bound column sums (see fb::launch_bias_gradient).
        void* workspace = later == nullptr ? m.workspace : region_of(m, region);
        FB_CUDA(fb::launch_bias_gradient(bias->gradient, dy, m.rows, bias->cols, accumulate != 0,
                                         workspace, s, true, later));
        return FLINT_OK;
    }
    return flint_bias_gradient(bias->gradient, dy, m.rows, bias->cols, accumulate, m.workspace,
                               m.workspace_bytes, s);
}

// dres (+)= the gradient through a LayerNorm whose output gradient is dh. With
// `half_copy` the kernel also leaves dres rounded to FP16 in dres_half, the operand of
// the GEMMs that follow.
flint_status layernorm_backward(const flint_gpt2& m, const Tensor* gain, const Tensor* bias,
                                const void* x, const void* mean, const void* rstd,
                                int accumulate_dx, int accumulate, bool half_copy, flint_stream s,
                                fb::ColumnFinishList* later = nullptr, int region = 0) {
    void* workspace = later == nullptr ? m.workspace : region_of(m, region);
    FB_CUDA(fb::launch_layernorm_backward(m.dres, gain->gradient, bias->gradient, m.dh, x, mean,
                                          rstd, gain->data, m.rows, m.config.width,
                                          accumulate_dx != 0, accumulate != 0, workspace, s,
                                          half_copy ? m.dres_half : nullptr, m.flash, later));
    return FLINT_OK;
}

// On entry dres is the gradient of the residual stream leaving block i; on
// return, of the stream entering it.
flint_status backward_block(const flint_gpt2& m, size_t i, int accumulate, flint_stream s) {
    const flint_gpt2_config& c = m.config;
    const BlockWeights& wt = m.weights[i];
    const BlockBuffers& a = m.blocks[i];
    const size_t rows = m.rows;
    const size_t w = c.width;
    const size_t hw = m.head_width;
    const size_t hb = m.head_batches;
    const size_t len = c.length;

    // The fused-attention model runs the block's eight column-sum second passes as one launch
    // at the end (the first passes write to six separate regions meanwhile).
    fb::ColumnFinishList finishes;
    fb::ColumnFinishList* later = m.flash ? &finishes : nullptr;

    // MLP. dres_half already holds dres in FP16 (written by the LayerNorm backward before).
    FB_TRY(weight_gradient(m, wt.fcproj_w, m.dres_half, a.gelu, accumulate, s));
    FB_TRY(bias_gradient(m, wt.fcproj_b, m.dres_half, accumulate, s, later, 0));
    FB_TRY(flint_gemm_nn_dgelu(m.dpre, m.dres_half, wt.fcproj_w->half, a.pre, rows, 4 * w, w, s));
    FB_TRY(weight_gradient(m, wt.fc_w, m.dpre, a.h2, accumulate, s));
    FB_TRY(bias_gradient(m, wt.fc_b, m.dpre, accumulate, s, later, 1));
    FB_TRY(flint_gemm_nn(m.dh, m.dpre, wt.fc_w->half, rows, w, 4 * w, s));
    FB_TRY(layernorm_backward(m, wt.ln2_w, wt.ln2_b, a.x_mid, a.mean2, a.rstd2, 1, accumulate, true,
                              s, later, 2));

    // Attention output projection.
    FB_TRY(weight_gradient(m, wt.proj_w, m.dres_half, a.attn, accumulate, s));
    FB_TRY(bias_gradient(m, wt.proj_b, m.dres_half, accumulate, s, later, 3));
    FB_TRY(flint_gemm_nn(m.dh, m.dres_half, wt.proj_w->half, rows, w, w, s));
    if (m.flash) {
        // dO is dh (rows layout), O is the saved attention output, and dQ, dK, dV land
        // directly in the packed qkv gradient rows.
        FB_CUDA(fb::attention_backward(
            rows_view(m.qkv, 0, 3 * w, len), rows_view(m.qkv, w, 3 * w, len),
            rows_view(m.qkv, 2 * w, 3 * w, len), rows_view(m.dh, 0, w, len),
            rows_view(a.attn, 0, w, len), static_cast<const float*>(a.lse),
            static_cast<float*>(m.delta), rows_view(a.qkv, 0, 3 * w, len),
            rows_view(a.qkv, w, 3 * w, len), rows_view(a.qkv, 2 * w, 3 * w, len),
            fb::AttentionShape{c.sequences, c.heads, len}, score_scale(hw), s));
    } else {
        // dO in the heads layout, reusing the forward pass's heads buffer.
        FB_TRY(flint_heads_split(m.heads_out, m.dh, c.sequences, len, c.heads, hw, w, 0, s));
        FB_TRY(flint_gemm_tn_batched(m.dv, a.p, m.heads_out, hb, len, hw, len, s));
        FB_TRY(flint_gemm_nt_batched(m.scores, m.heads_out, a.v, hb, len, len, hw, 1.0f, s));
        FB_TRY(flint_causal_softmax_backward(m.scores, a.p, m.scores, hb, len, score_scale(hw),
                                             s));
        FB_TRY(flint_gemm_nn_batched(m.dq, m.scores, a.k, hb, len, hw, len, s));
        FB_TRY(flint_gemm_tn_batched(m.dk, m.scores, a.q, hb, len, hw, len, s));
        const void* const parts[] = {m.dq, m.dk, m.dv};
        for (size_t j = 0; j < 3; ++j) {
            FB_TRY(flint_heads_merge(m.qkv, parts[j], c.sequences, len, c.heads, hw, 3 * w, j * w,
                                     s));
        }
    }
    FB_TRY(weight_gradient(m, wt.attn_w, m.qkv, a.h1, accumulate, s));
    FB_TRY(bias_gradient(m, wt.attn_b, m.qkv, accumulate, s, later, 4));
    FB_TRY(flint_gemm_nn(m.dh, m.qkv, wt.attn_w->half, rows, w, 3 * w, s));
    // Block 0's result feeds the embedding backward, which reads FP32.
    FB_TRY(layernorm_backward(m, wt.ln1_w, wt.ln1_b, a.x_in, a.mean1, a.rstd1, 1, accumulate, i > 0,
                              s, later, 5));
    FB_CUDA(fb::launch_column_finishes(finishes, rows, s));
    return FLINT_OK;
}

flint_status create(const char* name, const flint_gpt2_config* config, bool flash,
                    flint_gpt2** model) {
    if (model == nullptr) {
        return fb::fail(kInvalid, "%s: model is null", name);
    }
    *model = nullptr;
    FB_TRY(check_config(name, config));
    if (flash && config->width / config->heads != 64) {
        return fb::fail(kInvalid, "%s: flash attention needs heads of width 64, not %zu", name,
                        config->width / config->heads);
    }
    try {
        auto m = std::make_unique<flint_gpt2>();
        m->config = *config;
        m->flash = flash;
        FB_TRY(plan(*m));
        m->host_row_loss.resize(m->rows);
        FB_TRY(allocate(*m));
        link(*m);
        *model = m.release();
    } catch (const std::bad_alloc&) {
        return fb::fail(FLINT_ERROR_CUDA, "%s: out of host memory", name);
    }
    return FLINT_OK;
}

flint_status tensor_info(const char* name, const flint_gpt2* model, size_t index,
                         flint_gpt2_parameter_info* info, bool gradient) {
    if (model == nullptr || info == nullptr) {
        return fb::fail(kInvalid, "%s: model and info must not be null", name);
    }
    if (gradient && model->config.backward == 0) {
        return fb::fail(kInvalid,
                        "%s: the model was created without backward, so it has no gradients",
                        name);
    }
    if (index >= model->tensors.size()) {
        return fb::fail(kInvalid, "%s: index (%zu) must be below %zu", name, index,
                        model->tensors.size());
    }
    const Tensor& t = model->tensors[index];
    *info = {t.name.c_str(), gradient ? t.gradient : t.data, t.rows, t.cols};
    return FLINT_OK;
}

using BucketCallback = void (*)(void* user, int bucket, void* gradients, size_t bytes);

flint_status backward_impl(const char* name, flint_gpt2* model, const void* tokens, int accumulate,
                           flint_stream stream, BucketCallback callback, void* user) {
    if (model == nullptr) {
        return fb::fail(kInvalid, "%s: model is null", name);
    }
    const flint_gpt2& m = *model;
    const flint_gpt2_config& c = m.config;
    if (c.backward == 0) {
        return fb::fail(kInvalid, "%s: the model was created without backward", name);
    }
    if (callback != nullptr && m.gradient_base == nullptr) {
        return fb::fail(kInvalid, "%s: bucket callbacks need a model without separate_buffers",
                        name);
    }
    const size_t rows = m.rows;
    const size_t w = c.width;
    const fb::Span spans[] = {
        {"logits", m.logits, rows * c.padded_vocab * 2},
        {"dlogits", m.dlogits, rows * c.padded_vocab * 2},
        {"row_loss", m.row_loss, rows * 4},
        {"tokens", tokens, rows * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 3));
    for (const Tensor& t : m.tensors) {
        if (fb::overlap(tokens, rows * 2, t.gradient, t.count() * 4)) {
            return fb::fail(kInvalid, "%s: tokens and the gradient of %s overlap", name,
                            t.name.c_str());
        }
    }
    auto notify = [&](int bucket, const Tensor* first, const Tensor* last) {
        if (callback != nullptr) {
            char* begin = static_cast<char*>(first->gradient);
            char* end = static_cast<char*>(last->gradient) + last->count() * 4;
            callback(user, bucket, begin, static_cast<size_t>(end - begin));
        }
    };

    FB_TRY(weight_gradient(m, m.wte, m.dlogits, m.h_f, accumulate, stream));
    FB_TRY(flint_gemm_nn(m.dh, m.dlogits, m.wte->half, rows, w, c.padded_vocab, stream));
    FB_TRY(layernorm_backward(m, m.lnf_w, m.lnf_b, m.x_final, m.mean_f, m.rstd_f, 0, accumulate,
                              true, stream));
    int bucket = 0;
    notify(bucket++, m.lnf_w, m.lnf_b);
    for (size_t i = m.blocks.size(); i-- > 0;) {
        FB_TRY(backward_block(m, i, accumulate, stream));
        notify(bucket++, m.weights[i].ln1_w, m.weights[i].fcproj_b);
    }
    // The tied table: (old + output layer) + embedding, in that order.
    FB_TRY(flint_embedding_backward(m.wte->gradient, m.wpe->gradient, m.dres, tokens, c.sequences,
                                    c.length, c.padded_vocab, w, 1, accumulate, m.workspace,
                                    m.workspace_bytes, stream));
    if (accumulate == 0 && c.block_size > c.length) {
        char* unseen = static_cast<char*>(m.wpe->gradient) + c.length * w * 4;
        FB_CUDA(cudaMemsetAsync(unseen, 0, (c.block_size - c.length) * w * 4, stream));
    }
    notify(bucket++, m.wte, m.wpe);
    return FLINT_OK;
}

using StageCallback = void (*)(void* user, int stage);

flint_status forward_impl(const char* name, flint_gpt2* model, const void* tokens,
                          const void* targets, float scale, flint_stream stream,
                          StageCallback callback, void* user) {
    if (model == nullptr) {
        return fb::fail(kInvalid, "%s: model is null", name);
    }
    if (!std::isfinite(scale)) {
        return fb::fail(kInvalid, "%s: scale (%g) must be finite", name,
                        static_cast<double>(scale));
    }
    const flint_gpt2& m = *model;
    const flint_gpt2_config& c = m.config;
    const size_t rows = m.rows;
    const fb::Span spans[] = {
        {"logits", m.logits, rows * c.padded_vocab * 2},
        {"dlogits", m.dlogits, rows * c.padded_vocab * 2},
        {"row_loss", m.row_loss, rows * 4},
        {"tokens", tokens, rows * 2},
        {"targets", targets, rows * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 3));
    auto enter = [&](int stage) {
        if (callback != nullptr) {
            callback(user, stage);
        }
    };

    enter(0);
    FB_TRY(flint_embedding_forward(m.blocks[0].x_in, tokens, m.wte->data, m.wpe->data, c.sequences,
                                   c.length, c.padded_vocab, c.width, stream));
    for (size_t i = 0; i < m.blocks.size(); ++i) {
        enter(static_cast<int>(i) + 1);
        FB_TRY(forward_block(m, i, stream));
    }
    enter(static_cast<int>(m.blocks.size()) + 1);
    FB_TRY(layernorm(m, m.lnf_w, m.lnf_b, m.x_final, m.h_f, m.mean_f, m.rstd_f, stream));
    FB_TRY(flint_gemm_nt(m.logits, m.h_f, m.wte->half, rows, c.padded_vocab, c.width, stream));
    return flint_softmax_cross_entropy(m.dlogits, m.row_loss, m.logits, targets, scale, rows,
                                       c.vocab, c.padded_vocab, stream);
}

}  // namespace

flint_gpt2::~flint_gpt2() {
    for (void* p : allocations) {
        cudaFree(p);
    }
    cudaGetLastError();
}

extern "C" {

flint_status flint_gpt2_bytes(const flint_gpt2_config* config, size_t* bytes) {
    constexpr const char* name = "flint_gpt2_bytes";
    FB_TRY(check_config(name, config));
    if (bytes == nullptr) {
        return fb::fail(kInvalid, "%s: bytes is null", name);
    }
    try {
        flint_gpt2 m;
        m.config = *config;
        FB_TRY(plan(m));
        *bytes = planned_bytes(m);
    } catch (const std::bad_alloc&) {
        return fb::fail(FLINT_ERROR_CUDA, "%s: out of host memory", name);
    }
    return FLINT_OK;
}

flint_status flint_gpt2_create(const flint_gpt2_config* config, flint_gpt2** model) {
    return create("flint_gpt2_create", config, false, model);
}

flint_status flint_b200_gpt2_create(const flint_gpt2_config* config, int flash_attention,
                                    flint_gpt2** model) {
    return create("flint_b200_gpt2_create", config, flash_attention != 0, model);
}

void flint_gpt2_destroy(flint_gpt2* model) { delete model; }

size_t flint_gpt2_parameter_count(const flint_gpt2* model) {
    return model == nullptr ? 0 : model->tensors.size();
}

flint_status flint_gpt2_parameter(const flint_gpt2* model, size_t index,
                                  flint_gpt2_parameter_info* info) {
    return tensor_info("flint_gpt2_parameter", model, index, info, false);
}

flint_status flint_gpt2_gradient(const flint_gpt2* model, size_t index,
                                 flint_gpt2_parameter_info* info) {
    return tensor_info("flint_gpt2_gradient", model, index, info, true);
}

flint_status flint_gpt2_sync_weights(flint_gpt2* model, flint_stream stream) {
    if (model == nullptr) {
        return fb::fail(kInvalid, "flint_gpt2_sync_weights: model is null");
    }
    for (const Tensor& t : model->tensors) {
        if (t.half != nullptr) {
            FB_TRY(flint_fp32_to_fp16(t.half, t.data, t.count(), stream));
        }
    }
    return FLINT_OK;
}

flint_status flint_gpt2_forward(flint_gpt2* model, const void* tokens, const void* targets,
                                float scale, flint_stream stream) {
    return forward_impl("flint_gpt2_forward", model, tokens, targets, scale, stream, nullptr,
                        nullptr);
}

flint_status flint_b200_gpt2_forward_stages(flint_gpt2* model, const void* tokens,
                                            const void* targets, float scale, flint_stream stream,
                                            flint_b200_stage_callback callback, void* user) {
    return forward_impl("flint_b200_gpt2_forward_stages", model, tokens, targets, scale, stream,
                        callback, user);
}

flint_status flint_gpt2_backward(flint_gpt2* model, const void* tokens, int accumulate,
                                 flint_stream stream) {
    return backward_impl("flint_gpt2_backward", model, tokens, accumulate, stream, nullptr,
                         nullptr);
}

flint_status flint_b200_gpt2_backward_buckets(flint_gpt2* model, const void* tokens,
                                              int accumulate, flint_stream stream,
                                              flint_b200_bucket_callback callback, void* user) {
    return backward_impl("flint_b200_gpt2_backward_buckets", model, tokens, accumulate, stream,
                         callback, user);
}

flint_status flint_b200_gpt2_gradient_arena(const flint_gpt2* model, void** base, size_t* bytes) {
    constexpr const char* name = "flint_b200_gpt2_gradient_arena";
    if (model == nullptr || base == nullptr || bytes == nullptr) {
        return fb::fail(kInvalid, "%s: model, base and bytes must not be null", name);
    }
    if (model->config.backward == 0 || model->gradient_base == nullptr) {
        return fb::fail(kInvalid,
                        "%s: needs a model created with backward and without separate_buffers",
                        name);
    }
    *base = model->gradient_base;
    *bytes = model->gradient_bytes;
    return FLINT_OK;
}

flint_status flint_b200_gpt2_compute_copy(const flint_gpt2* model, size_t index, void** address) {
    constexpr const char* name = "flint_b200_gpt2_compute_copy";
    if (model == nullptr || address == nullptr) {
        return fb::fail(kInvalid, "%s: model and address must not be null", name);
    }
    if (index >= model->tensors.size()) {
        return fb::fail(kInvalid, "%s: index (%zu) must be below %zu", name, index,
                        model->tensors.size());
    }
    *address = model->tensors[index].half;
    return FLINT_OK;
}

flint_status flint_gpt2_outputs(const flint_gpt2* model, const void** logits, const void** dlogits,
                                const void** row_loss) {
    if (model == nullptr) {
        return fb::fail(kInvalid, "flint_gpt2_outputs: model is null");
    }
    if (logits != nullptr) {
        *logits = model->logits;
    }
    if (dlogits != nullptr) {
        *dlogits = model->dlogits;
    }
    if (row_loss != nullptr) {
        *row_loss = model->row_loss;
    }
    return FLINT_OK;
}

flint_status flint_gpt2_mean_loss(flint_gpt2* model, flint_stream stream, double* loss) {
    constexpr const char* name = "flint_gpt2_mean_loss";
    if (model == nullptr || loss == nullptr) {
        return fb::fail(kInvalid, "%s: model and loss must not be null", name);
    }
    std::vector<float>& host = model->host_row_loss;
    FB_CUDA(cudaMemcpyAsync(host.data(), model->row_loss, host.size() * sizeof(float),
                            cudaMemcpyDeviceToHost, stream));
    FB_CUDA(cudaStreamSynchronize(stream));
    double sum = 0.0;
    for (const float v : host) {
        sum += static_cast<double>(v);
    }
    *loss = sum / static_cast<double>(host.size());
    return FLINT_OK;
}

}  // extern "C"
