// Data-movement entry points: flint_copy, flint_fp32_to_fp16, flint_heads_split,
// flint_heads_merge and flint_embedding_forward.
//
// All five are HBM-bound. Each thread moves 16-byte words (two per iteration
// where the layout allows it) and grids are sized to a few CTAs per SM with
// grid-stride loops, so one launch covers any size the ABI allows.
//
// Argument checks and message texts follow the reference's API layer:
// src/api/copy.cpp:7-28, src/api/convert.cpp:8-29, src/api/heads.cpp:12-64,
// src/api/embedding.cpp:10-51.
#include <algorithm>
#include <cstdint>

#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"

namespace {

constexpr int kThreads = 256;
constexpr size_t kMaxRows8 = size_t{0x7fffffff} * 8;  // row limit of the row-wise kernels

// Enough CTAs to fill the GPU a few times over, never more than the work.
unsigned grid_for(size_t items, size_t per_block) {
    int sms = 148;
    fb::sm_count(&sms);
    const size_t wanted = (items + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(sms) * 16;
    return static_cast<unsigned>(std::max<size_t>(1, std::min(wanted, cap)));
}

// ---- copy -------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
    fb_copy_words(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t words) {
    const size_t stride = size_t{gridDim.x} * kThreads;
    size_t i = size_t{blockIdx.x} * kThreads + threadIdx.x;
    // Two independent 16-byte loads in flight per thread.
    for (; i + stride < words; i += 2 * stride) {
        const uint4 a = src[i];
        const uint4 b = src[i + stride];
        dst[i] = a;
        dst[i + stride] = b;
    }
    if (i < words) {
        dst[i] = src[i];
    }
}

__global__ void __launch_bounds__(kThreads)
    fb_copy_bytes(unsigned char* __restrict__ dst, const unsigned char* __restrict__ src,
                  size_t bytes) {
    const size_t stride = size_t{gridDim.x} * kThreads;
    for (size_t i = size_t{blockIdx.x} * kThreads + threadIdx.x; i < bytes; i += stride) {
        dst[i] = src[i];
    }
}

// ---- fp32 -> fp16 -------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
    fb_fp32_to_fp16(__half* __restrict__ y, const float* __restrict__ x, size_t count) {
    const size_t octets = count / 8;
    const size_t stride = size_t{gridDim.x} * kThreads;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint4* y4 = reinterpret_cast<uint4*>(y);
    for (size_t i = size_t{blockIdx.x} * kThreads + threadIdx.x; i < octets; i += stride) {
        const float4 a = x4[2 * i];
        const float4 b = x4[2 * i + 1];
        y4[i] = make_uint4(fb::pack2(a.x, a.y), fb::pack2(a.z, a.w), fb::pack2(b.x, b.y),
                           fb::pack2(b.z, b.w));
    }
    // Up to 7 trailing values.
    const size_t tail = octets * 8;
    if (blockIdx.x == 0 && threadIdx.x < count - tail) {
        y[tail + threadIdx.x] = __float2half_rn(x[tail + threadIdx.x]);
    }
}

// ---- heads split / merge --------------------------------------------------------

// One 16-byte word per (row, head, word-in-head). A CTA takes a run of
// consecutive rows so that the rows-layout side is read or written in long
// contiguous stretches; the 64-bit row -> (batch, t) division happens once per
// CTA.
template <bool kSplit>
__global__ void __launch_bounds__(kThreads)
    fb_heads_move(uint4* __restrict__ y, const uint4* __restrict__ x, size_t rows, size_t length,
                  unsigned heads, unsigned words_per_head, unsigned words_per_row,
                  unsigned first_word, unsigned rows_per_block) {
    const unsigned span = heads * words_per_head;  // words moved per row
    const bool short_length = length < (size_t{1} << 31);
    const unsigned length32 = static_cast<unsigned>(length);
    for (size_t base = size_t{blockIdx.x} * rows_per_block; base < rows;
         base += size_t{gridDim.x} * rows_per_block) {
        const size_t batch0 = base / length;
        const size_t t0 = base - batch0 * length;
        const unsigned here = static_cast<unsigned>(
            rows - base < rows_per_block ? rows - base : rows_per_block);
        const unsigned total = here * span;
        for (unsigned i = threadIdx.x; i < total; i += kThreads) {
            const unsigned r = i / span;
            const unsigned in_row = i - r * span;
            const unsigned h = in_row / words_per_head;
            const unsigned c = in_row - h * words_per_head;
            size_t b = batch0;
            size_t t = t0 + r;
            if (short_length) {
                // t0 < 2^31 and r < 2^12, so 32-bit division is enough.
                const unsigned tt = static_cast<unsigned>(t);
                const unsigned q = tt / length32;
                b += q;
                t = tt - q * length32;
            } else if (t >= length) {
                // A CTA's rows span at most one batch boundary here.
                b += 1;
                t -= length;
            }
            const size_t rows_at = (base + r) * words_per_row + first_word + in_row;
            const size_t heads_at = ((b * heads + h) * length + t) * words_per_head + c;
            if (kSplit) {
                y[heads_at] = x[rows_at];
            } else {
                y[rows_at] = x[heads_at];
            }
        }
    }
}

flint_status move_heads(bool split, void* y, const void* x, size_t batches, size_t length,
                        size_t heads, size_t head_width, size_t row_width, size_t first,
                        flint_stream stream) {
    const char* name = split ? "flint_heads_split" : "flint_heads_merge";
    constexpr size_t kMaxRowWidth = size_t{1} << 24;
    if (row_width == 0 || row_width % 8 != 0 || row_width > kMaxRowWidth) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: row_width (%zu) must be a multiple of 8 from 8 to %zu", name,
                        row_width, kMaxRowWidth);
    }
    if (head_width == 0 || head_width % 8 != 0) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: head_width (%zu) must be a positive multiple of 8", name, head_width);
    }
    if (first % 8 != 0) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: first (%zu) must be a multiple of 8",
                        name, first);
    }
    if (heads == 0) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: heads must be positive", name);
    }
    if (heads > row_width / head_width || first > row_width - heads * head_width) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: %zu heads of %zu columns from column %zu run past row_width (%zu)",
                        name, heads, head_width, first, row_width);
    }
    if (length != 0 && batches > kMaxRows8 / length) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: batches (%zu) x length (%zu) can be up to %zu rows", name, batches,
                        length, kMaxRows8);
    }
    if (batches == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t rows = batches * length;
    const size_t rows_bytes = rows * row_width * 2;
    const size_t heads_bytes = rows * heads * head_width * 2;
    const fb::Span spans[] = {
        {"y", y, split ? heads_bytes : rows_bytes},
        {"x", x, split ? rows_bytes : heads_bytes},
    };
    FB_TRY(fb::check_spans(name, spans, 1));

    const unsigned span = static_cast<unsigned>(heads * head_width / 8);
    // About 2048 words per CTA pass.
    const unsigned rows_per_block = std::max(1u, 2048u / span);
    const unsigned grid = grid_for(rows, rows_per_block);
    auto* yq = static_cast<uint4*>(y);
    const auto* xq = static_cast<const uint4*>(x);
    if (split) {
        fb_heads_move<true><<<grid, kThreads, 0, stream>>>(
            yq, xq, rows, length, static_cast<unsigned>(heads),
            static_cast<unsigned>(head_width / 8), static_cast<unsigned>(row_width / 8),
            static_cast<unsigned>(first / 8), rows_per_block);
    } else {
        fb_heads_move<false><<<grid, kThreads, 0, stream>>>(
            yq, xq, rows, length, static_cast<unsigned>(heads),
            static_cast<unsigned>(head_width / 8), static_cast<unsigned>(row_width / 8),
            static_cast<unsigned>(first / 8), rows_per_block);
    }
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

// ---- embedding forward ------------------------------------------------------------

// A warp per row: lane 0 reads the token, the warp gathers the word row and
// adds the position row, one FP32 add per value.
__global__ void __launch_bounds__(kThreads)
    fb_embedding_forward(float4* __restrict__ x, const uint16_t* __restrict__ tokens,
                         const float4* __restrict__ wte, const float4* __restrict__ wpe,
                         size_t rows, size_t length, unsigned quads) {
    const unsigned lane = threadIdx.x % 32;
    const unsigned warp = threadIdx.x / 32;
    for (size_t row = size_t{blockIdx.x} * (kThreads / 32) + warp; row < rows;
         row += size_t{gridDim.x} * (kThreads / 32)) {
        unsigned token = 0;
        if (lane == 0) {
            token = tokens[row];
        }
        token = __shfl_sync(fb::kFullMask, token, 0);
        const size_t t = row % length;
        const float4* word = wte + size_t{token} * quads;
        const float4* pos = wpe + t * quads;
        float4* out = x + row * quads;
        for (unsigned i = lane; i < quads; i += 32) {
            const float4 a = word[i];
            const float4 b = pos[i];
            out[i] = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z),
                                 __fadd_rn(a.w, b.w));
        }
    }
}

}  // namespace

extern "C" {

flint_status flint_copy(void* dst, const void* src, size_t bytes, flint_stream stream) {
    if (bytes == 0) {
        return FLINT_OK;
    }
    if (dst == nullptr) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "flint_copy: dst is null");
    }
    if (src == nullptr) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "flint_copy: src is null");
    }
    if (!fb::fits(dst, bytes) || !fb::fits(src, bytes)) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "flint_copy: %zu bytes run past the end of the address space", bytes);
    }
    if (fb::overlap(dst, bytes, src, bytes)) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "flint_copy: dst and src overlap");
    }
    auto* d = static_cast<unsigned char*>(dst);
    const auto* s = static_cast<const unsigned char*>(src);
    const uintptr_t da = reinterpret_cast<uintptr_t>(d);
    const uintptr_t sa = reinterpret_cast<uintptr_t>(s);
    if ((da - sa) % 16 != 0) {
        // No common 16-byte phase: byte loads (rare; the harness paths are aligned).
        fb_copy_bytes<<<grid_for(bytes, kThreads), kThreads, 0, stream>>>(d, s, bytes);
        FB_CUDA(fb::after_launch());
        return FLINT_OK;
    }
    // Head up to the first 16-byte boundary, the aligned body, then the tail.
    const size_t head = std::min<size_t>(bytes, (16 - da % 16) % 16);
    const size_t words = (bytes - head) / 16;
    const size_t tail = bytes - head - words * 16;
    if (head > 0) {
        fb_copy_bytes<<<1, 32, 0, stream>>>(d, s, head);
        FB_CUDA(fb::after_launch());
    }
    if (words > 0) {
        fb_copy_words<<<grid_for(words, 2 * kThreads), kThreads, 0, stream>>>(
            reinterpret_cast<uint4*>(d + head), reinterpret_cast<const uint4*>(s + head), words);
        FB_CUDA(fb::after_launch());
    }
    if (tail > 0) {
        fb_copy_bytes<<<1, 32, 0, stream>>>(d + head + words * 16, s + head + words * 16, tail);
        FB_CUDA(fb::after_launch());
    }
    return FLINT_OK;
}

flint_status flint_fp32_to_fp16(void* y, const void* x, size_t count, flint_stream stream) {
    constexpr const char* name = "flint_fp32_to_fp16";
    constexpr size_t kMaxCount = SIZE_MAX / 4;
    if (count > kMaxCount) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: count (%zu) can be up to %zu", name,
                        count, kMaxCount);
    }
    if (count == 0) {
        return FLINT_OK;
    }
    const fb::Span spans[] = {
        {"y", y, count * 2},
        {"x", x, count * 4},
    };
    FB_TRY(fb::check_spans(name, spans, 1));
    fb_fp32_to_fp16<<<grid_for(count / 8 + 1, kThreads), kThreads, 0, stream>>>(
        static_cast<__half*>(y), static_cast<const float*>(x), count);
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_heads_split(void* y, const void* x, size_t batches, size_t length, size_t heads,
                               size_t head_width, size_t row_width, size_t first,
                               flint_stream stream) {
    return move_heads(true, y, x, batches, length, heads, head_width, row_width, first, stream);
}

flint_status flint_heads_merge(void* y, const void* x, size_t batches, size_t length, size_t heads,
                               size_t head_width, size_t row_width, size_t first,
                               flint_stream stream) {
    return move_heads(false, y, x, batches, length, heads, head_width, row_width, first, stream);
}

flint_status flint_embedding_forward(void* x, const void* tokens, const void* wte, const void* wpe,
                                     size_t sequences, size_t length, size_t vocab, size_t width,
                                     flint_stream stream) {
    constexpr const char* name = "flint_embedding_forward";
    constexpr size_t kMaxWidth = size_t{1} << 24;
    constexpr size_t kMaxVocab = size_t{1} << 16;
    if (width == 0 || width % 8 != 0 || width > kMaxWidth) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: width (%zu) must be a multiple of 8 from 8 to %zu", name, width,
                        kMaxWidth);
    }
    if (vocab == 0 || vocab > kMaxVocab) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: vocab (%zu) must be from 1 to %zu",
                        name, vocab, kMaxVocab);
    }
    if (length != 0 && sequences > kMaxRows8 / length) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: sequences (%zu) x length (%zu) can be up to %zu rows", name,
                        sequences, length, kMaxRows8);
    }
    if (sequences == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t rows = sequences * length;
    const fb::Span spans[] = {
        {"x", x, rows * width * 4},
        {"tokens", tokens, rows * 2},
        {"wte", wte, vocab * width * 4},
        {"wpe", wpe, length * width * 4},
    };
    FB_TRY(fb::check_spans(name, spans, 1));
    fb_embedding_forward<<<grid_for(rows, kThreads / 32), kThreads, 0, stream>>>(
        static_cast<float4*>(x), static_cast<const uint16_t*>(tokens),
        static_cast<const float4*>(wte), static_cast<const float4*>(wpe), rows, length,
        static_cast<unsigned>(width / 4));
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

}  // extern "C"
