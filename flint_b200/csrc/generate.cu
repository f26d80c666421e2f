// Autoregressive decoding for a GPT-2 model's weights: a KV cache, single-query
// (decode) attention, and weight-only int8 linear layers (extension; the reference
// lists this as its inference milestone in README.md:148 and has no code for it).
// The oracle is the reference's PyTorch model run on the whole sequence
// (scripts/gpt2_torch.py:52-131): the logits at each position must agree.
//
// Two regimes:
//   prefill   the prompt's rows go through the library's tensor-core GEMMs and the
//             fused causal attention kernel, exactly as in the training forward pass,
//             and their keys and values are copied into the cache
//   decode    one new token per sequence. The step is bound by HBM traffic: every
//             weight is read once per step (2 bytes each in FP16, 1 in int8) and the
//             cache of every layer once; the linear layers for up to eight sequences
//             run on a streaming kernel (a warp per one or two output features, 16-byte
//             weight loads past L1, the eight rows' activations through L1, FP32
//             accumulation), more sequences use the tensor-core GEMMs.
//             Positions live in device memory, so a step's launches do not change from
//             token to token and are captured once into a CUDA graph.
//
// Cache layout: [layer][K or V][sequence][head][position][64] FP16. A position's key is
// 128 contiguous bytes and a head's positions are contiguous, so decode attention
// reads whole cache lines in order.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <memory>
#include <new>
#include <vector>

#include <cuda_fp16.h>

#include "attention.h"
#include "common.h"
#include "device_utils.cuh"
#include "flint/flint_b200.h"
#include "gemm.h"
#include "gpt2.h"

namespace {

constexpr flint_status kInvalid = FLINT_ERROR_INVALID_ARGUMENT;
constexpr int kHeadWidth = 64;
constexpr int kSkinnyRows = 8;       // sequences the streaming linear kernel serves at once
constexpr int kLinearWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kEps = 1e-5f;

enum class Act { kNone, kGelu, kResidual, kLogits };

struct Matrix {
    const __half* half = nullptr;   // [n, k] FP16 (the model's compute copy)
    int8_t* q = nullptr;            // [n, k] int8 (generator-owned) or null
    float* scale = nullptr;         // [n] FP32: w[n, :] ~ q[n, :] * scale[n]
    const float* bias = nullptr;    // [n] FP32 or null
    size_t n = 0, k = 0;
};

struct Layer {
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    Matrix attn, proj, fc, fcproj;
};

__device__ __forceinline__ float gelu_tanh(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
}

// ---- per-row int8 quantisation -----------------------------------------------------------------

// One warp per row: scale = max|w| / 127, q = round(w / scale).
__global__ void __launch_bounds__(256)
    fb_quantize_rows(int8_t* __restrict__ q, float* __restrict__ scale,
                     const __half* __restrict__ w, size_t rows, size_t cols) {
    const size_t row = blockIdx.x * 8ull + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= rows) {
        return;
    }
    const __half* src = w + row * cols;
    float top = 0.0f;
    for (size_t c = lane; c < cols; c += 32) {
        top = fmaxf(top, fabsf(__half2float(src[c])));
    }
    top = fb::warp_max(top);
    const float s = top > 0.0f ? top / 127.0f : 1.0f;
    const float inv = 1.0f / s;
    for (size_t c = lane; c < cols; c += 32) {
        const float v = rintf(__half2float(src[c]) * inv);
        q[row * cols + c] = static_cast<int8_t>(fminf(fmaxf(v, -127.0f), 127.0f));
    }
    if (lane == 0) {
        scale[row] = s;
    }
}

// int8 rows back to FP16 (prefill and many-sequence steps run on the tensor cores).
__global__ void __launch_bounds__(256)
    fb_dequantize_rows(__half* __restrict__ w, const int8_t* __restrict__ q,
                       const float* __restrict__ scale, size_t rows, size_t cols) {
    const size_t total = rows * cols;
    for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        w[i] = __float2half_rn(static_cast<float>(q[i]) * scale[i / cols]);
    }
}

// ---- the streaming linear layer for up to eight rows ---------------------------------------------
//
// y[b, n] = act(sum_k x[b, k] w[n, k] (* scale[n]) + bias[n]) for eight rows b. A warp owns F
// output features (1 for narrow outputs, so that enough warps exist to keep HBM busy; 2
// otherwise, halving the activations' L1 traffic per weight byte). In one step a lane takes
// 16 bytes of each feature's weights (8 FP16 or 16 int8 values: a warp reads 512 contiguous
// bytes of a weight row) and the matching activations of all eight rows, which come through
// L1: the eight rows are at most 48 KB and every warp of the SM reads the same ones. The
// weights are touched once, so they are loaded past L1. FP32 accumulation; the lanes' sums
// are added by a butterfly at the end.

template <typename W>
struct WeightVector;

template <>
struct WeightVector<__half> {
    static constexpr int kValues = 8;
    static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[8]) {
        fb::unpack8(v, raw);
    }
};

template <>
struct WeightVector<int8_t> {
    static constexpr int kValues = 16;
    static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[16]) {
        const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int word = static_cast<int>(words[i]);
            v[4 * i] = static_cast<float>(static_cast<int8_t>(word));
            v[4 * i + 1] = static_cast<float>(static_cast<int8_t>(word >> 8));
            v[4 * i + 2] = static_cast<float>(static_cast<int8_t>(word >> 16));
            v[4 * i + 3] = static_cast<float>(word >> 24);
        }
    }
};

// 16 bytes that will not be read again: bypass L1.
__device__ __forceinline__ uint4 load_streaming(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// S warps share a feature group: S = 1 gives every warp of the CTA its own F features; S = 4
// gives the CTA's four warps a quarter of k each for the same F features (their sums meet
// in shared memory and are added in warp order), which multiplies the warps, and the bytes
// in flight, for narrow outputs whose few features would otherwise leave most SMs idle.
template <typename W, Act A, int F, int S>
__global__ void __launch_bounds__(32 * kLinearWarps)
    fb_decode_linear(void* __restrict__ out, const W* __restrict__ w,
                     const float* __restrict__ scale, const float* __restrict__ bias,
                     const __half* __restrict__ x, const float* __restrict__ residual, int n,
                     int k, int out_stride) {
    constexpr int kValues = WeightVector<W>::kValues;
    constexpr int kRows = kSkinnyRows;
    constexpr int kGroups = kLinearWarps / S;          // feature groups per CTA
    static_assert(S == 1 || S == kLinearWarps, "a feature group is one warp or the whole CTA");
    __shared__ float meet[S == 1 ? 1 : kLinearWarps][F][kRows];
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int first = (blockIdx.x * kGroups + (S == 1 ? warp : 0)) * F;
    if (S == 1 && first >= n) {
        return;
    }
    // This warp's share of k, in whole lane-steps.
    const int steps = (k + 32 * kValues - 1) / (32 * kValues);
    const int share = (steps + S - 1) / S;
    const int k_begin = (S == 1 ? 0 : warp * share) * 32 * kValues;
    const int k_end = min(k, (S == 1 ? steps : (warp + 1) * share) * 32 * kValues);
    float acc[F][kRows];
#pragma unroll
    for (int f = 0; f < F; ++f) {
#pragma unroll
        for (int b = 0; b < kRows; ++b) {
            acc[f][b] = 0.0f;
        }
    }
#pragma unroll 2
    for (int k0 = k_begin + lane * kValues; k0 < k_end; k0 += 32 * kValues) {
        uint4 raw[F];
#pragma unroll
        for (int f = 0; f < F; ++f) {
            const int feature = min(first + f, n - 1);
            raw[f] = load_streaming(w + static_cast<size_t>(feature) * k + k0);
        }
        float wv[F][kValues];
#pragma unroll
        for (int f = 0; f < F; ++f) {
            WeightVector<W>::unpack(raw[f], wv[f]);
        }
#pragma unroll
        for (int b = 0; b < kRows; ++b) {
            const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<size_t>(b) * k + k0);
#pragma unroll
            for (int piece = 0; piece < kValues / 8; ++piece) {
                float xv[8];
                fb::unpack8(xv, __ldg(row + piece));
#pragma unroll
                for (int f = 0; f < F; ++f) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[f][b] = fmaf(wv[f][8 * piece + j], xv[j], acc[f][b]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int f = 0; f < F; ++f) {
#pragma unroll
        for (int b = 0; b < kRows; ++b) {
            acc[f][b] = fb::warp_sum_rn(acc[f][b]);
        }
    }
    // Lane (f, b) holds output (b, first + f).
    const int f = lane / kRows;
    const int b = lane % kRows;
    float v = 0.0f;
#pragma unroll
    for (int ff = 0; ff < F; ++ff) {
#pragma unroll
        for (int bb = 0; bb < kRows; ++bb) {
            v = (ff == f && bb == b) ? acc[ff][bb] : v;
        }
    }
    if constexpr (S > 1) {
        if (lane < F * kRows) {
            meet[warp][f][b] = v;
        }
        __syncthreads();
        if (warp != 0) {
            return;
        }
        if (lane < F * kRows) {
            v = meet[0][f][b];
#pragma unroll
            for (int other = 1; other < S; ++other) {
                v += meet[other][f][b];
            }
        }
    }
    if (lane < F * kRows && first + f < n) {
        const int feature = first + f;
        if (scale != nullptr) {
            v *= scale[feature];
        }
        if (bias != nullptr) {
            v += bias[feature];
        }
        const size_t at = static_cast<size_t>(b) * out_stride + feature;
        if constexpr (A == Act::kResidual) {
            static_cast<float*>(out)[at] = residual[at] + v;
        } else if constexpr (A == Act::kLogits) {
            static_cast<float*>(out)[at] = v;
        } else if constexpr (A == Act::kGelu) {
            static_cast<__half*>(out)[at] = __float2half_rn(gelu_tanh(v));
        } else {
            static_cast<__half*>(out)[at] = __float2half_rn(v);
        }
    }
}

// ---- decode-side element kernels ------------------------------------------------------------------

// x[b, :] = wte[tokens[b], :] + wpe[position, :] for one new token per sequence.
__global__ void __launch_bounds__(256)
    fb_decode_embed(float* __restrict__ x, const uint16_t* __restrict__ tokens,
                    const float* __restrict__ wte, const float* __restrict__ wpe,
                    const int* __restrict__ position, int width, int vocab_rows) {
    const int b = blockIdx.x;
    const int token = min(static_cast<int>(tokens[b]), vocab_rows - 1);
    const int pos = *position;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        x[static_cast<size_t>(b) * width + c] =
            wte[static_cast<size_t>(token) * width + c] + wpe[static_cast<size_t>(pos) * width + c];
    }
}

// Copies the keys and values of `count` consecutive positions per sequence from packed qkv
// rows [sequences * count, 3 width] into the cache, starting at cache position *position
// (decode: count 1) or `first` when position is null (prefill).
__global__ void __launch_bounds__(256)
    fb_cache_store(__half* __restrict__ cache_k, __half* __restrict__ cache_v,
                   const __half* __restrict__ qkv, const int* __restrict__ position, int first,
                   int count, int heads, int max_length) {
    const int width = heads * kHeadWidth;
    const int row = blockIdx.x;            // sequence * count + offset
    const int sequence = row / count;
    const int t = (position != nullptr ? *position : first) + row % count;
    const uint4* src = reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(row) * 3 * width);
    const int pieces = width / 8;          // 16-byte pieces per K (or V) row
    for (int i = threadIdx.x; i < 2 * pieces; i += blockDim.x) {
        const int which = i / pieces;      // 0: K, 1: V
        const int piece = i % pieces;
        const int head = piece / (kHeadWidth / 8);
        const int inner = piece % (kHeadWidth / 8);
        __half* dst = (which == 0 ? cache_k : cache_v) +
                      ((static_cast<size_t>(sequence) * heads + head) * max_length + t) * kHeadWidth;
        reinterpret_cast<uint4*>(dst)[inner] = src[(1 + which) * pieces + piece];
    }
}

// One query per (sequence, head) against the cache's positions 0 .. *position. The new
// token's own key and value come straight from its qkv row; the CTA also stores them in the
// cache for the steps to come (no other CTA reads that position during this launch).
constexpr int kDecodeThreads = 512;

__global__ void __launch_bounds__(kDecodeThreads)
    fb_decode_attention(__half* __restrict__ out, const __half* __restrict__ qkv,
                        __half* __restrict__ cache_k, __half* __restrict__ cache_v,
                        const int* __restrict__ position, int heads, int max_length, float scale) {
    extern __shared__ float scores[];      // [max_length]
    constexpr int kGroups = kDecodeThreads / 8;
    __shared__ float q[kHeadWidth];
    __shared__ float red[kDecodeThreads / 32];
    __shared__ float partial[kGroups][kHeadWidth];
    const int head = blockIdx.x % heads;
    const int sequence = blockIdx.x / heads;
    const int width = heads * kHeadWidth;
    const int newest = *position;
    const int length = newest + 1;
    const int tid = threadIdx.x;
    const int lane = tid % 32;
    const int warp = tid / 32;
    const __half* row_q = qkv + static_cast<size_t>(sequence) * 3 * width + head * kHeadWidth;
    const __half* new_k = row_q + width;
    const __half* new_v = row_q + 2 * width;
    __half* keys = cache_k + (static_cast<size_t>(sequence) * heads + head) * max_length * kHeadWidth;
    __half* values = cache_v + (static_cast<size_t>(sequence) * heads + head) * max_length * kHeadWidth;
    if (tid < kHeadWidth) {
        q[tid] = __half2float(row_q[tid]) * scale * kLog2e;
    } else if (tid < kHeadWidth + 8) {
        const int piece = tid - kHeadWidth;
        reinterpret_cast<uint4*>(keys + static_cast<size_t>(newest) * kHeadWidth)[piece] =
            reinterpret_cast<const uint4*>(new_k)[piece];
    } else if (tid < kHeadWidth + 16) {
        const int piece = tid - kHeadWidth - 8;
        reinterpret_cast<uint4*>(values + static_cast<size_t>(newest) * kHeadWidth)[piece] =
            reinterpret_cast<const uint4*>(new_v)[piece];
    }
    __syncthreads();
    float top = -INFINITY;
    for (int t = tid; t < length; t += kDecodeThreads) {
        const uint4* row = reinterpret_cast<const uint4*>(
            t == newest ? new_k : keys + static_cast<size_t>(t) * kHeadWidth);
        uint4 raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            raw[i] = load_streaming(row + i);
        }
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float v[8];
            fb::unpack8(v, raw[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s = fmaf(v[j], q[8 * i + j], s);
            }
        }
        scores[t] = s;
        top = fmaxf(top, s);
    }
    top = fb::warp_max(top);
    if (lane == 0) {
        red[warp] = top;
    }
    __syncthreads();
    top = red[0];
#pragma unroll
    for (int i = 1; i < kDecodeThreads / 32; ++i) {
        top = fmaxf(top, red[i]);
    }
    __syncthreads();
    float sum = 0.0f;
    for (int t = tid; t < length; t += kDecodeThreads) {
        const float p = exp2f(scores[t] - top);
        scores[t] = p;
        sum += p;
    }
    sum = fb::warp_sum_rn(sum);
    if (lane == 0) {
        red[warp] = sum;
    }
    __syncthreads();
    sum = red[0];
#pragma unroll
    for (int i = 1; i < kDecodeThreads / 32; ++i) {
        sum += red[i];
    }
    // Thread (group, piece): positions group, group + 64, ...; eight output columns.
    const int piece = tid % 8;
    const int group = tid / 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 8
    for (int t = group; t < length; t += kGroups) {
        const __half* row = t == newest ? new_v : values + static_cast<size_t>(t) * kHeadWidth;
        const uint4 raw = load_streaming(reinterpret_cast<const uint4*>(row) + piece);
        float v[8];
        fb::unpack8(v, raw);
        const float p = scores[t];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[j] = fmaf(p, v[j], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        partial[group][piece * 8 + j] = acc[j];
    }
    __syncthreads();
    if (tid < kHeadWidth) {
        float total = 0.0f;
#pragma unroll 8
        for (int g2 = 0; g2 < kGroups; ++g2) {
            total += partial[g2][tid];
        }
        out[static_cast<size_t>(sequence) * width + head * kHeadWidth + tid] =
            __float2half_rn(total / sum);
    }
}

// The last position's row of each sequence: [sequences * length, width] -> [sequences, width].
__global__ void __launch_bounds__(256)
    fb_take_last_rows(float* __restrict__ out, const float* __restrict__ x, int length, int width) {
    const int b = blockIdx.x;
    const float* src = x + (static_cast<size_t>(b) * length + length - 1) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        out[static_cast<size_t>(b) * width + c] = src[c];
    }
}

// Greedy choice: the lowest index of the largest logit below `vocab`.
__global__ void __launch_bounds__(256)
    fb_argmax_rows(uint16_t* __restrict__ next, const float* __restrict__ logits, int vocab,
                   int stride) {
    __shared__ float best_value[8];
    __shared__ int best_index[8];
    const float* row = logits + static_cast<size_t>(blockIdx.x) * stride;
    float value = -INFINITY;
    int index = 0;
    for (int c = threadIdx.x; c < vocab; c += 256) {
        const float v = row[c];
        if (v > value) {
            value = v;
            index = c;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(fb::kFullMask, value, off);
        const int oi = __shfl_xor_sync(fb::kFullMask, index, off);
        if (ov > value || (ov == value && oi < index)) {
            value = ov;
            index = oi;
        }
    }
    if (threadIdx.x % 32 == 0) {
        best_value[threadIdx.x / 32] = value;
        best_index[threadIdx.x / 32] = index;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w2 = 1; w2 < 8; ++w2) {
            if (best_value[w2] > value || (best_value[w2] == value && best_index[w2] < index)) {
                value = best_value[w2];
                index = best_index[w2];
            }
        }
        next[blockIdx.x] = static_cast<uint16_t>(index);
    }
}

__global__ void fb_advance_position(int* position, int by) { *position += by; }

}  // namespace

struct flint_b200_generator {
    const flint_gpt2* model = nullptr;
    size_t sequences = 0, max_length = 0;
    size_t layers = 0, heads = 0, width = 0, vocab = 0, padded_vocab = 0;
    bool int8 = false;
    std::vector<Layer> blocks;
    Matrix head;                       // the tied output layer (wte)
    const float *wte = nullptr, *wpe = nullptr, *lnf_w = nullptr, *lnf_b = nullptr;
    size_t host_position = 0;          // tokens held per sequence (mirror of *position)
    // device
    int* position = nullptr;
    __half* cache = nullptr;           // [layers][2][sequences][heads][max_length][64]
    float *x_a = nullptr, *x_b = nullptr, *last = nullptr;
    __half *h = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *pre = nullptr;
    float *mean = nullptr, *rstd = nullptr, *lse = nullptr, *logits = nullptr;
    uint16_t* next = nullptr;
    __half* dequantized = nullptr;     // int8: FP16 scratch for one matrix
    std::vector<void*> owned;
    cudaGraphExec_t step_graph = nullptr;
    const void* graph_tokens = nullptr;
    void* graph_next = nullptr;

    ~flint_b200_generator() {
        if (step_graph != nullptr) {
            cudaGraphExecDestroy(step_graph);
        }
        for (void* p : owned) {
            cudaFree(p);
        }
        cudaGetLastError();
    }
    size_t cache_stride() const { return sequences * heads * max_length * kHeadWidth; }
    __half* keys(size_t layer) const { return cache + (2 * layer) * cache_stride(); }
    __half* values(size_t layer) const { return cache + (2 * layer + 1) * cache_stride(); }
};

namespace {

template <typename T>
flint_status allocate(flint_b200_generator& g, T** out, size_t count) {
    void* p = nullptr;
    FB_CUDA(cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
    g.owned.push_back(p);
    *out = static_cast<T*>(p);
    return FLINT_OK;
}

Matrix matrix_of(const fb::Tensor* weight, const fb::Tensor* bias) {
    Matrix m;
    m.half = static_cast<const __half*>(weight->half);
    m.bias = bias == nullptr ? nullptr : static_cast<const float*>(bias->data);
    m.n = weight->rows;
    m.k = weight->cols;
    return m;
}

flint_status quantize(flint_b200_generator& g, Matrix& m, cudaStream_t stream) {
    if (m.q == nullptr) {
        FB_TRY(allocate(g, &m.q, m.n * m.k));
        FB_TRY(allocate(g, &m.scale, m.n));
    }
    fb_quantize_rows<<<static_cast<unsigned>((m.n + 7) / 8), 256, 0, stream>>>(m.q, m.scale, m.half,
                                                                                m.n, m.k);
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

template <typename W, Act A, int F, int S>
flint_status launch_skinny(void* out, const W* w, const float* scale, const float* bias,
                           const __half* x, const float* residual, size_t n, size_t k,
                           size_t out_stride, cudaStream_t stream) {
    const size_t per_cta = static_cast<size_t>(kLinearWarps / S) * F;
    const unsigned grid = static_cast<unsigned>((n + per_cta - 1) / per_cta);
    fb_decode_linear<W, A, F, S><<<grid, 32 * kLinearWarps, 0, stream>>>(
        out, w, scale, bias, x, residual, static_cast<int>(n), static_cast<int>(k),
        static_cast<int>(out_stride));
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

// Eight rows at `x` (spare rows of the caller's buffers are scratch when fewer are live).
template <Act A>
flint_status skinny(const flint_b200_generator& g, const Matrix& m, void* out, const __half* x,
                    const float* residual, size_t out_stride, cudaStream_t stream) {
    // Narrow outputs: two features per CTA with k split over its four warps (as many CTAs as
    // a wide output has). Wide outputs: two features per warp.
    const bool narrow = m.n <= 1024;
    if (g.int8) {
        return narrow ? launch_skinny<int8_t, A, 2, kLinearWarps>(out, m.q, m.scale, m.bias, x, residual,
                                                                  m.n, m.k, out_stride, stream)
                      : launch_skinny<int8_t, A, 2, 1>(out, m.q, m.scale, m.bias, x, residual, m.n, m.k,
                                                       out_stride, stream);
    }
    return narrow ? launch_skinny<__half, A, 2, kLinearWarps>(out, m.half, nullptr, m.bias, x, residual,
                                                              m.n, m.k, out_stride, stream)
                  : launch_skinny<__half, A, 2, 1>(out, m.half, nullptr, m.bias, x, residual, m.n, m.k,
                                                   out_stride, stream);
}

// The FP16 weights the tensor-core GEMMs read: the model's copy, or the int8 weights
// expanded into the scratch matrix.
flint_status dense_weights(const flint_b200_generator& g, const Matrix& m, const __half** w,
                           cudaStream_t stream) {
    if (!g.int8) {
        *w = m.half;
        return FLINT_OK;
    }
    fb_dequantize_rows<<<1184, 256, 0, stream>>>(g.dequantized, m.q, m.scale, m.n, m.k);
    FB_CUDA(fb::after_launch());
    *w = g.dequantized;
    return FLINT_OK;
}

// y = act(x w^T + bias) for `rows` rows. kNone/kGelu: FP16 out; kResidual: FP32 out =
// residual + (x w^T + bias). (The output layer always takes the streaming kernel.)
template <Act A>
flint_status linear(const flint_b200_generator& g, const Matrix& m, void* out, const __half* x,
                    const float* residual, size_t rows, bool decode, cudaStream_t stream) {
    static_assert(A != Act::kLogits, "the output layer does not come through here");
    if (decode && rows <= kSkinnyRows) {
        return skinny<A>(g, m, out, x, residual, m.n, stream);
    }
    if (decode && g.int8) {
        // More than eight sequences on int8 weights: groups of eight through the streaming
        // kernel (the weights are re-read per group; the tensor cores take FP16 only).
        for (size_t first = 0; first < rows; first += kSkinnyRows) {
            const size_t stride = m.n;
            const size_t bytes = A == Act::kResidual ? 4 : 2;
            FB_TRY(skinny<A>(g, m, static_cast<char*>(out) + first * stride * bytes,
                             x + first * m.k, residual == nullptr ? nullptr : residual + first * m.n,
                             stride, stream));
        }
        return FLINT_OK;
    }
    const __half* w = nullptr;
    FB_TRY(dense_weights(g, m, &w, stream));
    if constexpr (A == Act::kNone) {
        FB_CUDA(fb::gemm_nt(fb::Epilogue::kBias, out, nullptr, x, w, m.bias, nullptr, rows, m.n, m.k,
                            stream));
    } else if constexpr (A == Act::kGelu) {
        FB_CUDA(fb::gemm_nt(fb::Epilogue::kBiasGelu, out, g.pre, x, w, m.bias, nullptr, rows, m.n,
                            m.k, stream));
    } else {
        FB_CUDA(fb::gemm_nt(fb::Epilogue::kBiasResidual, out, nullptr, x, w, m.bias, residual, rows,
                            m.n, m.k, stream));
    }
    return FLINT_OK;
}

flint_status layernorm(const flint_b200_generator& g, const float* gain, const float* bias,
                       const float* x, size_t rows, cudaStream_t stream) {
    return flint_layernorm_forward(g.h, g.mean, g.rstd, x, gain, bias, rows, g.width, kEps, stream);
}

// The transformer over `rows` = sequences * count rows. decode: count == 1 and attention
// runs against the cache; otherwise the fused causal kernel runs over the prompt.
flint_status run_blocks(flint_b200_generator& g, size_t count, bool decode, cudaStream_t stream) {
    const size_t rows = g.sequences * count;
    float* x = g.x_a;
    float* other = g.x_b;
    const float scale = 1.0f / std::sqrt(static_cast<float>(kHeadWidth));
    for (size_t i = 0; i < g.layers; ++i) {
        const Layer& l = g.blocks[i];
        FB_TRY(layernorm(g, l.ln1_w, l.ln1_b, x, rows, stream));
        FB_TRY(linear<Act::kNone>(g, l.attn, g.qkv, g.h, nullptr, rows, decode, stream));
        if (decode) {
            // (The kernel also stores the new token's key and value in the cache.)
            const int smem = static_cast<int>(g.max_length * sizeof(float));
            fb_decode_attention<<<static_cast<unsigned>(g.sequences * g.heads), kDecodeThreads, smem,
                                  stream>>>(
                g.attn, g.qkv, g.keys(i), g.values(i), g.position, static_cast<int>(g.heads),
                static_cast<int>(g.max_length), scale);
            FB_CUDA(fb::after_launch());
        } else {
            fb_cache_store<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
                g.keys(i), g.values(i), g.qkv, nullptr, static_cast<int>(g.host_position),
                static_cast<int>(count), static_cast<int>(g.heads), static_cast<int>(g.max_length));
            FB_CUDA(fb::after_launch());
            const size_t w3 = 3 * g.width;
            auto view = [&](const void* base, size_t first, size_t row_width) {
                return fb::AttentionView{static_cast<const __half*>(base) + first,
                                         static_cast<long long>(row_width), kHeadWidth,
                                         static_cast<long long>(count * row_width)};
            };
            FB_CUDA(fb::attention_forward(view(g.attn, 0, g.width), g.lse, view(g.qkv, 0, w3),
                                          view(g.qkv, g.width, w3), view(g.qkv, 2 * g.width, w3),
                                          fb::AttentionShape{g.sequences, g.heads, count}, scale,
                                          stream));
        }
        FB_TRY(linear<Act::kResidual>(g, l.proj, other, g.attn, x, rows, decode, stream));
        std::swap(x, other);
        FB_TRY(layernorm(g, l.ln2_w, l.ln2_b, x, rows, stream));
        FB_TRY(linear<Act::kGelu>(g, l.fc, g.act, g.h, nullptr, rows, decode, stream));
        FB_TRY(linear<Act::kResidual>(g, l.fcproj, other, g.act, x, rows, decode, stream));
        std::swap(x, other);
    }
    if (x != g.x_a) {
        // An even number of swaps per block keeps the stream in x_a; this is a safeguard.
        FB_CUDA(cudaMemcpyAsync(g.x_a, x, rows * g.width * 4, cudaMemcpyDeviceToDevice, stream));
    }
    return FLINT_OK;
}

// Final LayerNorm + output layer over the `sequences` rows at `x`, then the greedy choice.
flint_status run_head(flint_b200_generator& g, const float* x, void* next_tokens,
                      cudaStream_t stream) {
    FB_TRY(layernorm(g, g.lnf_w, g.lnf_b, x, g.sequences, stream));
    // Groups of eight rows through the streaming kernel: FP32 logits straight from the sums.
    for (size_t first = 0; first < g.sequences; first += kSkinnyRows) {
        FB_TRY(skinny<Act::kLogits>(g, g.head, g.logits + first * g.padded_vocab, g.h + first * g.width,
                                    nullptr, g.padded_vocab, stream));
    }
    uint16_t* next = next_tokens != nullptr ? static_cast<uint16_t*>(next_tokens) : g.next;
    fb_argmax_rows<<<static_cast<unsigned>(g.sequences), 256, 0, stream>>>(
        next, g.logits, static_cast<int>(g.vocab), static_cast<int>(g.padded_vocab));
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status enqueue_step(flint_b200_generator& g, const void* tokens, void* next_tokens,
                          cudaStream_t stream) {
    fb_decode_embed<<<static_cast<unsigned>(g.sequences), 256, 0, stream>>>(
        g.x_a, static_cast<const uint16_t*>(tokens), g.wte, g.wpe, g.position,
        static_cast<int>(g.width), static_cast<int>(g.padded_vocab));
    FB_CUDA(fb::after_launch());
    FB_TRY(run_blocks(g, 1, true, stream));
    FB_TRY(run_head(g, g.x_a, next_tokens, stream));
    fb_advance_position<<<1, 1, 0, stream>>>(g.position, 1);
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status build(flint_b200_generator& g, cudaStream_t stream) {
    const flint_gpt2& m = *g.model;
    const flint_gpt2_config& c = m.config;
    g.layers = c.layers;
    g.heads = c.heads;
    g.width = c.width;
    g.vocab = c.vocab;
    g.padded_vocab = c.padded_vocab;
    g.wte = static_cast<const float*>(m.wte->data);
    g.wpe = static_cast<const float*>(m.wpe->data);
    g.lnf_w = static_cast<const float*>(m.lnf_w->data);
    g.lnf_b = static_cast<const float*>(m.lnf_b->data);
    g.head = matrix_of(m.wte, nullptr);
    for (size_t i = 0; i < c.layers; ++i) {
        const fb::BlockWeights& w = m.weights[i];
        Layer l;
        l.ln1_w = static_cast<const float*>(w.ln1_w->data);
        l.ln1_b = static_cast<const float*>(w.ln1_b->data);
        l.ln2_w = static_cast<const float*>(w.ln2_w->data);
        l.ln2_b = static_cast<const float*>(w.ln2_b->data);
        l.attn = matrix_of(w.attn_w, w.attn_b);
        l.proj = matrix_of(w.proj_w, w.proj_b);
        l.fc = matrix_of(w.fc_w, w.fc_b);
        l.fcproj = matrix_of(w.fcproj_w, w.fcproj_b);
        g.blocks.push_back(l);
    }
    // The streaming kernel always computes groups of eight rows: every buffer holds whole groups.
    const size_t groups = (g.sequences + kSkinnyRows - 1) / kSkinnyRows * kSkinnyRows;
    const size_t rows = std::max<size_t>(g.sequences * g.max_length, groups);
    const size_t w = g.width;
    FB_TRY(allocate(g, &g.position, 4));
    FB_CUDA(cudaMemsetAsync(g.position, 0, 16, stream));
    FB_TRY(allocate(g, &g.cache, 2 * g.layers * g.cache_stride()));
    FB_TRY(allocate(g, &g.x_a, rows * w));
    FB_TRY(allocate(g, &g.x_b, rows * w));
    FB_TRY(allocate(g, &g.last, groups * w));
    FB_TRY(allocate(g, &g.h, rows * w));
    FB_TRY(allocate(g, &g.qkv, rows * 3 * w));
    FB_TRY(allocate(g, &g.attn, rows * w));
    FB_TRY(allocate(g, &g.act, rows * 4 * w));
    FB_TRY(allocate(g, &g.pre, rows * 4 * w));
    FB_TRY(allocate(g, &g.mean, rows));
    FB_TRY(allocate(g, &g.rstd, rows));
    FB_TRY(allocate(g, &g.lse, g.sequences * g.heads * g.max_length));
    FB_TRY(allocate(g, &g.logits, groups * g.padded_vocab));
    FB_TRY(allocate(g, &g.next, groups));
    FB_CUDA(cudaMemsetAsync(g.last, 0, groups * w * 4, stream));
    // Spare rows of the small buffers are read by the streaming kernel: keep them finite.
    FB_CUDA(cudaMemsetAsync(g.h, 0, rows * w * 2, stream));
    FB_CUDA(cudaMemsetAsync(g.attn, 0, rows * w * 2, stream));
    FB_CUDA(cudaMemsetAsync(g.act, 0, rows * 4 * w * 2, stream));
    FB_CUDA(cudaMemsetAsync(g.x_a, 0, rows * w * 4, stream));
    FB_CUDA(cudaMemsetAsync(g.x_b, 0, rows * w * 4, stream));
    if (g.int8) {
        // Holds one matrix at a time: the largest of the output layer and the MLP's.
        FB_TRY(allocate(g, &g.dequantized, std::max(g.padded_vocab * w, 4 * w * w)));
    }
    return FLINT_OK;
}

}  // namespace

extern "C" {

flint_status flint_b200_generator_create(const flint_gpt2* model, size_t sequences,
                                         size_t max_length, int int8_weights,
                                         flint_b200_generator** generator) {
    constexpr const char* name = "flint_b200_generator_create";
    if (generator == nullptr) {
        return fb::fail(kInvalid, "%s: generator is null", name);
    }
    *generator = nullptr;
    if (model == nullptr) {
        return fb::fail(kInvalid, "%s: model is null", name);
    }
    const flint_gpt2_config& c = model->config;
    if (c.width / c.heads != kHeadWidth || c.width % 128 != 0 || c.width > 1600) {
        return fb::fail(kInvalid, "%s: needs heads of width 64 and a width (%zu) that is a "
                        "multiple of 128 up to 1600", name, c.width);
    }
    if (model->tensors.empty() || model->wte->half == nullptr) {
        return fb::fail(kInvalid, "%s: the model has no FP16 weight copies", name);
    }
    if (sequences < 1 || sequences > 64) {
        return fb::fail(kInvalid, "%s: sequences (%zu) must be from 1 to 64", name, sequences);
    }
    if (max_length < 8 || max_length % 8 != 0 || max_length > c.block_size || max_length > 1024) {
        return fb::fail(kInvalid, "%s: max_length (%zu) must be a multiple of 8 from 8 to "
                        "min(block_size (%zu), 1024)", name, max_length, c.block_size);
    }
    std::unique_ptr<flint_b200_generator> g(new (std::nothrow) flint_b200_generator);
    if (!g) {
        return fb::fail(FLINT_ERROR_CUDA, "%s: out of host memory", name);
    }
    g->model = model;
    g->sequences = sequences;
    g->max_length = max_length;
    g->int8 = int8_weights != 0;
    try {
        FB_TRY(build(*g, nullptr));
        FB_TRY(flint_b200_generator_refresh(g.get(), nullptr));
    } catch (const std::bad_alloc&) {
        return fb::fail(FLINT_ERROR_CUDA, "%s: out of host memory", name);
    }
    FB_CUDA(cudaDeviceSynchronize());
    *generator = g.release();
    return FLINT_OK;
}

void flint_b200_generator_destroy(flint_b200_generator* generator) { delete generator; }

flint_status flint_b200_generator_refresh(flint_b200_generator* generator, flint_stream stream) {
    if (generator == nullptr) {
        return fb::fail(kInvalid, "flint_b200_generator_refresh: generator is null");
    }
    flint_b200_generator& g = *generator;
    if (g.int8) {
        for (Layer& l : g.blocks) {
            FB_TRY(quantize(g, l.attn, stream));
            FB_TRY(quantize(g, l.proj, stream));
            FB_TRY(quantize(g, l.fc, stream));
            FB_TRY(quantize(g, l.fcproj, stream));
        }
        FB_TRY(quantize(g, g.head, stream));
    }
    return FLINT_OK;
}

flint_status flint_b200_generator_prefill(flint_b200_generator* generator, const void* tokens,
                                          size_t length, flint_stream stream) {
    constexpr const char* name = "flint_b200_generator_prefill";
    if (generator == nullptr) {
        return fb::fail(kInvalid, "%s: generator is null", name);
    }
    flint_b200_generator& g = *generator;
    if (length < 8 || length % 8 != 0 || length > g.max_length) {
        return fb::fail(kInvalid, "%s: length (%zu) must be a multiple of 8 from 8 to max_length "
                        "(%zu)", name, length, g.max_length);
    }
    const size_t rows = g.sequences * length;
    const fb::Span spans[] = {{"tokens", tokens, rows * 2}};
    FB_TRY(fb::check_spans(name, spans, 0));
    g.host_position = 0;
    FB_CUDA(cudaMemsetAsync(g.position, 0, 4, stream));
    FB_TRY(flint_embedding_forward(g.x_a, tokens, g.wte, g.wpe, g.sequences, length, g.padded_vocab,
                                   g.width, stream));
    FB_TRY(run_blocks(g, length, false, stream));
    fb_take_last_rows<<<static_cast<unsigned>(g.sequences), 256, 0, stream>>>(
        g.last, g.x_a, static_cast<int>(length), static_cast<int>(g.width));
    FB_CUDA(fb::after_launch());
    FB_TRY(run_head(g, g.last, nullptr, stream));
    fb_advance_position<<<1, 1, 0, stream>>>(g.position, static_cast<int>(length));
    FB_CUDA(fb::after_launch());
    g.host_position = length;
    return FLINT_OK;
}

flint_status flint_b200_generator_step(flint_b200_generator* generator, const void* tokens,
                                       void* next_tokens, int use_graph, flint_stream stream) {
    constexpr const char* name = "flint_b200_generator_step";
    if (generator == nullptr) {
        return fb::fail(kInvalid, "%s: generator is null", name);
    }
    flint_b200_generator& g = *generator;
    if (g.host_position >= g.max_length) {
        return fb::fail(kInvalid, "%s: the cache is full (%zu positions)", name, g.max_length);
    }
    const fb::Span spans[] = {{"tokens", tokens, g.sequences * 2}};
    FB_TRY(fb::check_spans(name, spans, 0));
    if (use_graph == 0) {
        FB_TRY(enqueue_step(g, tokens, next_tokens, stream));
        g.host_position += 1;
        return FLINT_OK;
    }
    // The step's launches depend on the position only through device memory, so one
    // captured graph serves every token as long as the caller's buffers stay the same.
    if (g.step_graph != nullptr && (g.graph_tokens != tokens || g.graph_next != next_tokens)) {
        cudaGraphExecDestroy(g.step_graph);
        g.step_graph = nullptr;
    }
    if (g.step_graph == nullptr) {
        cudaStream_t capture = nullptr;
        FB_CUDA(cudaStreamCreateWithFlags(&capture, cudaStreamNonBlocking));
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamBeginCapture(capture, cudaStreamCaptureModeThreadLocal);
        flint_status status = FLINT_OK;
        if (e == cudaSuccess) {
            status = enqueue_step(g, tokens, next_tokens, capture);
            e = cudaStreamEndCapture(capture, &graph);
        }
        if (e == cudaSuccess && status == FLINT_OK) {
            e = cudaGraphInstantiate(&g.step_graph, graph, 0);
        }
        if (graph != nullptr) {
            cudaGraphDestroy(graph);
        }
        cudaStreamDestroy(capture);
        if (status != FLINT_OK) {
            return status;
        }
        FB_CUDA(e);
        g.graph_tokens = tokens;
        g.graph_next = next_tokens;
    }
    FB_CUDA(cudaGraphLaunch(g.step_graph, stream));
    g.host_position += 1;
    return FLINT_OK;
}

flint_status flint_b200_generator_logits(const flint_b200_generator* generator,
                                         const void** logits, size_t* position) {
    if (generator == nullptr) {
        return fb::fail(kInvalid, "flint_b200_generator_logits: generator is null");
    }
    if (logits != nullptr) {
        *logits = generator->logits;
    }
    if (position != nullptr) {
        *position = generator->host_position;
    }
    return FLINT_OK;
}

flint_status flint_b200_generator_bytes_per_step(const flint_b200_generator* generator,
                                                 size_t* weight_bytes, size_t* cache_bytes) {
    if (generator == nullptr) {
        return fb::fail(kInvalid, "flint_b200_generator_bytes_per_step: generator is null");
    }
    const flint_b200_generator& g = *generator;
    const size_t element = g.int8 ? 1 : 2;
    size_t weights = g.head.n * g.head.k * element;
    for (const Layer& l : g.blocks) {
        for (const Matrix* m : {&l.attn, &l.proj, &l.fc, &l.fcproj}) {
            weights += m->n * m->k * element;
        }
    }
    // The output layer is streamed once per group of eight sequences.
    weights += g.head.n * g.head.k * element * ((g.sequences + kSkinnyRows - 1) / kSkinnyRows - 1);
    if (weight_bytes != nullptr) {
        *weight_bytes = weights;
    }
    if (cache_bytes != nullptr) {
        *cache_bytes = 2 * g.layers * g.sequences * g.heads * (g.host_position + 1) * kHeadWidth * 2;
    }
    return FLINT_OK;
}

}  // extern "C"
