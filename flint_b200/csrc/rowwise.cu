// Row-wise entry points: flint_layernorm_forward, flint_causal_softmax_forward,
// flint_causal_softmax_backward and flint_softmax_cross_entropy.
//
// Each kernel reads its row from HBM once. LayerNorm and the attention
// softmax keep a row in the registers of one warp (GPT-2's rows are 768 FP32
// and at most 1,024 FP16 values); the cross-entropy stages a 100 KB row of
// logits in shared memory for its three passes. Sums run in FP32 with
// compensated (TwoSum) accumulation where the reference does, in the same
// lane order, so statistics match it to the bit where its tests pin them:
// src/kernels/layernorm.cu:105-155, src/kernels/softmax.cu:68-122,
// src/kernels/softmax_backward.cu:111-154, src/kernels/cross_entropy.cu:106-172.
//
// Argument checks follow src/api/layernorm.cpp:11-51, src/api/softmax.cpp:11-76
// and src/api/cross_entropy.cpp:9-49.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>

#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"

namespace {

using fb::Comp;

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = 32 * kWarpsPerBlock;
constexpr size_t kMaxRows8 = size_t{0x7fffffff} * 8;

// ---- LayerNorm forward -----------------------------------------------------------

// Rows of up to 128 * kQuads values with cols % 4 == 0: the warp holds the row
// in registers, lane l owning float4 groups l, l + 32, ...
// kPlain (the model on the fused attention kernels only; the public entry point never uses it):
// the two row sums take ordinary FP32 adds in four interleaved streams and a butterfly,
// deterministic and within a few 2^-24 of the compensated result, at a seventh of the
// arithmetic; everything after the sums is the same.
template <int kQuads, bool kPlain = false>
__global__ void __launch_bounds__(kThreads)
    fb_layernorm_forward_regs(__half* __restrict__ y, float* __restrict__ mean,
                              float* __restrict__ rstd, const float* __restrict__ x,
                              const float* __restrict__ gamma, const float* __restrict__ beta,
                              size_t rows, int cols, float eps) {
    fb::dependency_wait();
    fb::dependency_release();
    const size_t row = size_t{blockIdx.x} * kWarpsPerBlock + threadIdx.x / 32;
    if (row >= rows) {
        return;
    }
    const int lane = threadIdx.x % 32;
    const int groups = cols / 4;
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    float4 v[kQuads];
#pragma unroll
    for (int j = 0; j < kQuads; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < groups ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const float n = static_cast<float>(cols);

    float m;
    float var;
    if (kPlain) {
        // Absent groups hold zeros, which the first sum ignores and the second one masks.
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            a = make_float4(a.x + v[j].x, a.y + v[j].y, a.z + v[j].z, a.w + v[j].w);
        }
        m = __fdiv_rn(fb::warp_sum_rn((a.x + a.y) + (a.z + a.w)), n);
        float4 q = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            if (lane + 32 * j < groups) {
                const float d0 = v[j].x - m, d1 = v[j].y - m, d2 = v[j].z - m, d3 = v[j].w - m;
                q = make_float4(fmaf(d0, d0, q.x), fmaf(d1, d1, q.y), fmaf(d2, d2, q.z),
                                fmaf(d3, d3, q.w));
            }
        }
        var = __fdiv_rn(fb::warp_sum_rn((q.x + q.y) + (q.z + q.w)), n);
    } else {
        Comp sum;
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            if (lane + 32 * j < groups) {
                fb::comp_add(sum, v[j].x);
                fb::comp_add(sum, v[j].y);
                fb::comp_add(sum, v[j].z);
                fb::comp_add(sum, v[j].w);
            }
        }
        sum = fb::comp_warp_merge(sum);
        m = __fdiv_rn(__fadd_rn(sum.s, sum.e), n);

        Comp sq;
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            if (lane + 32 * j < groups) {
                const float d0 = __fsub_rn(v[j].x, m);
                const float d1 = __fsub_rn(v[j].y, m);
                const float d2 = __fsub_rn(v[j].z, m);
                const float d3 = __fsub_rn(v[j].w, m);
                fb::comp_add_product(sq, d0, d0);
                fb::comp_add_product(sq, d1, d1);
                fb::comp_add_product(sq, d2, d2);
                fb::comp_add_product(sq, d3, d3);
            }
        }
        sq = fb::comp_warp_merge(sq);
        var = __fdiv_rn(__fadd_rn(sq.s, sq.e), n);
    }
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));

    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
    uint2* yr = reinterpret_cast<uint2*>(y + row * cols);
#pragma unroll
    for (int j = 0; j < kQuads; ++j) {
        const int i = lane + 32 * j;
        if (i < groups) {
            const float4 g = g4[i];
            const float4 b = b4[i];
            const float o0 = fmaf(__fmul_rn(__fsub_rn(v[j].x, m), r), g.x, b.x);
            const float o1 = fmaf(__fmul_rn(__fsub_rn(v[j].y, m), r), g.y, b.y);
            const float o2 = fmaf(__fmul_rn(__fsub_rn(v[j].z, m), r), g.z, b.z);
            const float o3 = fmaf(__fmul_rn(__fsub_rn(v[j].w, m), r), g.w, b.w);
            yr[i] = make_uint2(fb::pack2(o0, o1), fb::pack2(o2, o3));
        }
    }
    if (lane == 0) {
        mean[row] = m;
        rstd[row] = r;
    }
}

// Any width: three passes over the row in global memory (the later ones hit
// L1/L2). kVec is 4 when cols % 4 == 0, else 1.
template <int kVec>
__global__ void __launch_bounds__(kThreads)
    fb_layernorm_forward_stream(__half* __restrict__ y, float* __restrict__ mean,
                                float* __restrict__ rstd, const float* __restrict__ x,
                                const float* __restrict__ gamma, const float* __restrict__ beta,
                                size_t rows, int cols, float eps) {
    const size_t row = size_t{blockIdx.x} * kWarpsPerBlock + threadIdx.x / 32;
    if (row >= rows) {
        return;
    }
    const int lane = threadIdx.x % 32;
    const float* xr = x + row * cols;
    __half* yr = y + row * cols;
    const int groups = cols / kVec;
    const float n = static_cast<float>(cols);

    auto load = [&](const float* p, int i, float (&f)[kVec]) {
        if constexpr (kVec == 4) {
            const float4 q = reinterpret_cast<const float4*>(p)[i];
            f[0] = q.x;
            f[1] = q.y;
            f[2] = q.z;
            f[3] = q.w;
        } else {
            f[0] = p[i];
        }
    };

    Comp sum;
    for (int i = lane; i < groups; i += 32) {
        float f[kVec];
        load(xr, i, f);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            fb::comp_add(sum, f[j]);
        }
    }
    sum = fb::comp_warp_merge(sum);
    const float m = __fdiv_rn(__fadd_rn(sum.s, sum.e), n);

    Comp sq;
    for (int i = lane; i < groups; i += 32) {
        float f[kVec];
        load(xr, i, f);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const float d = __fsub_rn(f[j], m);
            fb::comp_add_product(sq, d, d);
        }
    }
    sq = fb::comp_warp_merge(sq);
    const float var = __fdiv_rn(__fadd_rn(sq.s, sq.e), n);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));

    for (int i = lane; i < groups; i += 32) {
        float f[kVec];
        float g[kVec];
        float b[kVec];
        load(xr, i, f);
        load(gamma, i, g);
        load(beta, i, b);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            f[j] = fmaf(__fmul_rn(__fsub_rn(f[j], m), r), g[j], b[j]);
        }
        if constexpr (kVec == 4) {
            reinterpret_cast<uint2*>(yr)[i] =
                make_uint2(fb::pack2(f[0], f[1]), fb::pack2(f[2], f[3]));
        } else {
            yr[i] = __float2half_rn(f[0]);
        }
    }
    if (lane == 0) {
        mean[row] = m;
        rstd[row] = r;
    }
}

// ---- causal softmax ------------------------------------------------------------------

constexpr int kMaxChunksPerLane = 4;  // 1024 columns / 8 per chunk / 32 lanes

// A warp per row; lane l owns the 16-byte chunks l, l + 32, l + 64, l + 96.
template <int kChunks>
__global__ void __launch_bounds__(kThreads)
    fb_causal_softmax_forward(uint4* __restrict__ p, const uint4* __restrict__ s, size_t rows,
                              int length) {
    const size_t row = size_t{blockIdx.x} * kWarpsPerBlock + threadIdx.x / 32;
    if (row >= rows) {
        return;
    }
    const int lane = threadIdx.x % 32;
    const int chunks = length / 8;
    const int t = static_cast<int>(row % static_cast<size_t>(length));
    const int visible_chunks = t / 8 + 1;
    const uint4* sr = s + row * chunks;
    uint4* pr = p + row * chunks;

    float v[kChunks][8];
    int count[kChunks];  // visible values of each owned chunk (0 when masked)
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        const int i = lane + 32 * j;
        count[j] = i < visible_chunks ? min(t + 1 - i * 8, 8) : 0;
        if (count[j] > 0) {
            fb::unpack8(v[j], sr[i]);
        }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < count[j]) {
                mx = fmaxf(mx, v[j][c]);
            }
        }
    }
    mx = fb::warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < count[j]) {
                v[j][c] = expf(__fsub_rn(v[j][c], mx));
                sum = __fadd_rn(sum, v[j][c]);
            }
        }
    }
    sum = fb::warp_sum_rn(sum);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        const int i = lane + 32 * j;
        if (i >= chunks) {
            continue;
        }
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            o[c] = c < count[j] ? __fmul_rn(v[j][c], inv) : 0.0f;
        }
        pr[i] = fb::pack8(o);
    }
}

template <int kChunks>
__global__ void __launch_bounds__(kThreads)
    fb_causal_softmax_backward(uint4* ds, const uint4* __restrict__ p, const uint4* dp,
                               size_t rows, int length, float scale) {
    const size_t row = size_t{blockIdx.x} * kWarpsPerBlock + threadIdx.x / 32;
    if (row >= rows) {
        return;
    }
    const int lane = threadIdx.x % 32;
    const int chunks = length / 8;
    const int t = static_cast<int>(row % static_cast<size_t>(length));
    const int visible_chunks = t / 8 + 1;
    const uint4* pr = p + row * chunks;
    const uint4* dpr = dp + row * chunks;
    uint4* dsr = ds + row * chunks;

    float pv[kChunks][8];
    float dv[kChunks][8];
    int count[kChunks];
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        const int i = lane + 32 * j;
        count[j] = i < visible_chunks ? min(t + 1 - i * 8, 8) : 0;
        if (count[j] > 0) {
            fb::unpack8(pv[j], pr[i]);
            fb::unpack8(dv[j], dpr[i]);
        }
    }
    // D = sum of p * dp over the visible columns; each product of two FP16
    // values is exact in FP32.
    Comp d;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < count[j]) {
                fb::comp_add(d, __fmul_rn(pv[j][c], dv[j][c]));
            }
        }
    }
    d = fb::comp_warp_merge(d);
    if (!isfinite(d.s)) {
        d.e = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        const int i = lane + 32 * j;
        if (i >= chunks) {
            continue;
        }
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float diff = __fsub_rn(__fsub_rn(dv[j][c], d.s), d.e);
            o[c] = c < count[j] ? __fmul_rn(__fmul_rn(pv[j][c], diff), scale) : 0.0f;
        }
        dsr[i] = fb::pack8(o);
    }
}

flint_status check_softmax_dims(const char* name, size_t batches, size_t length) {
    constexpr size_t kMaxLength = 1024;
    constexpr size_t kMaxBatches = 65535;
    if (length % 8 != 0 || length > kMaxLength) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: length (%zu) must be a multiple of 8 up to %zu", name, length,
                        kMaxLength);
    }
    if (batches > kMaxBatches) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: batches (%zu) can be up to %zu", name,
                        batches, kMaxBatches);
    }
    return FLINT_OK;
}

// ---- softmax + cross-entropy ------------------------------------------------------------

constexpr int kCeThreads = 1024;
constexpr int kCeWarps = kCeThreads / 32;

__device__ __forceinline__ float ce_block_max(float v, float* scratch) {
    v = fb::warp_max(v);
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    float m = scratch[lane];  // kCeWarps == 32: one value per lane
    return fb::warp_max(m);
}

// Every thread receives the same total: warp butterflies, then one butterfly
// over the 32 warp totals, all in a fixed order.
__device__ __forceinline__ float ce_block_total(Comp a, float* scratch) {
    a = fb::comp_warp_merge(a);
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    __syncthreads();
    if (lane == 0) {
        scratch[2 * warp] = a.s;
        scratch[2 * warp + 1] = a.e;
    }
    __syncthreads();
    Comp total;
    total.s = scratch[2 * lane];
    total.e = scratch[2 * lane + 1];
    total = fb::comp_warp_merge(total);
    return __fadd_rn(total.s, total.e);
}

// e^x for two values x <= 0 at a time (x >= -64 after the clamp below):
// n = round(x log2 e) by the magic-number add, r = x - n ln 2 in two fused steps
// (n ln2_hi is exact), 2^(r log2 e) on the special-function unit with |r log2 e|
// <= 1/2, and n added into the exponent. About 2 ulps, like expf.
__device__ __forceinline__ void exp_pair(fb::F2 x, float& e0, float& e1) {
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
    constexpr float kLn2Hi = 0.693145751953125f;
    constexpr float kLn2Lo = 1.42860682030941723212e-6f;
    const fb::F2 t = fb::f2_fma(x, fb::f2_pack(kLog2e, kLog2e), fb::f2_pack(kMagic, kMagic));
    const fb::F2 n = fb::f2_sub(t, fb::f2_pack(kMagic, kMagic));
    fb::F2 r = fb::f2_fma(n, fb::f2_pack(-kLn2Hi, -kLn2Hi), x);
    r = fb::f2_fma(n, fb::f2_pack(-kLn2Lo, -kLn2Lo), r);
    float y0, y1, t0, t1;
    fb::f2_unpack(fb::f2_mul(r, fb::f2_pack(kLog2e, kLog2e)), y0, y1);
    fb::f2_unpack(t, t0, t1);
    float p0, p1;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(y0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(y1));
    // The low mantissa bits of t hold n (two's complement): 2^n is built from them
    // and multiplied in, so a NaN stays a NaN.
    const float s0 = __int_as_float((__float_as_int(t0) << 23) + 0x3f800000);
    const float s1 = __int_as_float((__float_as_int(t1) << 23) + 0x3f800000);
    fb::f2_unpack(fb::f2_mul(fb::f2_pack(p0, p1), fb::f2_pack(s0, s1)), e0, e1);
}

// The four pairs of a 16-byte word of logits as x = v - mx, with v first clamped
// (as FP16) to mx - 64: e^-64 is far below what the sums or an FP16 gradient can
// see, and the clamp keeps the exponent arithmetic above in range for any logits.
__device__ __forceinline__ void gaps8(fb::F2 (&x)[4], const uint4& q, __half2 floor2, fb::F2 mx2) {
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __hmax2_nan(*reinterpret_cast<const __half2*>(&w[i]), floor2);
        const float2 f = __half22float2(h);
        x[i] = fb::f2_sub(fb::f2_pack(f.x, f.y), mx2);
    }
}

__device__ __forceinline__ float half_max8(const uint4& q) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
    const __half2 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(__low2float(m), __high2float(m));
}

// Set when a bounded wait in this file gave up; read and cleared by
// flint_b200_kernel_fault through rowwise_error_flag.
__device__ int g_rowwise_error = 0;

// Persistent CTAs, one row at a time. Thread 0 streams each row's logits into
// shared memory with one bulk asynchronous copy (two row buffers when they fit,
// so the next row loads while this one is processed); the three passes (max on
// the raw FP16 values, compensated sum of exp, gradient) then run out of shared
// memory, and the row leaves as coalesced 16-byte stores. This kernel serves rows of
// more than 53,248 columns; shorter rows take the rolling kernel further down.
__global__ void __launch_bounds__(kCeThreads, 1)
    fb_softmax_cross_entropy(uint4* __restrict__ dlogits, float* __restrict__ row_loss,
                             const uint4* __restrict__ logits,
                             const uint16_t* __restrict__ targets, float scale, size_t rows,
                             int vocab, int cols, int buffers) {
    extern __shared__ uint4 staged[];
    __shared__ float scratch[2 * kCeWarps];
    __shared__ alignas(8) unsigned long long barriers[2];
    __shared__ int abort_flag;
    const int chunks = cols / 8;
    const int vocab_chunks = (vocab + 7) / 8;
    const uint32_t copy_bytes = static_cast<uint32_t>(vocab_chunks) * 16u;
    const uint32_t bar0 = static_cast<uint32_t>(__cvta_generic_to_shared(&barriers[0]));
    const uint32_t stage0 = static_cast<uint32_t>(__cvta_generic_to_shared(staged));

    auto issue = [&](size_t row, int buffer) {
        const uint32_t bar = bar0 + 8u * buffer;
        const uint32_t dst = stage0 + static_cast<uint32_t>(buffer) * copy_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                     "r"(copy_bytes)
                     : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            ::"r"(dst), "l"(logits + row * chunks), "r"(copy_bytes), "r"(bar)
            : "memory");
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    fb::dependency_wait();
    if (threadIdx.x == 0) {
        fb::dependency_release();
        if (blockIdx.x < rows) {
            issue(blockIdx.x, 0);
        }
    }
    __syncthreads();

    int buffer = 0;
    uint32_t phase[2] = {0u, 0u};
    bool aborted = false;
    bool pending[2] = {blockIdx.x < rows, false};  // thread 0: copies started and not yet seen
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t next = row + gridDim.x;
        if (buffers == 2 && threadIdx.x == 0 && next < rows) {
            issue(next, buffer ^ 1);  // that buffer's readers finished at the last __syncthreads
            pending[buffer ^ 1] = true;
        }
        // Wait for this row's bytes (bounded; on a timeout the row is skipped).
        {
            const uint32_t bar = bar0 + 8u * buffer;
            bool landed = false;
            const long long start = clock64();
            for (uint32_t spin = 0; !landed; ++spin) {
                uint32_t done = 0;
                asm volatile(
                    "{\n.reg .pred p;\n"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                    "selp.u32 %0, 1, 0, p;\n}\n"
                    : "=r"(done)
                    : "r"(bar), "r"(phase[buffer])
                    : "memory");
                landed = done != 0;
                if (!landed && (spin & 255u) == 255u &&
                    (abort_flag != 0 || clock64() - start > 2000000000LL)) {
                    abort_flag = 1;
                    break;
                }
            }
            phase[buffer] ^= 1u;
            // One decision for the whole block: a thread whose wait succeeded must not go
            // on to the block-wide reductions below while others have given up.
            if (__syncthreads_or(landed ? 0 : 1) != 0) {
                aborted = true;
                break;
            }
            pending[buffer] = false;
        }
        const uint4* in = staged + static_cast<size_t>(buffer) * vocab_chunks;
        uint4* out = dlogits + row * chunks;
        const int last_count = vocab - (vocab_chunks - 1) * 8;  // values in the last chunk

        float mx = -INFINITY;
        for (int i = threadIdx.x; i < vocab_chunks; i += kCeThreads) {
            const uint4 q = in[i];
            if (i + 1 < vocab_chunks || last_count == 8) {
                mx = fmaxf(mx, half_max8(q));
            } else {
                float v[8];
                fb::unpack8(v, q);
                for (int c = 0; c < last_count; ++c) {
                    mx = fmaxf(mx, v[c]);
                }
            }
        }
        mx = ce_block_max(mx, scratch);

        // mx is a maximum of FP16 values, so it is one itself; mx - 64 rounds to FP16
        // within 16 for any finite mx (kept finite, so a -inf logit is clamped too).
        const __half2 floor2 = __float2half2_rn(fmaxf(__fsub_rn(mx, 64.0f), -65504.0f));
        const fb::F2 mx2 = fb::f2_pack(mx, mx);
        const int full_chunks = vocab / 8;  // chunks whose 8 values all count

        // A thread adds its (at most 7) words plainly into eight partial sums, one per
        // column of the word: each takes a handful of values in (0, 1], so its rounding
        // error is a few units of 2^-24 of itself. Everything after that (the eight
        // partials, the lanes, the warps) is merged with compensated adds.
        fb::F2 part[4] = {0, 0, 0, 0};
        for (int i = threadIdx.x; i < full_chunks; i += kCeThreads) {
            fb::F2 x[4];
            gaps8(x, in[i], floor2, mx2);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float e0, e1;
                exp_pair(x[c], e0, e1);
                part[c] = fb::f2_add(part[c], fb::f2_pack(e0, e1));
            }
        }
        Comp mine;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float s0, s1;
            fb::f2_unpack(part[c], s0, s1);
            fb::comp_add(mine, s0);
            fb::comp_add(mine, s1);
        }
        if (full_chunks < vocab_chunks && threadIdx.x == (full_chunks % kCeThreads)) {
            // The last, partly filled word: its counted values one by one.
            fb::F2 x[4];
            gaps8(x, in[full_chunks], floor2, mx2);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float e0, e1;
                exp_pair(x[c], e0, e1);
                if (2 * c < last_count) {
                    fb::comp_add(mine, e0);
                }
                if (2 * c + 1 < last_count) {
                    fb::comp_add(mine, e1);
                }
            }
        }
        const float sum = ce_block_total(mine, scratch);
        const float inv = __fdiv_rn(1.0f, sum);
        const fb::F2 inv2 = fb::f2_pack(inv, inv);
        const fb::F2 scale2 = fb::f2_pack(scale, scale);

        const int target = targets[row];
        const int target_chunk = target / 8;
        const int target_slot = target % 8;
        for (int i = threadIdx.x; i < chunks; i += kCeThreads) {
            if (i >= vocab_chunks) {
                out[i] = make_uint4(0u, 0u, 0u, 0u);
                continue;
            }
            fb::F2 x[4];
            gaps8(x, in[i], floor2, mx2);
            float o[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float e0, e1;
                exp_pair(x[c], e0, e1);
                fb::f2_unpack(fb::f2_mul(fb::f2_mul(fb::f2_pack(e0, e1), inv2), scale2), o[2 * c],
                              o[2 * c + 1]);
            }
            if (i >= full_chunks) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    o[c] = c < last_count ? o[c] : 0.0f;
                }
            }
            if (i == target_chunk) {
                // The target column: p - 1, and the row's loss, from the unclamped logit.
                float v[8];
                fb::unpack8(v, in[i]);
                const float gap = __fsub_rn(v[target_slot], mx);
                float e0, e1;
                exp_pair(fb::f2_pack(fmaxf(gap, -64.0f), 0.0f), e0, e1);
                row_loss[row] = __fsub_rn(logf(sum), gap);
                o[target_slot] = __fmul_rn(__fsub_rn(__fmul_rn(e0, inv), 1.0f), scale);
            }
            out[i] = fb::pack8(o);
        }
        __syncthreads();  // everyone is done with this buffer before it is refilled
        if (buffers == 1 && threadIdx.x == 0 && next < rows) {
            issue(next, 0);
            pending[0] = true;
        }
        if (buffers == 2) {
            buffer ^= 1;
        }
    }
    if (aborted && threadIdx.x == 0) {
        // The rows from here on were not computed: report it, and give the copies that were
        // started a second, equally bounded chance to land before the CTA's shared memory
        // is released. (The failed buffer's phase bit was already flipped above.)
        atomicExch(&g_rowwise_error, 1);
        for (int b = 0; b < 2; ++b) {
            if (!pending[b]) {
                continue;
            }
            const uint32_t parity = b == buffer ? phase[b] ^ 1u : phase[b];
            const long long start = clock64();
            uint32_t done = 0;
            while (done == 0 && clock64() - start < 2000000000LL) {
                asm volatile(
                    "{\n.reg .pred p;\n"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                    "selp.u32 %0, 1, 0, p;\n}\n"
                    : "=r"(done)
                    : "r"(bar0 + 8u * b), "r"(parity)
                    : "memory");
            }
        }
    }
}

// Block-wide maximum of `mx` and compensated total of `acc`, both handed to every
// thread, in a fixed order: warp butterflies, then one butterfly over the warps'
// results (lanes beyond the warp count carry the identities).
template <int kWarps>
__device__ __forceinline__ float ce_block_max_total(float& mx, Comp acc, float* scratch) {
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    mx = fb::warp_max(mx);
    acc = fb::comp_warp_merge(acc);
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = mx;
        scratch[32 + 2 * warp] = acc.s;
        scratch[33 + 2 * warp] = acc.e;
    }
    __syncthreads();
    const bool mine = lane < kWarps;
    mx = fb::warp_max(mine ? scratch[lane] : -INFINITY);
    Comp total;
    total.s = mine ? scratch[32 + 2 * lane] : 0.0f;
    total.e = mine ? scratch[33 + 2 * lane] : 0.0f;
    total = fb::comp_warp_merge(total);
    return __fadd_rn(total.s, total.e);
}

// The same arithmetic with each exponential evaluated once, for rows whose
// exponentials fit in shared memory as FP32 (two planes of four values per 16-byte
// word of logits, so that a warp's accesses are contiguous).
//
// A thread owns the words tid, tid + kThreadsT, ... of every row: it holds the
// current row's words in registers, and the exponentials of its words in its own
// shared-memory slots, so the slots need no synchronisation. One step of the loop
// rolls three rows through a thread's slots word by word: the gradient of the row
// before leaves (its exponentials scaled, rounded and stored), the current row's
// exponentials take its place and are summed, and the next row's word is loaded
// into the register just consumed. Loads, stores and arithmetic of three rows are
// therefore in flight together; the only block-wide exchange per row merges the
// row's sum with the next row's maximum.
template <int kThreadsT, int kHeld>
__global__ void __launch_bounds__(kThreadsT, 1)
    fb_softmax_cross_entropy_rolling(uint4* __restrict__ dlogits, float* __restrict__ row_loss,
                                     const uint4* __restrict__ logits,
                                     const uint16_t* __restrict__ targets, float scale,
                                     size_t rows, int vocab, int cols) {
    extern __shared__ uint4 staged[];
    __shared__ float scratch[3 * 32];
    const int chunks = cols / 8;
    const int vocab_chunks = (vocab + 7) / 8;
    const int full_chunks = vocab / 8;  // chunks whose 8 values all count
    const int last_count = vocab - (vocab_chunks - 1) * 8;  // values in the last chunk
    // Two planes a compile-time distance apart: every slot address is the thread's base
    // plus a constant, so the compiler can tell the slots apart and overlap the words.
    constexpr int kSlots = kThreadsT * kHeld;
    float4* plane0 = reinterpret_cast<float4*>(staged);
    float4* plane1 = plane0 + kSlots;
    const int tid = static_cast<int>(threadIdx.x);
    const size_t first = blockIdx.x;
    const size_t stride = gridDim.x;
    const __half* logit_values = reinterpret_cast<const __half*>(logits);

    fb::dependency_wait();
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }
    if (first >= rows) {
        return;
    }
    const int steps = static_cast<int>((rows - first + stride - 1) / stride);
    auto prefetch_row = [&](size_t row) {
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(logits + row * chunks),
                     "r"(static_cast<uint32_t>(vocab_chunks) * 16u)
                     : "memory");
    };
    // The maximum of the words in `held` (of a row's counted values).
    uint4 held[kHeld];
    auto held_max = [&]() {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
            const int i = tid + j * kThreadsT;
            if (i < full_chunks) {
                mx = fmaxf(mx, half_max8(held[j]));
            } else if (i < vocab_chunks) {
                float v[8];
                fb::unpack8(v, held[j]);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    mx = c < last_count ? fmaxf(mx, v[c]) : mx;
                }
            }
        }
        return mx;
    };

    if (tid == 0 && steps > 1) {
        prefetch_row(first + stride);
    }
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
        const int i = tid + j * kThreadsT;
        held[j] = i < vocab_chunks ? __ldg(logits + first * chunks + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    float mx_cur = held_max();
    ce_block_max_total<kThreadsT / 32>(mx_cur, Comp{}, scratch);
    // A row's target and the target's logit are fetched a step before they are needed.
    int target_cur = targets[first];
    float target_logit_cur =
        target_cur < vocab ? __half2float(logit_values[first * cols + target_cur]) : 0.0f;

    // Of the row whose gradient is due: maximum, sum, target and the target's logit.
    float mx_prev = 0.0f, sum_prev = 1.0f, target_logit_prev = 0.0f;
    int target_prev = 0;
    const fb::F2 scale2 = fb::f2_pack(scale, scale);

    for (int s = 0; s <= steps; ++s) {
        const bool grad = s > 0;
        const bool expo = s < steps;
        const bool more = s + 1 < steps;
        const size_t row_cur = first + s * stride;
        const size_t row_prev = grad ? row_cur - stride : first;
        const uint4* next_in = logits + (more ? row_cur + stride : first) * chunks;
        uint4* out = dlogits + row_prev * chunks;
        if (tid == 0 && s + 2 < steps) {
            prefetch_row(row_cur + 2 * stride);
        }
        const int target_next = more ? targets[row_cur + stride] : 0;
        const float inv = __fdiv_rn(1.0f, sum_prev);
        const fb::F2 inv2 = fb::f2_pack(inv, inv);
        const int target_chunk = target_prev / 8;
        const int target_slot = target_prev % 8;
        const __half2 floor2 = __float2half2_rn(fmaxf(__fsub_rn(mx_cur, 64.0f), -65504.0f));
        const fb::F2 mx2 = fb::f2_pack(mx_cur, mx_cur);

        fb::F2 part[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
            const int i = tid + j * kThreadsT;
            if (i >= vocab_chunks) {
                continue;
            }
            if (grad) {
                const float4 a = plane0[i];
                const float4 b = plane1[i];
                const float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                float o[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    fb::f2_unpack(
                        fb::f2_mul(fb::f2_mul(fb::f2_pack(e[2 * c], e[2 * c + 1]), inv2), scale2),
                        o[2 * c], o[2 * c + 1]);
                }
                if (i >= full_chunks) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        o[c] = c < last_count ? o[c] : 0.0f;
                    }
                }
                if (i == target_chunk) {
                    // The target column: p - 1, and the row's loss, from the unclamped logit.
                    const float gap = __fsub_rn(target_logit_prev, mx_prev);
                    float e0, e1;
                    exp_pair(fb::f2_pack(fmaxf(gap, -64.0f), 0.0f), e0, e1);
                    row_loss[row_prev] = __fsub_rn(logf(sum_prev), gap);
                    const float target_out = __fmul_rn(__fsub_rn(__fmul_rn(e0, inv), 1.0f), scale);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        o[c] = c == target_slot ? target_out : o[c];
                    }
                }
                out[i] = fb::pack8(o);
            }
            if (expo) {
                fb::F2 x[4];
                gaps8(x, held[j], floor2, mx2);
                float e[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    exp_pair(x[c], e[2 * c], e[2 * c + 1]);
                }
                plane0[i] = make_float4(e[0], e[1], e[2], e[3]);
                plane1[i] = make_float4(e[4], e[5], e[6], e[7]);
                if (i < full_chunks) {
                    // Plain per-column partial sums of a thread's words; everything after
                    // that is merged with compensated adds.
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        part[c] = fb::f2_add(part[c], fb::f2_pack(e[2 * c], e[2 * c + 1]));
                    }
                }
            }
            if (more) {
                held[j] = __ldg(next_in + i);
            }
        }
        if (grad) {
            for (int i = vocab_chunks + tid; i < chunks; i += kThreadsT) {
                out[i] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        Comp mine;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float s0, s1;
            fb::f2_unpack(part[c], s0, s1);
            fb::comp_add(mine, s0);
            fb::comp_add(mine, s1);
        }
        if (expo && full_chunks < vocab_chunks && tid == full_chunks % kThreadsT) {
            // The last, partly filled word: its counted values one by one (this thread
            // wrote them to its slot above).
            const float4 a = plane0[full_chunks];
            const float4 b = plane1[full_chunks];
            const float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (c < last_count) {
                    fb::comp_add(mine, e[c]);
                }
            }
        }
        const float target_logit_next =
            more && target_next < vocab
                ? __half2float(logit_values[(row_cur + stride) * cols + target_next])
                : 0.0f;
        float mx_next = more ? held_max() : -INFINITY;
        const float sum_cur = ce_block_max_total<kThreadsT / 32>(mx_next, mine, scratch);
        mx_prev = mx_cur;
        mx_cur = mx_next;
        sum_prev = sum_cur;
        target_prev = target_cur;
        target_logit_prev = target_logit_cur;
        target_cur = target_next;
        target_logit_cur = target_logit_next;
    }
}

}  // namespace

namespace fb {

cudaError_t rowwise_error_flag(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_rowwise_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_rowwise_error, &zero, sizeof(int));
    }
    return e;
}

}  // namespace fb

namespace fb {
// The plain-sum variant for rows of up to 768 values with cols % 4 == 0; false when the
// shape is not covered (the caller then uses the public entry point).
bool launch_layernorm_forward_plain(void* y, void* mean, void* rstd, const void* x,
                                    const void* gamma, const void* beta, size_t rows, size_t cols,
                                    float eps, cudaStream_t stream, cudaError_t* error) {
    if (cols % 4 != 0 || cols > 128 * 6 || rows == 0) {
        return false;
    }
    const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    *error = fb::launch_dependent(fb_layernorm_forward_regs<6, true>, dim3(blocks), dim3(kThreads), 0,
                                  stream, static_cast<__half*>(y), static_cast<float*>(mean),
                                  static_cast<float*>(rstd), static_cast<const float*>(x),
                                  static_cast<const float*>(gamma), static_cast<const float*>(beta),
                                  rows, static_cast<int>(cols), eps);
    return true;
}
}  // namespace fb

extern "C" {

flint_status flint_layernorm_forward(void* y, void* mean, void* rstd, const void* x,
                                     const void* gamma, const void* beta, size_t rows,
                                     size_t cols, float eps, flint_stream stream) {
    constexpr const char* name = "flint_layernorm_forward";
    constexpr size_t kMaxCols = size_t{1} << 24;
    if (cols == 0 || cols > kMaxCols) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: cols (%zu) must be from 1 to %zu", name,
                        cols, kMaxCols);
    }
    if (rows > kMaxRows8) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: rows (%zu) can be up to %zu", name,
                        rows, kMaxRows8);
    }
    if (!std::isfinite(eps) || eps < 0.0f) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: eps (%g) must be finite and non-negative", name,
                        static_cast<double>(eps));
    }
    if (rows == 0) {
        return FLINT_OK;
    }
    const fb::Span spans[] = {
        {"y", y, rows * cols * 2},   {"mean", mean, rows * 4},   {"rstd", rstd, rows * 4},
        {"x", x, rows * cols * 4},   {"gamma", gamma, cols * 4}, {"beta", beta, cols * 4},
    };
    FB_TRY(fb::check_spans(name, spans, 3));

    const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto* yh = static_cast<__half*>(y);
    auto* mf = static_cast<float*>(mean);
    auto* rf = static_cast<float*>(rstd);
    const auto* xf = static_cast<const float*>(x);
    const auto* gf = static_cast<const float*>(gamma);
    const auto* bf = static_cast<const float*>(beta);
    const int c = static_cast<int>(cols);
    if (cols % 4 == 0 && cols <= 128 * 2) {
        FB_CUDA(fb::launch_dependent(fb_layernorm_forward_regs<2>, dim3(blocks), dim3(kThreads), 0,
                                     stream, yh, mf, rf, xf, gf, bf, rows, c, eps));
    } else if (cols % 4 == 0 && cols <= 128 * 6) {
        FB_CUDA(fb::launch_dependent(fb_layernorm_forward_regs<6>, dim3(blocks), dim3(kThreads), 0,
                                     stream, yh, mf, rf, xf, gf, bf, rows, c, eps));
    } else if (cols % 4 == 0 && cols <= 128 * 12) {
        FB_CUDA(fb::launch_dependent(fb_layernorm_forward_regs<12>, dim3(blocks), dim3(kThreads), 0,
                                     stream, yh, mf, rf, xf, gf, bf, rows, c, eps));
    } else if (cols % 4 == 0) {
        fb_layernorm_forward_stream<4><<<blocks, kThreads, 0, stream>>>(yh, mf, rf, xf, gf, bf,
                                                                         rows, c, eps);
        FB_CUDA(fb::after_launch());
    } else {
        fb_layernorm_forward_stream<1><<<blocks, kThreads, 0, stream>>>(yh, mf, rf, xf, gf, bf,
                                                                         rows, c, eps);
        FB_CUDA(fb::after_launch());
    }
    return FLINT_OK;
}

flint_status flint_causal_softmax_forward(void* p, const void* s, size_t batches, size_t length,
                                          flint_stream stream) {
    constexpr const char* name = "flint_causal_softmax_forward";
    FB_TRY(check_softmax_dims(name, batches, length));
    if (batches == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t bytes = batches * length * length * 2;
    const fb::Span spans[] = {{"p", p, bytes}, {"s", s, bytes}};
    FB_TRY(fb::check_spans(name, spans, 1));
    const size_t rows = batches * length;
    const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto* pq = static_cast<uint4*>(p);
    const auto* sq = static_cast<const uint4*>(s);
    const int len = static_cast<int>(length);
    if (length <= 256) {
        fb_causal_softmax_forward<1><<<blocks, kThreads, 0, stream>>>(pq, sq, rows, len);
    } else if (length <= 512) {
        fb_causal_softmax_forward<2><<<blocks, kThreads, 0, stream>>>(pq, sq, rows, len);
    } else {
        fb_causal_softmax_forward<kMaxChunksPerLane><<<blocks, kThreads, 0, stream>>>(pq, sq, rows,
                                                                                      len);
    }
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_causal_softmax_backward(void* ds, const void* p, const void* dp, size_t batches,
                                           size_t length, float scale, flint_stream stream) {
    constexpr const char* name = "flint_causal_softmax_backward";
    FB_TRY(check_softmax_dims(name, batches, length));
    if (!std::isfinite(scale)) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: scale (%g) must be finite", name,
                        static_cast<double>(scale));
    }
    if (batches == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t bytes = batches * length * length * 2;
    // Computing in place (ds == dp) is allowed; then dp is not a separate span.
    const fb::Span spans[] = {{"ds", ds, bytes}, {"p", p, bytes}, {"dp", dp, bytes}};
    FB_TRY(fb::check_spans(name, spans, ds == dp ? 2 : 3, 1));
    const size_t rows = batches * length;
    const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto* dsq = static_cast<uint4*>(ds);
    const auto* pq = static_cast<const uint4*>(p);
    const auto* dpq = static_cast<const uint4*>(dp);
    const int len = static_cast<int>(length);
    if (length <= 256) {
        fb_causal_softmax_backward<1><<<blocks, kThreads, 0, stream>>>(dsq, pq, dpq, rows, len,
                                                                       scale);
    } else if (length <= 512) {
        fb_causal_softmax_backward<2><<<blocks, kThreads, 0, stream>>>(dsq, pq, dpq, rows, len,
                                                                       scale);
    } else {
        fb_causal_softmax_backward<kMaxChunksPerLane><<<blocks, kThreads, 0, stream>>>(
            dsq, pq, dpq, rows, len, scale);
    }
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_softmax_cross_entropy(void* dlogits, void* row_loss, const void* logits,
                                         const void* targets, float scale, size_t rows,
                                         size_t vocab, size_t cols, flint_stream stream) {
    constexpr const char* name = "flint_softmax_cross_entropy";
    constexpr size_t kMaxCols = size_t{1} << 16;
    if (cols == 0 || cols % 8 != 0 || cols > kMaxCols) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: cols (%zu) must be a multiple of 8 from 8 to %zu", name, cols,
                        kMaxCols);
    }
    if (vocab == 0 || vocab > cols) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: vocab (%zu) must be from 1 to cols (%zu)", name, vocab, cols);
    }
    if (rows > kMaxRows8) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: rows (%zu) can be up to %zu", name,
                        rows, kMaxRows8);
    }
    if (!std::isfinite(scale)) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: scale (%g) must be finite", name,
                        static_cast<double>(scale));
    }
    if (rows == 0) {
        return FLINT_OK;
    }
    const fb::Span spans[] = {
        {"dlogits", dlogits, rows * cols * 2},
        {"row_loss", row_loss, rows * 4},
        {"logits", logits, rows * cols * 2},
        {"targets", targets, rows * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 2));

    int sms = 148;
    FB_CUDA(fb::sm_count(&sms));
    const unsigned blocks = static_cast<unsigned>(std::min<size_t>(rows, static_cast<size_t>(sms)));
    constexpr size_t kMaxSmem = 220 * 1024;
    const size_t vocab_chunks = (vocab + 7) / 8;
    // 16 warps with 13 words each: 6,656 words cover GPT-2's 6,283 at 94%; measured against
    // 18 to 25 warps with fewer words and registers each, this was the fastest.
    constexpr int kRollThreads = 512, kRollHeld = 13;
    static_assert(size_t{kRollThreads} * kRollHeld * 32 <= kMaxSmem, "the exponentials' planes");
    if (vocab_chunks <= static_cast<size_t>(kRollHeld) * kRollThreads) {
        static std::atomic<bool> roll_configured[64] = {};
        FB_CUDA(fb::allow_shared_memory(fb_softmax_cross_entropy_rolling<kRollThreads, kRollHeld>,
                                        static_cast<int>(kMaxSmem), roll_configured));
        FB_CUDA(fb::launch_dependent(fb_softmax_cross_entropy_rolling<kRollThreads, kRollHeld>,
                                     dim3(blocks), dim3(kRollThreads),
                                     size_t{kRollThreads} * kRollHeld * 32, stream,
                                     static_cast<uint4*>(dlogits), static_cast<float*>(row_loss),
                                     static_cast<const uint4*>(logits),
                                     static_cast<const uint16_t*>(targets), scale, rows,
                                     static_cast<int>(vocab), static_cast<int>(cols)));
        return FLINT_OK;
    }
    // Longer rows: only the vocab columns are staged as FP16; two row buffers when they fit.
    const size_t row_bytes = vocab_chunks * 16;
    const int buffers = 2 * row_bytes <= kMaxSmem ? 2 : 1;
    static std::atomic<bool> configured[64] = {};
    FB_CUDA(fb::allow_shared_memory(fb_softmax_cross_entropy, static_cast<int>(kMaxSmem),
                                    configured));
    FB_CUDA(fb::launch_dependent(fb_softmax_cross_entropy, dim3(blocks), dim3(kCeThreads),
                                 buffers * row_bytes, stream, static_cast<uint4*>(dlogits),
                                 static_cast<float*>(row_loss), static_cast<const uint4*>(logits),
                                 static_cast<const uint16_t*>(targets), scale, rows,
                                 static_cast<int>(vocab), static_cast<int>(cols), buffers));
    return FLINT_OK;
}

}  // extern "C"
