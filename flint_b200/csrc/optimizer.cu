// Optimizer-side extension kernels: fused AdamW with the FP16 weight sync,
// and the non-finite / squared-norm check behind dynamic loss scaling. All
// HBM-bound element-wise passes with 128-bit accesses.
//
// Semantics are torch.optim.AdamW's (decoupled weight decay, bias-corrected
// moments), as the reference's oracle configures it in
// scripts/gpt2_torch.py:161-192.
#include <algorithm>
#include <cmath>
#include <cstdint>

#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"
#include "flint/flint_b200.h"
#include "gemm.h"

namespace {

constexpr int kThreads = 256;
constexpr flint_status kInvalid = FLINT_ERROR_INVALID_ARGUMENT;

struct AdamArgs {
    float lr, beta1, beta2, eps, weight_decay, grad_scale, correction1, correction2;
};

__device__ __forceinline__ float adam_one(float& p, float& m, float& v, float g,
                                          const AdamArgs& a) {
    g *= a.grad_scale;
    m = a.beta1 * m + (1.0f - a.beta1) * g;
    v = a.beta2 * v + (1.0f - a.beta2) * g * g;
    const float m_hat = m / a.correction1;
    const float v_hat = v / a.correction2;
    p = p - a.lr * (a.weight_decay * p + m_hat / (sqrtf(v_hat) + a.eps));
    return p;
}

__global__ void __launch_bounds__(kThreads)
    fb_adamw(float4* __restrict__ param, float4* __restrict__ m, float4* __restrict__ v,
             const float4* __restrict__ grad, uint2* __restrict__ half_copy, size_t quads,
             size_t count, AdamArgs a, const int* __restrict__ skip) {
    if (skip != nullptr && *skip != 0) {
        return;
    }
    const size_t stride = size_t{gridDim.x} * kThreads;
    for (size_t i = size_t{blockIdx.x} * kThreads + threadIdx.x; i < quads; i += stride) {
        float4 p = param[i];
        float4 mm = m[i];
        float4 vv = v[i];
        const float4 g = grad[i];
        adam_one(p.x, mm.x, vv.x, g.x, a);
        adam_one(p.y, mm.y, vv.y, g.y, a);
        adam_one(p.z, mm.z, vv.z, g.z, a);
        adam_one(p.w, mm.w, vv.w, g.w, a);
        param[i] = p;
        m[i] = mm;
        v[i] = vv;
        if (half_copy != nullptr) {
            half_copy[i] = make_uint2(fb::pack2(p.x, p.y), fb::pack2(p.z, p.w));
        }
    }
    // Up to three trailing values.
    const size_t tail = quads * 4;
    if (blockIdx.x == 0 && threadIdx.x < count - tail) {
        const size_t i = tail + threadIdx.x;
        float* ps = reinterpret_cast<float*>(param);
        float* ms = reinterpret_cast<float*>(m);
        float* vs = reinterpret_cast<float*>(v);
        const float g = reinterpret_cast<const float*>(grad)[i];
        adam_one(ps[i], ms[i], vs[i], g, a);
        if (half_copy != nullptr) {
            reinterpret_cast<__half*>(half_copy)[i] = __float2half_rn(ps[i]);
        }
    }
}

__global__ void __launch_bounds__(kThreads)
    fb_check_gradients(const float* __restrict__ grad, size_t count, float scale,
                       int* __restrict__ found, double* __restrict__ sum_squares) {
    __shared__ double warp_sums[kThreads / 32];
    __shared__ int warp_bad[kThreads / 32];
    const size_t stride = size_t{gridDim.x} * kThreads;
    const size_t quads = count / 4;
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    bool bad = false;
    float partial = 0.0f;
    double total = 0.0;
    int folded = 0;
    for (size_t i = size_t{blockIdx.x} * kThreads + threadIdx.x; i < quads; i += stride) {
        const float4 g = g4[i];
        bad |= !(isfinite(g.x) && isfinite(g.y) && isfinite(g.z) && isfinite(g.w));
        const float a = g.x * scale, b = g.y * scale, c = g.z * scale, d = g.w * scale;
        partial += a * a + b * b + c * c + d * d;
        if (++folded == 64) {  // keep the FP32 partial short
            total += partial;
            partial = 0.0f;
            folded = 0;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < count - quads * 4) {
        const float g = grad[quads * 4 + threadIdx.x];
        bad |= !isfinite(g);
        partial += g * scale * g * scale;
    }
    total += partial;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        total += __shfl_xor_sync(fb::kFullMask, total, off);
    }
    const bool any_bad = __any_sync(fb::kFullMask, bad);
    const int warp = threadIdx.x / 32;
    if (threadIdx.x % 32 == 0) {
        warp_sums[warp] = total;
        warp_bad[warp] = any_bad ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double block_total = 0.0;
        int block_bad = 0;
        for (int w = 0; w < kThreads / 32; ++w) {
            block_total += warp_sums[w];
            block_bad |= warp_bad[w];
        }
        if (block_bad) {
            *found = 1;  // every writer stores the same value
        }
        if (sum_squares != nullptr) {
            atomicAdd(sum_squares, block_total);
        }
    }
}

unsigned grid_for(size_t items) {
    int sms = 148;
    fb::sm_count(&sms);
    const size_t wanted = (items + kThreads - 1) / kThreads;
    return static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(wanted, size_t(sms) * 8)));
}

}  // namespace

extern "C" {

flint_status flint_b200_adamw(void* param, void* m, void* v, const void* grad, void* half_copy,
                              size_t count, float lr, float beta1, float beta2, float eps,
                              float weight_decay, float grad_scale, int step, const int* skip,
                              flint_stream stream) {
    constexpr const char* name = "flint_b200_adamw";
    if (step < 1) {
        return fb::fail(kInvalid, "%s: step (%d) must be at least 1", name, step);
    }
    if (!std::isfinite(lr) || !std::isfinite(grad_scale) || !(beta1 >= 0.0f && beta1 < 1.0f) ||
        !(beta2 >= 0.0f && beta2 < 1.0f) || !(eps >= 0.0f) || !std::isfinite(weight_decay)) {
        return fb::fail(kInvalid, "%s: hyper-parameters must be finite, with betas in [0, 1)",
                        name);
    }
    if (count == 0) {
        return FLINT_OK;
    }
    if (count > SIZE_MAX / 4) {
        return fb::fail(kInvalid, "%s: count (%zu) can be up to %zu", name, count, SIZE_MAX / 4);
    }
    const fb::Span spans[] = {
        {"param", param, count * 4},
        {"m", m, count * 4},
        {"v", v, count * 4},
        {"grad", grad, count * 4},
    };
    FB_TRY(fb::check_spans(name, spans, 3));
    if (half_copy != nullptr) {
        const fb::Span extra[] = {
            {"half_copy", half_copy, count * 2}, {"param", param, count * 4},
            {"m", m, count * 4},                 {"v", v, count * 4},
            {"grad", grad, count * 4},
        };
        FB_TRY(fb::check_spans(name, extra, 1));
    }
    AdamArgs a;
    a.lr = lr;
    a.beta1 = beta1;
    a.beta2 = beta2;
    a.eps = eps;
    a.weight_decay = weight_decay;
    a.grad_scale = grad_scale;
    a.correction1 = static_cast<float>(1.0 - std::pow(static_cast<double>(beta1), step));
    a.correction2 = static_cast<float>(1.0 - std::pow(static_cast<double>(beta2), step));
    fb_adamw<<<grid_for(count / 4 + 1), kThreads, 0, stream>>>(
        static_cast<float4*>(param), static_cast<float4*>(m), static_cast<float4*>(v),
        static_cast<const float4*>(grad), static_cast<uint2*>(half_copy), count / 4, count, a,
        skip);
    FB_CUDA(cudaGetLastError());
    return FLINT_OK;
}

flint_status flint_b200_check_gradients(const void* grad, size_t count, float scale,
                                        int* found_nonfinite, double* sum_squares,
                                        flint_stream stream) {
    constexpr const char* name = "flint_b200_check_gradients";
    if (found_nonfinite == nullptr) {
        return fb::fail(kInvalid, "%s: found_nonfinite is null", name);
    }
    if (count == 0) {
        return FLINT_OK;
    }
    const fb::Span spans[] = {{"grad", grad, count * 4}};
    FB_TRY(fb::check_spans(name, spans, 0));
    fb_check_gradients<<<grid_for(count / 4 + 1), kThreads, 0, stream>>>(
        static_cast<const float*>(grad), count, scale, found_nonfinite, sum_squares);
    FB_CUDA(cudaGetLastError());
    return FLINT_OK;
}

flint_status flint_b200_kernel_fault(int* raised) {
    if (raised == nullptr) {
        return fb::fail(kInvalid, "flint_b200_kernel_fault: raised is null");
    }
    FB_CUDA(fb::gemm_error_flag(raised, true));
    return FLINT_OK;
}

}  // extern "C"
