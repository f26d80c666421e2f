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
#include <cstring>
#include <vector>

#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"
#include "flint/flint_b200.h"
#include "attention.h"
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

// ---- multi-tensor AdamW: one launch for a whole model ---------------------------------------

constexpr size_t kItemValues = 8192;  // values per work item (multiple of 4)

struct AdamTensor {
    float* param;
    float* m;
    float* v;
    const float* grad;
    __half* half_copy;
    size_t count;
    float weight_decay;
    float pad;
};

struct AdamItem {
    unsigned tensor;
    unsigned pad;
    size_t first;  // first value of the tensor this item covers
};

struct AdamPlanHeader {
    size_t tensors;
    size_t items;
    size_t tensor_offset;  // bytes from the start of the plan
    size_t item_offset;
};

__global__ void __launch_bounds__(kThreads)
    fb_adamw_multi(const unsigned char* __restrict__ plan, AdamArgs a,
                   const int* __restrict__ skip) {
    if (skip != nullptr && *skip != 0) {
        return;
    }
    const AdamPlanHeader* header = reinterpret_cast<const AdamPlanHeader*>(plan);
    const AdamTensor* tensors = reinterpret_cast<const AdamTensor*>(plan + header->tensor_offset);
    const AdamItem* items = reinterpret_cast<const AdamItem*>(plan + header->item_offset);
    for (size_t it = blockIdx.x; it < header->items; it += gridDim.x) {
        const AdamItem item = items[it];
        const AdamTensor t = tensors[item.tensor];
        a.weight_decay = t.weight_decay;
        const size_t end = min(t.count, item.first + kItemValues);
        // Tensors start 16-byte aligned and items start at multiples of 8,192 values.
        const size_t quads = (end - item.first) / 4;
        float4* p4 = reinterpret_cast<float4*>(t.param + item.first);
        float4* m4 = reinterpret_cast<float4*>(t.m + item.first);
        float4* v4 = reinterpret_cast<float4*>(t.v + item.first);
        const float4* g4 = reinterpret_cast<const float4*>(t.grad + item.first);
        uint2* h4 = t.half_copy == nullptr ? nullptr
                                           : reinterpret_cast<uint2*>(t.half_copy + item.first);
        for (size_t i = threadIdx.x; i < quads; i += kThreads) {
            float4 p = p4[i];
            float4 mm = m4[i];
            float4 vv = v4[i];
            const float4 g = g4[i];
            adam_one(p.x, mm.x, vv.x, g.x, a);
            adam_one(p.y, mm.y, vv.y, g.y, a);
            adam_one(p.z, mm.z, vv.z, g.z, a);
            adam_one(p.w, mm.w, vv.w, g.w, a);
            p4[i] = p;
            m4[i] = mm;
            v4[i] = vv;
            if (h4 != nullptr) {
                h4[i] = make_uint2(fb::pack2(p.x, p.y), fb::pack2(p.z, p.w));
            }
        }
        const size_t tail = item.first + quads * 4;
        if (threadIdx.x < end - tail) {
            const size_t i = tail + threadIdx.x;
            adam_one(t.param[i], t.m[i], t.v[i], t.grad[i], a);
            if (t.half_copy != nullptr) {
                t.half_copy[i] = __float2half_rn(t.param[i]);
            }
        }
    }
}

size_t plan_items(const flint_b200_adamw_tensor* tensors, size_t count) {
    size_t items = 0;
    for (size_t i = 0; i < count; ++i) {
        items += (tensors[i].count + kItemValues - 1) / kItemValues;
    }
    return items;
}

flint_status check_hyper(const char* name, float lr, float beta1, float beta2, float eps,
                         float grad_scale, int step) {
    if (step < 1) {
        return fb::fail(kInvalid, "%s: step (%d) must be at least 1", name, step);
    }
    if (!std::isfinite(lr) || !std::isfinite(grad_scale) || !(beta1 >= 0.0f && beta1 < 1.0f) ||
        !(beta2 >= 0.0f && beta2 < 1.0f) || !(eps >= 0.0f)) {
        return fb::fail(kInvalid, "%s: hyper-parameters must be finite, with betas in [0, 1)",
                        name);
    }
    return FLINT_OK;
}

AdamArgs make_args(float lr, float beta1, float beta2, float eps, float weight_decay,
                   float grad_scale, int step) {
    AdamArgs a;
    a.lr = lr;
    a.beta1 = beta1;
    a.beta2 = beta2;
    a.eps = eps;
    a.weight_decay = weight_decay;
    a.grad_scale = grad_scale;
    a.correction1 = static_cast<float>(1.0 - std::pow(static_cast<double>(beta1), step));
    a.correction2 = static_cast<float>(1.0 - std::pow(static_cast<double>(beta2), step));
    return a;
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
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_b200_adamw_plan_bytes(const flint_b200_adamw_tensor* tensors, size_t count,
                                         size_t* bytes) {
    constexpr const char* name = "flint_b200_adamw_plan_bytes";
    if (tensors == nullptr || bytes == nullptr) {
        return fb::fail(kInvalid, "%s: tensors and bytes must not be null", name);
    }
    *bytes = sizeof(AdamPlanHeader) + count * sizeof(AdamTensor) +
             plan_items(tensors, count) * sizeof(AdamItem);
    return FLINT_OK;
}

flint_status flint_b200_adamw_plan(void* plan, size_t plan_bytes,
                                   const flint_b200_adamw_tensor* tensors, size_t count,
                                   flint_stream stream) {
    constexpr const char* name = "flint_b200_adamw_plan";
    if (plan == nullptr || tensors == nullptr) {
        return fb::fail(kInvalid, "%s: plan and tensors must not be null", name);
    }
    if (!fb::aligned16(plan)) {
        return fb::fail(kInvalid, "%s: plan is not 16-byte aligned", name);
    }
    const size_t items = plan_items(tensors, count);
    const size_t needed =
        sizeof(AdamPlanHeader) + count * sizeof(AdamTensor) + items * sizeof(AdamItem);
    if (plan_bytes < needed) {
        return fb::fail(kInvalid, "%s: needs %zu bytes, given %zu", name, needed, plan_bytes);
    }
    std::vector<unsigned char> host(needed);
    AdamPlanHeader header;
    header.tensors = count;
    header.items = items;
    header.tensor_offset = sizeof(AdamPlanHeader);
    header.item_offset = header.tensor_offset + count * sizeof(AdamTensor);
    std::memcpy(host.data(), &header, sizeof header);
    auto* out_tensors = reinterpret_cast<AdamTensor*>(host.data() + header.tensor_offset);
    auto* out_items = reinterpret_cast<AdamItem*>(host.data() + header.item_offset);
    size_t at = 0;
    for (size_t i = 0; i < count; ++i) {
        const flint_b200_adamw_tensor& t = tensors[i];
        if (t.param == nullptr || t.m == nullptr || t.v == nullptr || t.grad == nullptr) {
            return fb::fail(kInvalid, "%s: tensor %zu has a null pointer", name, i);
        }
        if (!fb::aligned16(t.param) || !fb::aligned16(t.m) || !fb::aligned16(t.v) ||
            !fb::aligned16(t.grad) || !fb::aligned16(t.half_copy)) {
            return fb::fail(kInvalid, "%s: tensor %zu is not 16-byte aligned", name, i);
        }
        out_tensors[i] = AdamTensor{static_cast<float*>(t.param),
                                    static_cast<float*>(t.m),
                                    static_cast<float*>(t.v),
                                    static_cast<const float*>(t.grad),
                                    static_cast<__half*>(t.half_copy),
                                    t.count,
                                    t.weight_decay,
                                    0.0f};
        for (size_t first = 0; first < t.count; first += kItemValues) {
            out_items[at++] = AdamItem{static_cast<unsigned>(i), 0u, first};
        }
    }
    // A pageable source: the copy is staged before the call returns.
    FB_CUDA(cudaMemcpyAsync(plan, host.data(), needed, cudaMemcpyHostToDevice, stream));
    FB_CUDA(cudaStreamSynchronize(stream));
    return FLINT_OK;
}

flint_status flint_b200_adamw_run(const void* plan, size_t items, float lr, float beta1,
                                  float beta2, float eps, float grad_scale, int step,
                                  const int* skip, flint_stream stream) {
    constexpr const char* name = "flint_b200_adamw_run";
    if (plan == nullptr) {
        return fb::fail(kInvalid, "%s: plan is null", name);
    }
    FB_TRY(check_hyper(name, lr, beta1, beta2, eps, grad_scale, step));
    if (items == 0) {
        return FLINT_OK;
    }
    int sms = 148;
    FB_CUDA(fb::sm_count(&sms));
    const unsigned grid = static_cast<unsigned>(std::min<size_t>(items, size_t(sms) * 16));
    fb_adamw_multi<<<grid, kThreads, 0, stream>>>(
        static_cast<const unsigned char*>(plan),
        make_args(lr, beta1, beta2, eps, 0.0f, grad_scale, step), skip);
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_b200_adamw_plan_items(const flint_b200_adamw_tensor* tensors, size_t count,
                                         size_t* items) {
    if (tensors == nullptr || items == nullptr) {
        return fb::fail(kInvalid, "flint_b200_adamw_plan_items: tensors and items must not be null");
    }
    *items = plan_items(tensors, count);
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
    FB_CUDA(fb::after_launch());
    return FLINT_OK;
}

flint_status flint_b200_launch_count(unsigned long long* launches) {
    if (launches == nullptr) {
        return fb::fail(kInvalid, "flint_b200_launch_count: launches is null");
    }
    *launches = fb::launch_count();
    return FLINT_OK;
}

flint_status flint_b200_kernel_fault(int* raised) {
    if (raised == nullptr) {
        return fb::fail(kInvalid, "flint_b200_kernel_fault: raised is null");
    }
    int gemm = 0;
    int attention = 0;
    FB_CUDA(fb::gemm_error_flag(&gemm, true));
    FB_CUDA(fb::attention_error_flag(&attention, true));
    int reductions = 0;
    FB_CUDA(fb::reductions_error_flag(&reductions, true));
    int rowwise = 0;
    FB_CUDA(fb::rowwise_error_flag(&rowwise, true));
    *raised = (gemm != 0 || attention != 0 || reductions != 0 || rowwise != 0) ? 1 : 0;
    return FLINT_OK;
}

}  // extern "C"
