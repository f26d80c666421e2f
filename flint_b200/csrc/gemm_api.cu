// C ABI of the GEMM family: argument validation in the order, and with the
// message texts, of the reference's src/api/gemm.cpp:27-454, then a launch of
// the tensor-core kernel.
#include <cmath>

#include "common.h"
#include "gemm.h"

namespace {

using fb::aligned16;
using fb::fail;
using fb::fits;
using fb::overlap;

constexpr size_t kMaxMN = size_t{65535} * 128;  // 8,388,480
constexpr size_t kMaxK = size_t{1} << 16;
constexpr size_t kMaxBatches = 65535;
constexpr size_t kBatchedMaxM = 1024;
constexpr flint_status kInvalid = FLINT_ERROR_INVALID_ARGUMENT;

const char* first_of(bool a, bool b) { return a ? "y" : b ? "x" : "w"; }

// Shared by NT and NN (m, n > 0). y_element is 2 (FP16) or 4 (residual form).
flint_status check_nt_nn(const char* name, bool n_chunked, const void* y, const void* x,
                         const void* w, size_t m, size_t n, size_t k, size_t y_element = 2) {
    if (k == 0 || k % 8 != 0) {
        return fail(kInvalid, "%s: k (%zu) must be a positive multiple of 8", name, k);
    }
    if (n_chunked && n % 8 != 0) {
        return fail(kInvalid, "%s: n (%zu) must be a multiple of 8", name, n);
    }
    if (m > kMaxMN || n > kMaxMN || k > kMaxK) {
        return fail(kInvalid,
                    "%s: %zu x %zu x %zu is too large: m and n can be up to %zu, and k up to %zu",
                    name, m, n, k, kMaxMN, kMaxK);
    }
    if (y == nullptr || x == nullptr || w == nullptr) {
        return fail(kInvalid, "%s: %s is null", name, first_of(y == nullptr, x == nullptr));
    }
    if (!aligned16(y) || !aligned16(x) || !aligned16(w)) {
        return fail(kInvalid, "%s: %s is not 16-byte aligned", name,
                    first_of(!aligned16(y), !aligned16(x)));
    }
    const size_t yb = m * n * y_element;
    const size_t xb = m * k * 2;
    const size_t wb = n * k * 2;
    if (!fits(y, yb) || !fits(x, xb) || !fits(w, wb)) {
        return fail(kInvalid, "%s: %s runs past the end of the address space", name,
                    first_of(!fits(y, yb), !fits(x, xb)));
    }
    if (overlap(y, yb, x, xb)) {
        return fail(kInvalid, "%s: y and x overlap", name);
    }
    if (overlap(y, yb, w, wb)) {
        return fail(kInvalid, "%s: y and w overlap", name);
    }
    return FLINT_OK;
}

// An extra operand (bias, pre, residual) checked after the main three:
// null, alignment, fit, overlap with y.
flint_status check_extra(const char* name, const char* what, const void* y, size_t y_bytes,
                         const void* extra, size_t extra_bytes) {
    if (extra == nullptr) {
        return fail(kInvalid, "%s: %s is null", name, what);
    }
    if (!aligned16(extra)) {
        return fail(kInvalid, "%s: %s is not 16-byte aligned", name, what);
    }
    if (!fits(extra, extra_bytes)) {
        return fail(kInvalid, "%s: %s runs past the end of the address space", name, what);
    }
    if (overlap(y, y_bytes, extra, extra_bytes)) {
        return fail(kInvalid, "%s: y and %s overlap", name, what);
    }
    return FLINT_OK;
}

flint_status check_tn_dims(const char* name, size_t m, size_t n, size_t k) {
    if (k == 0) {
        return fail(kInvalid, "%s: k must be positive", name);
    }
    if (m % 8 != 0 || n % 8 != 0) {
        return fail(kInvalid, "%s: %s (%zu) must be a multiple of 8", name,
                    m % 8 != 0 ? "m" : "n", m % 8 != 0 ? m : n);
    }
    if (m > kMaxMN || n > kMaxMN || k > kMaxK) {
        return fail(kInvalid,
                    "%s: %zu x %zu x %zu is too large: m and n can be up to %zu, and k up to %zu",
                    name, m, n, k, kMaxMN, kMaxK);
    }
    return FLINT_OK;
}

flint_status check_batched_nt_nn(const char* name, bool n_chunked, size_t n, size_t k) {
    if (k == 0 || k % 8 != 0) {
        return fail(kInvalid, "%s: k (%zu) must be a positive multiple of 8", name, k);
    }
    if (n_chunked && n % 8 != 0) {
        return fail(kInvalid, "%s: n (%zu) must be a multiple of 8", name, n);
    }
    if (n > kMaxMN || k > kMaxK) {
        return fail(kInvalid, "%s: n (%zu) can be up to %zu, and k (%zu) up to %zu", name, n,
                    kMaxMN, k, kMaxK);
    }
    return FLINT_OK;
}

flint_status check_batched(const char* name, void* y, const void* x, const void* w,
                           size_t batches, size_t m, size_t n, size_t k) {
    if (batches > kMaxBatches) {
        return fail(kInvalid, "%s: batches (%zu) can be up to %zu", name, batches, kMaxBatches);
    }
    if (m > kBatchedMaxM) {
        return fail(kInvalid, "%s: m (%zu) can be up to %zu", name, m, kBatchedMaxM);
    }
    const fb::Span spans[] = {
        {"y", y, batches * m * n * 2},
        {"x", x, batches * m * k * 2},
        {"w", w, batches * n * k * 2},
    };
    return fb::check_spans(name, spans, 1);
}

cudaError_t tn_workspace_bytes(size_t m, size_t n, size_t k, size_t* bytes) {
    int sms = 0;
    const cudaError_t e = fb::sm_count(&sms);
    if (e != cudaSuccess) {
        return e;
    }
    const fb::TnSplit s = fb::tn_split(m, n, k, sms);
    *bytes = s.count > 1 ? static_cast<size_t>(s.count) * m * n * 4 : 0;
    return cudaSuccess;
}

}  // namespace

extern "C" {

flint_status flint_gemm_nt(void* y, const void* x, const void* w, size_t m, size_t n, size_t k,
                           flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    FB_TRY(check_nt_nn("flint_gemm_nt", false, y, x, w, m, n, k));
    FB_CUDA(fb::gemm_nt(fb::Epilogue::kNone, y, nullptr, x, w, nullptr, nullptr, m, n, k, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nt_bias(void* y, const void* x, const void* w, const void* bias, size_t m,
                                size_t n, size_t k, flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nt_bias";
    FB_TRY(check_nt_nn(name, false, y, x, w, m, n, k));
    FB_TRY(check_extra(name, "bias", y, m * n * 2, bias, n * 4));
    FB_CUDA(fb::gemm_nt(fb::Epilogue::kBias, y, nullptr, x, w, bias, nullptr, m, n, k, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nt_bias_gelu(void* y, void* pre, const void* x, const void* w,
                                     const void* bias, size_t m, size_t n, size_t k,
                                     flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nt_bias_gelu";
    FB_TRY(check_nt_nn(name, false, y, x, w, m, n, k));
    FB_TRY(check_extra(name, "bias", y, m * n * 2, bias, n * 4));
    FB_TRY(check_extra(name, "pre", y, m * n * 2, pre, m * n * 2));
    const size_t pre_bytes = m * n * 2;
    if (overlap(pre, pre_bytes, x, m * k * 2)) {
        return fail(kInvalid, "%s: pre and x overlap", name);
    }
    if (overlap(pre, pre_bytes, w, n * k * 2)) {
        return fail(kInvalid, "%s: pre and w overlap", name);
    }
    if (overlap(pre, pre_bytes, bias, n * 4)) {
        return fail(kInvalid, "%s: pre and bias overlap", name);
    }
    FB_CUDA(fb::gemm_nt(fb::Epilogue::kBiasGelu, y, pre, x, w, bias, nullptr, m, n, k, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nt_bias_residual(void* y, const void* x, const void* w, const void* bias,
                                         const void* residual, size_t m, size_t n, size_t k,
                                         flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nt_bias_residual";
    FB_TRY(check_nt_nn(name, false, y, x, w, m, n, k, 4));
    if (n % 2 != 0) {
        return fail(kInvalid, "%s: n (%zu) must be even", name, n);
    }
    FB_TRY(check_extra(name, "bias", y, m * n * 4, bias, n * 4));
    FB_TRY(check_extra(name, "residual", y, m * n * 4, residual, m * n * 4));
    FB_CUDA(fb::gemm_nt(fb::Epilogue::kBiasResidual, y, nullptr, x, w, bias, residual, m, n, k,
                        stream));
    return FLINT_OK;
}

flint_status flint_gemm_nn(void* y, const void* x, const void* w, size_t m, size_t n, size_t k,
                           flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    FB_TRY(check_nt_nn("flint_gemm_nn", true, y, x, w, m, n, k));
    FB_CUDA(fb::gemm_nn(fb::Epilogue::kNone, y, x, w, nullptr, m, n, k, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nn_dgelu(void* y, const void* x, const void* w, const void* pre, size_t m,
                                 size_t n, size_t k, flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nn_dgelu";
    FB_TRY(check_nt_nn(name, true, y, x, w, m, n, k));
    FB_TRY(check_extra(name, "pre", y, m * n * 2, pre, m * n * 2));
    FB_CUDA(fb::gemm_nn(fb::Epilogue::kDGelu, y, x, w, pre, m, n, k, stream));
    return FLINT_OK;
}

flint_status flint_gemm_tn_workspace(size_t m, size_t n, size_t k, size_t* bytes) {
    if (bytes == nullptr) {
        return fail(kInvalid, "flint_gemm_tn_workspace: bytes is null");
    }
    *bytes = 0;
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    FB_TRY(check_tn_dims("flint_gemm_tn_workspace", m, n, k));
    FB_CUDA(tn_workspace_bytes(m, n, k, bytes));
    return FLINT_OK;
}

flint_status flint_gemm_tn(void* y, const void* x, const void* w, size_t m, size_t n, size_t k,
                           int accumulate, void* workspace, size_t workspace_bytes,
                           flint_stream stream) {
    if (m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_tn";
    FB_TRY(check_tn_dims(name, m, n, k));
    if (y == nullptr || x == nullptr || w == nullptr) {
        return fail(kInvalid, "%s: %s is null", name, first_of(y == nullptr, x == nullptr));
    }
    if (!aligned16(y) || !aligned16(x) || !aligned16(w)) {
        return fail(kInvalid, "%s: %s is not 16-byte aligned", name,
                    first_of(!aligned16(y), !aligned16(x)));
    }
    const size_t yb = m * n * 4;
    const size_t xb = k * m * 2;
    const size_t wb = k * n * 2;
    if (!fits(y, yb) || !fits(x, xb) || !fits(w, wb)) {
        return fail(kInvalid, "%s: %s runs past the end of the address space", name,
                    first_of(!fits(y, yb), !fits(x, xb)));
    }
    if (overlap(y, yb, x, xb)) {
        return fail(kInvalid, "%s: y and x overlap", name);
    }
    if (overlap(y, yb, w, wb)) {
        return fail(kInvalid, "%s: y and w overlap", name);
    }
    size_t needed = 0;
    FB_CUDA(tn_workspace_bytes(m, n, k, &needed));
    if (needed > 0) {
        if (workspace == nullptr || workspace_bytes < needed) {
            return fail(kInvalid, "%s: needs %zu bytes of workspace, given %zu", name, needed,
                        workspace == nullptr ? size_t{0} : workspace_bytes);
        }
        if (!aligned16(workspace)) {
            return fail(kInvalid, "%s: workspace is not 16-byte aligned", name);
        }
        if (!fits(workspace, needed)) {
            return fail(kInvalid, "%s: workspace runs past the end of the address space", name);
        }
        if (overlap(workspace, needed, y, yb) || overlap(workspace, needed, x, xb) ||
            overlap(workspace, needed, w, wb)) {
            return fail(kInvalid, "%s: workspace overlaps y, x or w", name);
        }
    }
    FB_CUDA(fb::gemm_tn(y, x, w, m, n, k, accumulate != 0, workspace, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nt_batched(void* y, const void* x, const void* w, size_t batches, size_t m,
                                   size_t n, size_t k, float scale, flint_stream stream) {
    if (batches == 0 || m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nt_batched";
    FB_TRY(check_batched_nt_nn(name, false, n, k));
    if (!std::isfinite(scale)) {
        return fail(kInvalid, "%s: scale (%g) must be finite", name, static_cast<double>(scale));
    }
    FB_TRY(check_batched(name, y, x, w, batches, m, n, k));
    FB_CUDA(fb::gemm_batched(fb::Layout::kNT, y, x, w, batches, m, n, k, scale, stream));
    return FLINT_OK;
}

flint_status flint_gemm_nn_batched(void* y, const void* x, const void* w, size_t batches, size_t m,
                                   size_t n, size_t k, flint_stream stream) {
    if (batches == 0 || m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_nn_batched";
    FB_TRY(check_batched_nt_nn(name, true, n, k));
    FB_TRY(check_batched(name, y, x, w, batches, m, n, k));
    FB_CUDA(fb::gemm_batched(fb::Layout::kNN, y, x, w, batches, m, n, k, 1.0f, stream));
    return FLINT_OK;
}

flint_status flint_gemm_tn_batched(void* y, const void* x, const void* w, size_t batches, size_t m,
                                   size_t n, size_t k, flint_stream stream) {
    if (batches == 0 || m == 0 || n == 0) {
        return FLINT_OK;
    }
    constexpr const char* name = "flint_gemm_tn_batched";
    FB_TRY(check_tn_dims(name, m, n, k));
    FB_TRY(check_batched(name, y, x, w, batches, m, n, k));
    FB_CUDA(fb::gemm_batched(fb::Layout::kTN, y, x, w, batches, m, n, k, 1.0f, stream));
    return FLINT_OK;
}

}  // extern "C"
