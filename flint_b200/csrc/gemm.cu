// FP16 x FP16 -> FP32-accumulate GEMMs on the 5th-generation tensor cores:
// flint_gemm_nt / _nt_bias / _nt_bias_gelu / _nt_bias_residual / _nn / _nn_dgelu /
// _tn (+ workspace query) and the three batched forms.
//
// One persistent, warp-specialised kernel template serves every layout and
// epilogue:
//   warp 0      TMA producer: 128-byte-swizzled operand tiles into a shared
//               memory ring, one mbarrier per stage
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16)
//               from shared-memory descriptors into a tensor-memory accumulator;
//               tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-9   epilogue: tcgen05.ld of the FP32 accumulators, the fused
//               epilogue in registers, predicated global stores
// Tensor memory holds two accumulators, so the epilogue of tile i overlaps the
// main loop of tile i+1. Every k-block is 64 wide for every layout, so all
// variants of a shape add their products in the same order and the batched
// forms reproduce the plain ones bit for bit.
//
// Operand layouts map onto UMMA "major-ness" instead of register transposes:
// NT reads both operands K-major, NN reads w (k x n) MN-major, TN reads both x
// (k x m) and w (k x n) MN-major. Ragged edges come from TMA's zero fill.
//
// Reference behaviour: src/kernels/gemm.cu:419-587 (main loop and epilogues),
// :733-784 (split rule) and src/api/gemm.cpp:27-454 (checks and messages).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include <cuda.h>
#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"
#include "gemm.h"
#include "sm100.cuh"

namespace fb {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kEpilogueWarps = 8;  // two per TMEM lane quadrant, alternating 32-column chunks
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kRingBytes = 192 * 1024;
constexpr int kGroupM = 8;  // rows of tiles handed out together, for L2 reuse

// Set by a kernel whose bounded wait ran out; read by flint_b200_gemm_error().
__device__ int g_gemm_error = 0;

struct GemmParams {
    CUtensorMap map_a;
    CUtensorMap map_b;
    CUtensorMap map_y;    // FP16 outputs of the pair kernel leave through TMA stores
    CUtensorMap map_pre;  // bias+GELU: the pre-activation output
    int tma_out;          // the two maps above are valid
    void* y;
    void* aux_out;        // bias+GELU: the pre-activation output
    const void* aux_in;   // dGELU: pre-activations; residual: the FP32 residual
    const float* bias;
    float* partials;      // split TN: [split][m][n] FP32
    int m, n, k;
    int batches;          // 1 for the plain forms
    int splits;           // TN only
    int split_len;        // k per split, a multiple of 64
    int tiles_m, tiles_n;
    long long tiles_total;
    float scale;
    int accumulate;
    int batched;
};

// ---- epilogue math ----------------------------------------------------------------

// 2^x on the special-function unit (relative error about 2^-22; flushes denormals).
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// GPT-2's tanh GELU written as x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3):
// the same function without the cancellation of 1 + tanh(u) for negative x.
// e = exp(-2u) is taken as 2^(-2u log2 e) in one special-function instruction:
// its error (a few FP32 ulps) is three orders below the FP16 result's rounding.
// Two values at a time on the packed FP32 instructions; the scalar forms below
// run the same instructions, so every path gives the same bits.
__device__ __forceinline__ fb::F2 gelu_tanh2(fb::F2 x) {
    constexpr float kScale = -2.302208198144325f;  // -2 sqrt(2/pi) log2(e)
    const fb::F2 one = fb::f2_pack(1.0f, 1.0f);
    const fb::F2 t = fb::f2_fma(fb::f2_pack(0.044715f, 0.044715f), fb::f2_mul(x, x), one);
    const fb::F2 arg = fb::f2_mul(fb::f2_mul(fb::f2_pack(kScale, kScale), x), t);
    float a0, a1;
    fb::f2_unpack(arg, a0, a1);
    const fb::F2 d = fb::f2_add(fb::f2_pack(exp2_fast(a0), exp2_fast(a1)), one);
    float d0, d1;
    fb::f2_unpack(d, d0, d1);
    return fb::f2_mul(x, fb::f2_pack(rcp_fast(d0), rcp_fast(d1)));
}

__device__ __forceinline__ float gelu_tanh(float x) {
    float lo, hi;
    fb::f2_unpack(gelu_tanh2(fb::f2_pack(x, x)), lo, hi);
    return lo;
}

// d/dx of the above: s + x s (1 - s) * 2u', s = sigmoid(2u). For x >= 0,
// 1 - s is computed as e * s to keep its relative accuracy near s = 1.
__device__ __forceinline__ fb::F2 gelu_tanh_grad2(fb::F2 x) {
    constexpr float kScale = -2.302208198144325f;
    constexpr float k2Rt2OverPi = 1.5957691216057308f;
    constexpr float k6KappaRt2OverPi = 0.21406444946504453f;  // 2 sqrt(2/pi) * 3 * 0.044715
    const fb::F2 one = fb::f2_pack(1.0f, 1.0f);
    const fb::F2 x2 = fb::f2_mul(x, x);
    const fb::F2 t = fb::f2_fma(fb::f2_pack(0.044715f, 0.044715f), x2, one);
    const fb::F2 arg = fb::f2_mul(fb::f2_mul(fb::f2_pack(kScale, kScale), x), t);
    float a0, a1, x0, x1;
    fb::f2_unpack(arg, a0, a1);
    fb::f2_unpack(x, x0, x1);
    const fb::F2 e = fb::f2_pack(exp2_fast(a0), exp2_fast(a1));
    float d0, d1;
    fb::f2_unpack(fb::f2_add(e, one), d0, d1);
    const fb::F2 s = fb::f2_pack(rcp_fast(d0), rcp_fast(d1));
    float n0, n1, p0, p1;
    fb::f2_unpack(fb::f2_sub(one, s), n0, n1);  // 1 - s, accurate for x < 0
    fb::f2_unpack(fb::f2_mul(e, s), p0, p1);    // e s,   accurate for x >= 0
    const fb::F2 one_minus_s = fb::f2_pack(x0 < 0.0f ? n0 : p0, x1 < 0.0f ? n1 : p1);
    const fb::F2 slope = fb::f2_fma(fb::f2_pack(k6KappaRt2OverPi, k6KappaRt2OverPi), x2,
                                    fb::f2_pack(k2Rt2OverPi, k2Rt2OverPi));
    const fb::F2 q = fb::f2_mul(fb::f2_mul(x, one_minus_s), slope);
    float g0, g1;
    fb::f2_unpack(fb::f2_fma(s, q, s), g0, g1);
    g0 = isinf(x0) ? (x0 > 0.0f ? 1.0f : 0.0f) : g0;
    g1 = isinf(x1) ? (x1 > 0.0f ? 1.0f : 0.0f) : g1;
    return fb::f2_pack(g0, g1);
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
    float lo, hi;
    fb::f2_unpack(gelu_tanh_grad2(fb::f2_pack(x, x)), lo, hi);
    return lo;
}

__device__ __forceinline__ float half_bits_to_float(unsigned short h) {
    return __half2float(__ushort_as_half(h));
}

// One output row segment: 32 consecutive columns starting at `col` of row
// `row`, FP32 accumulators in acc. `valid` = how many of the 32 columns lie
// inside the matrix.
template <Epilogue E>
__device__ __forceinline__ void store_segment(const GemmParams& p, size_t batch_offset,
                                              long long split, size_t row, int col,
                                              float (&acc)[32], int valid) {
    const size_t n = static_cast<size_t>(p.n);
    const size_t at = batch_offset + row * n + col;
    if constexpr (E == Epilogue::kBias || E == Epilogue::kBiasGelu ||
                  E == Epilogue::kBiasResidual) {
        const float* bias = p.bias + col;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (j < valid) {
                acc[j] = __fadd_rn(acc[j], bias[j]);
            }
        }
    }
    if constexpr (E == Epilogue::kScale) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            acc[j] = __fmul_rn(acc[j], p.scale);
        }
    }
    if constexpr (E == Epilogue::kDGelu) {
        const __half* pre = static_cast<const __half*>(p.aux_in) + at;
        // NN's n is a multiple of 8, so 8-column groups are whole and 16-byte aligned.
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (g * 8 < valid) {
                const uint4 q = *reinterpret_cast<const uint4*>(pre + g * 8);
                const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = half_bits_to_float(static_cast<unsigned short>(w[j]));
                    const float hi = half_bits_to_float(static_cast<unsigned short>(w[j] >> 16));
                    acc[g * 8 + 2 * j] = __fmul_rn(acc[g * 8 + 2 * j], gelu_tanh_grad(lo));
                    acc[g * 8 + 2 * j + 1] = __fmul_rn(acc[g * 8 + 2 * j + 1], gelu_tanh_grad(hi));
                }
            }
        }
    }

    if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore ||
                  E == Epilogue::kTnPartial) {
        // FP32 outputs.
        float* out;
        if constexpr (E == Epilogue::kTnPartial) {
            out = p.partials + static_cast<size_t>(split) * p.m * n + row * n + col;
        } else {
            out = static_cast<float*>(p.y) + at;
        }
        const float* res = E == Epilogue::kBiasResidual
                               ? static_cast<const float*>(p.aux_in) + at
                               : out;
        const bool add = E == Epilogue::kBiasResidual || (E == Epilogue::kTnStore && p.accumulate);
        if (p.n % 4 == 0) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g * 4 < valid) {
                    float4 v = make_float4(acc[4 * g], acc[4 * g + 1], acc[4 * g + 2],
                                           acc[4 * g + 3]);
                    if (add) {
                        const float4 o = *reinterpret_cast<const float4*>(res + 4 * g);
                        v = make_float4(__fadd_rn(o.x, v.x), __fadd_rn(o.y, v.y),
                                        __fadd_rn(o.z, v.z), __fadd_rn(o.w, v.w));
                    }
                    *reinterpret_cast<float4*>(out + 4 * g) = v;
                }
            }
        } else {
            // n even (the residual form's only requirement): 8-byte pairs.
#pragma unroll
            for (int g = 0; g < 16; ++g) {
                if (g * 2 < valid) {
                    float2 v = make_float2(acc[2 * g], acc[2 * g + 1]);
                    if (add) {
                        const float2 o = *reinterpret_cast<const float2*>(res + 2 * g);
                        v = make_float2(__fadd_rn(o.x, v.x), __fadd_rn(o.y, v.y));
                    }
                    *reinterpret_cast<float2*>(out + 2 * g) = v;
                }
            }
        }
        return;
    } else {
        // FP16 outputs; the GELU form writes the pre-activation too.
        __half* out = static_cast<__half*>(p.y) + at;
        __half* pre_out = nullptr;
        if constexpr (E == Epilogue::kBiasGelu) {
            pre_out = static_cast<__half*>(p.aux_out) + at;
        }
        if (p.n % 8 == 0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (g * 8 < valid) {
                    uint4 q;
                    unsigned* w = reinterpret_cast<unsigned*>(&q);
                    if constexpr (E == Epilogue::kBiasGelu) {
                        uint4 qp;
                        unsigned* wp = reinterpret_cast<unsigned*>(&qp);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float a = acc[g * 8 + 2 * j];
                            const float b = acc[g * 8 + 2 * j + 1];
                            const __half2 hp = __floats2half2_rn(a, b);
                            const __half2 hy = __floats2half2_rn(gelu_tanh(a), gelu_tanh(b));
                            wp[j] = *reinterpret_cast<const unsigned*>(&hp);
                            w[j] = *reinterpret_cast<const unsigned*>(&hy);
                        }
                        *reinterpret_cast<uint4*>(pre_out + g * 8) = qp;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const __half2 h =
                                __floats2half2_rn(acc[g * 8 + 2 * j], acc[g * 8 + 2 * j + 1]);
                            w[j] = *reinterpret_cast<const unsigned*>(&h);
                        }
                    }
                    *reinterpret_cast<uint4*>(out + g * 8) = q;
                }
            }
        } else {
            // Any n (NT allows odd n): rows are only 2-byte aligned.
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < valid) {
                    if constexpr (E == Epilogue::kBiasGelu) {
                        pre_out[j] = __float2half_rn(acc[j]);
                        out[j] = __float2half_rn(gelu_tanh(acc[j]));
                    } else {
                        out[j] = __float2half_rn(acc[j]);
                    }
                }
            }
        }
    }
}

// ---- coalesced epilogue ------------------------------------------------------------------
//
// After tcgen05.ld each lane holds 32 consecutive columns of its own row, so a
// direct store touches 32 rows per instruction. Instead the warp stages its
// 32 x 32 chunk in a private 4 KB shared-memory buffer (16-byte slots, swizzled
// in groups of 8 so both directions are conflict-free) and reads it back so
// that consecutive lanes hold consecutive 16-byte pieces of a row: every global
// access then covers whole 64- or 128-byte row segments. Second operands (the
// saved pre-activation, the residual, the old value when accumulating) are
// fetched in the same coalesced layout.

__device__ __forceinline__ uint32_t stage_slot(uint32_t base, int logical) {
    return base + static_cast<uint32_t>(((logical & ~7) | ((logical & 7) ^ ((logical >> 3) & 7)))
                                        << 4);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint4 pack_half8(const float* v) {
    uint4 q;
    unsigned* w = reinterpret_cast<unsigned*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<const unsigned*>(&h);
    }
    return q;
}

// FP16 chunks that leave by a TMA store are staged row-major, 64 bytes per row, in
// the tensor map's 64-byte swizzle (16-byte piece c of row r at c ^ ((r >> 1) & 3)):
// lane = row stores are conflict-free and the copy engine undoes the swizzle. The
// store is asynchronous: the warp goes on to its next chunk and only waits, before it
// overwrites the slot, for the engine to have read it.
__device__ __forceinline__ void stage_row_for_store(uint32_t slot, int row, const float* v) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        st_shared_v4(slot + row * 64 + ((c ^ ((row >> 1) & 3)) << 4), pack_half8(v + 8 * c));
    }
}

__device__ __forceinline__ void store_wait_slots_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// One lane: the staged 32 x 32 chunk to rows [row, row + 32), columns [col, col + 32);
// parts outside the matrix are clipped by the copy engine.
__device__ __forceinline__ void store_chunk_async(const CUtensorMap* map, uint32_t slot, int col,
                                                  int row) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(slot), "r"(col), "r"(row)
        : "memory");
}

// Moves the warp's staged FP16 chunk (4 slots per row) to `out` (row-major, ld = n).
__device__ __forceinline__ void flush_half_chunk(uint32_t stage, __half* out_chunk, size_t n,
                                                 int rows_left, int valid, int lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int logical = lane + 32 * i;
        const int r = logical >> 2;
        const int c = logical & 3;
        if (r < rows_left && c * 8 < valid) {
            *reinterpret_cast<uint4*>(out_chunk + static_cast<size_t>(r) * n + c * 8) =
                ld_shared_v4(stage_slot(stage, logical));
        }
    }
}

// Second operands of a chunk, fetched in the coalesced layout before the
// accumulators are needed: the residual (bias+residual), the old value (TN
// store with accumulate) or the saved pre-activation (dGELU). The loads are
// issued a chunk ahead of their use, so their latency hides behind the previous
// chunk's work instead of stalling every store.
template <Epilogue E>
__host__ __device__ constexpr int aux_slots() {
    return (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore) ? 8
           : E == Epilogue::kDGelu                                   ? 4
                                                                      : 1;
}

template <Epilogue E>
struct Aux {
    uint4 q[aux_slots<E>()];
};

template <Epilogue E>
__device__ __forceinline__ void load_aux(Aux<E>& aux, const GemmParams& p, size_t batch_offset,
                                         size_t row0, int col, int valid, int lane) {
    const size_t n = static_cast<size_t>(p.n);
    const size_t at0 = batch_offset + row0 * n + col;
    const long long rows_long = static_cast<long long>(p.m) - static_cast<long long>(row0);
    const int rows_left = rows_long > 32 ? 32 : static_cast<int>(rows_long);
    if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore) {
        const bool add = E == Epilogue::kBiasResidual || p.accumulate;
        const float* old = E == Epilogue::kBiasResidual
                               ? static_cast<const float*>(p.aux_in) + at0
                               : static_cast<const float*>(p.y) + at0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int logical = lane + 32 * i;
            const int r = logical >> 3;
            const int c = logical & 7;
            aux.q[i] = make_uint4(0u, 0u, 0u, 0u);
            if (add && r < rows_left && c * 4 < valid) {
                aux.q[i] = *reinterpret_cast<const uint4*>(old + static_cast<size_t>(r) * n + c * 4);
            }
        }
    } else if constexpr (E == Epilogue::kDGelu) {
        // Each lane fetches its own row's 64 bytes (two whole sectors), so the saved
        // pre-activations need no trip through shared memory.
        const __half* pre = static_cast<const __half*>(p.aux_in) + at0 + static_cast<size_t>(lane) * n;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            aux.q[i] = make_uint4(0u, 0u, 0u, 0u);
            if (lane < rows_left && i * 8 < valid) {
                aux.q[i] = *reinterpret_cast<const uint4*>(pre + i * 8);
            }
        }
    }
}

// This lane's bias value for a chunk starting at column `col` (0 for the other
// epilogues and past the last column).
template <Epilogue E>
__device__ __forceinline__ float load_bias_lane(const GemmParams& p, int col, int lane) {
    if constexpr (E == Epilogue::kBias || E == Epilogue::kBiasGelu ||
                  E == Epilogue::kBiasResidual) {
        return col + lane < p.n ? __ldg(p.bias + col + lane) : 0.0f;
    } else {
        return 0.0f;
    }
}

// The whole warp calls this for one 32 x 32 chunk whose top-left element is
// (row0, col). acc holds this lane's row. Requires n % 8 == 0 (FP16 outputs) or
// n % 4 == 0 (FP32 outputs).
template <Epilogue E>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t stage,
                                            size_t batch_offset, long long split, size_t row0,
                                            int col, float (&acc)[32], int valid, int lane,
                                            const Aux<E>& aux, float bias_lane) {
    const size_t n = static_cast<size_t>(p.n);
    const size_t at0 = batch_offset + row0 * n + col;  // the chunk's first element
    const long long rows_long = static_cast<long long>(p.m) - static_cast<long long>(row0);
    const int rows_left = rows_long > 32 ? 32 : static_cast<int>(rows_long);

    if constexpr (E == Epilogue::kBias || E == Epilogue::kBiasGelu ||
                  E == Epilogue::kBiasResidual) {
        // Lane j holds bias[col + j] (fetched by the caller a chunk ahead, zero past the
        // matrix's edge); every lane needs all 32, so they are passed round by shuffles
        // instead of each lane waiting on its own loads.
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            acc[j] = __fadd_rn(acc[j], __shfl_sync(0xffffffffu, bias_lane, j));
        }
    }
    if constexpr (E == Epilogue::kScale) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            acc[j] = __fmul_rn(acc[j], p.scale);
        }
    }

    if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore ||
                  E == Epilogue::kTnPartial) {
        // FP32 output: 8 slots per row.
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            st_shared_v4(stage_slot(stage, lane * 8 + c),
                         make_uint4(__float_as_uint(acc[4 * c]), __float_as_uint(acc[4 * c + 1]),
                                    __float_as_uint(acc[4 * c + 2]),
                                    __float_as_uint(acc[4 * c + 3])));
        }
        __syncwarp();
        float* out;
        if constexpr (E == Epilogue::kTnPartial) {
            out = p.partials + static_cast<size_t>(split) * p.m * n + row0 * n + col;
        } else {
            out = static_cast<float*>(p.y) + at0;
        }
        bool add = false;
        if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore) {
            add = E == Epilogue::kBiasResidual || p.accumulate;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int logical = lane + 32 * i;
            const int r = logical >> 3;
            const int c = logical & 7;
            if (r < rows_left && c * 4 < valid) {
                const uint4 q = ld_shared_v4(stage_slot(stage, logical));
                float4 v = make_float4(__uint_as_float(q.x), __uint_as_float(q.y),
                                       __uint_as_float(q.z), __uint_as_float(q.w));
                const size_t off = static_cast<size_t>(r) * n + c * 4;
                if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore) {
                    if (add) {
                        const uint4 o = aux.q[i];
                        v = make_float4(__fadd_rn(__uint_as_float(o.x), v.x),
                                        __fadd_rn(__uint_as_float(o.y), v.y),
                                        __fadd_rn(__uint_as_float(o.z), v.z),
                                        __fadd_rn(__uint_as_float(o.w), v.w));
                    }
                }
                *reinterpret_cast<float4*>(out + off) = v;
            }
        }
        __syncwarp();
        return;
    } else {
        __half* out = static_cast<__half*>(p.y) + at0;
        if constexpr (E == Epilogue::kDGelu) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 q = aux.q[c];
                const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = half_bits_to_float(static_cast<unsigned short>(w[j]));
                    const float hi = half_bits_to_float(static_cast<unsigned short>(w[j] >> 16));
                    float g0, g1;
                    fb::f2_unpack(gelu_tanh_grad2(fb::f2_pack(lo, hi)), g0, g1);
                    acc[c * 8 + 2 * j] = __fmul_rn(acc[c * 8 + 2 * j], g0);
                    acc[c * 8 + 2 * j + 1] = __fmul_rn(acc[c * 8 + 2 * j + 1], g1);
                }
            }
        }
        if (p.tma_out != 0) {
            // Asynchronous stores: wait until the copy engine has read what this slot held.
            if (lane == 0) {
                store_wait_slots_read();
            }
            __syncwarp();
            if constexpr (E == Epilogue::kBiasGelu) {
                stage_row_for_store(stage, lane, acc);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    fb::f2_unpack(gelu_tanh2(fb::f2_pack(acc[2 * j], acc[2 * j + 1])), acc[2 * j],
                                  acc[2 * j + 1]);
                }
                stage_row_for_store(stage + 2048u, lane, acc);
            } else {
                stage_row_for_store(stage, lane, acc);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if constexpr (E == Epilogue::kBiasGelu) {
                    store_chunk_async(&p.map_pre, stage, col, static_cast<int>(row0));
                    store_chunk_async(&p.map_y, stage + 2048u, col, static_cast<int>(row0));
                } else {
                    store_chunk_async(&p.map_y, stage, col, static_cast<int>(row0));
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            return;
        }
        if constexpr (E == Epilogue::kBiasGelu) {
            // The pre-activation goes to the slot's first half, GELU of the unrounded
            // sums to the second; one trip through shared memory serves both outputs.
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                st_shared_v4(stage_slot(stage, lane * 4 + c), pack_half8(acc + 8 * c));
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                fb::f2_unpack(gelu_tanh2(fb::f2_pack(acc[2 * j], acc[2 * j + 1])), acc[2 * j],
                              acc[2 * j + 1]);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                st_shared_v4(stage_slot(stage + 2048u, lane * 4 + c), pack_half8(acc + 8 * c));
            }
            __syncwarp();
            flush_half_chunk(stage, static_cast<__half*>(p.aux_out) + at0, n, rows_left, valid,
                             lane);
            flush_half_chunk(stage + 2048u, out, n, rows_left, valid, lane);
            __syncwarp();
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                st_shared_v4(stage_slot(stage, lane * 4 + c), pack_half8(acc + 8 * c));
            }
            __syncwarp();
            flush_half_chunk(stage, out, n, rows_left, valid, lane);
            __syncwarp();
        }
    }
}

template <Epilogue E>
__device__ __forceinline__ bool chunk_path_ok(const GemmParams& p) {
    if constexpr (E == Epilogue::kBiasResidual || E == Epilogue::kTnStore ||
                  E == Epilogue::kTnPartial) {
        return p.n % 4 == 0;
    } else {
        return p.n % 8 == 0;
    }
}

// ---- the tensor-core kernel --------------------------------------------------------------

template <int BN>
struct Ring {
    static constexpr int kStageA = kBM * kBK * 2;
    static constexpr int kStageB = BN * kBK * 2;
    static constexpr int kStage = kStageA + kStageB;
    static constexpr int kStages = kRingBytes / kStage;
    // ring + epilogue staging (4 KB per epilogue warp) + barriers + alignment slack
    static constexpr int kSmemBytes = kStages * kStage + kEpilogueWarps * 4096 + 1024 + 256;
};

struct TileCoord {
    long long z;  // batch (batched forms) or split (TN)
    int tm, tn;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, long long id) {
    const long long per = static_cast<long long>(p.tiles_m) * p.tiles_n;
    TileCoord c;
    c.z = id / per;
    const long long r = id - c.z * per;
    const long long group_span = static_cast<long long>(kGroupM) * p.tiles_n;
    const long long g = r / group_span;
    const int first_m = static_cast<int>(g) * kGroupM;
    const int rows_here = min(kGroupM, p.tiles_m - first_m);
    const long long in_group = r - g * group_span;
    c.tm = first_m + static_cast<int>(in_group % rows_here);
    c.tn = static_cast<int>(in_group / rows_here);
    return c;
}

template <Layout L, Epilogue E, int BN>
__global__ void __launch_bounds__(kThreads, 1)
    fb_gemm_tc(const __grid_constant__ GemmParams p) {
    using R = Ring<BN>;
    constexpr bool kAMn = L == Layout::kTN;
    constexpr bool kBMn = L != Layout::kNT;
    constexpr bool kIsTn = L == Layout::kTN;
    constexpr uint32_t kIdesc = sm100::instr_desc_f16(kBM, BN, kAMn, kBMn);
    constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging = smem_base + R::kStages * R::kStage;
    const uint32_t bars = staging + kEpilogueWarps * 4096;
    // barrier slots (8 bytes each): full[kStages], empty[kStages], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (R::kStages + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * R::kStages + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * R::kStages + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < R::kStages; ++s) {
            sm100::mbar_init(full_bar(s), 1);
            sm100::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            sm100::mbar_init(acc_full_bar(a), 1);
            sm100::mbar_init(acc_empty_bar(a), kEpilogueWarps);
        }
        sm100::mbar_fence_init();
        sm100::tma_prefetch_descriptor(&p.map_a);
        sm100::tma_prefetch_descriptor(&p.map_b);
    }
    if (warp == 1) {
        sm100::tmem_alloc(sm100::smem_u32(&tmem_base_slot), kTmemCols);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;
    // Everything above ran while the previous kernel in the stream may still have been
    // finishing; global memory is touched only from here on.
    fb::dependency_wait();
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long id = blockIdx.x; ok && id < p.tiles_total; id += gridDim.x) {
                const TileCoord t = decode_tile(p, id);
                const bool split_k = kIsTn && !p.batched;
                const int k0 = split_k ? static_cast<int>(t.z) * p.split_len : 0;
                const int k1 = split_k ? min(p.k, k0 + p.split_len) : p.k;
                const int batch = p.batched ? static_cast<int>(t.z) : 0;
                const int row_a = t.tm * kBM;
                const int row_b = t.tn * BN;
                for (int kk = k0; kk < k1; kk += kBK) {
                    if (!sm100::mbar_wait(empty_bar(stage), phase ^ 1u, abort)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * R::kStage;
                    const uint32_t b_dst = a_dst + R::kStageA;
                    const uint32_t bar = full_bar(stage);
                    sm100::mbar_expect_tx(bar, R::kStage);
                    if constexpr (!kAMn) {
                        if (p.batched) {
                            sm100::tma_load_3d(a_dst, &p.map_a, bar, kk, row_a, batch);
                        } else {
                            sm100::tma_load_2d(a_dst, &p.map_a, bar, kk, row_a);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < kBM / 64; ++j) {
                            if (p.batched) {
                                sm100::tma_load_3d(a_dst + j * 8192, &p.map_a, bar, row_a + 64 * j,
                                                   kk, batch);
                            } else {
                                sm100::tma_load_2d(a_dst + j * 8192, &p.map_a, bar, row_a + 64 * j,
                                                   kk);
                            }
                        }
                    }
                    if constexpr (!kBMn) {
                        if (p.batched) {
                            sm100::tma_load_3d(b_dst, &p.map_b, bar, kk, row_b, batch);
                        } else {
                            sm100::tma_load_2d(b_dst, &p.map_b, bar, kk, row_b);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) {
                            if (p.batched) {
                                sm100::tma_load_3d(b_dst + j * 8192, &p.map_b, bar, row_b + 64 * j,
                                                   kk, batch);
                            } else {
                                sm100::tma_load_2d(b_dst + j * 8192, &p.map_b, bar, row_b + 64 * j,
                                                   kk);
                            }
                        }
                    }
                    if (++stage == R::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (long long id = blockIdx.x; ok && id < p.tiles_total; id += gridDim.x) {
                const TileCoord t = decode_tile(p, id);
                const bool split_k = kIsTn && !p.batched;
                const int k0 = split_k ? static_cast<int>(t.z) * p.split_len : 0;
                const int k1 = split_k ? min(p.k, k0 + p.split_len) : p.k;
                if (!sm100::mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort)) {
                    ok = false;
                    break;
                }
                sm100::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                uint32_t accumulate = 0;
                for (int kk = k0; kk < k1; kk += kBK) {
                    if (!sm100::mbar_wait(full_bar(stage), phase, abort)) {
                        ok = false;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                    const uint32_t a_addr = smem_base + stage * R::kStage;
                    const uint32_t b_addr = a_addr + R::kStageA;
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks) {
                        // K-major: 16 halves = 32 bytes along the swizzled row.
                        // MN-major: 16 k-rows of 128 bytes.
                        const uint64_t a_desc =
                            kAMn ? sm100::smem_desc_sw128(a_addr + ks * 2048, 8192, 1024)
                                 : sm100::smem_desc_sw128(a_addr + ks * 32, 16, 1024);
                        const uint64_t b_desc =
                            kBMn ? sm100::smem_desc_sw128(b_addr + ks * 2048, 8192, 1024)
                                 : sm100::smem_desc_sw128(b_addr + ks * 32, 16, 1024);
                        sm100::mma_f16_ss(d_tmem, a_desc, b_desc, kIdesc, accumulate);
                        accumulate = 1;
                    }
                    sm100::mma_commit(empty_bar(stage));
                    if (++stage == R::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                sm100::mma_commit(acc_full_bar(acc));
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---- epilogue warps ----
        const int quadrant = warp % 4;      // the TMEM lanes this warp may read
        const int column_half = (warp - 2) / 4;  // which of the alternating 32-column chunks
        const bool coalesced = chunk_path_ok<E>(p);
        const bool prefetch = coalesced && aux_slots<E>() > 1;
        const uint32_t stage = staging + static_cast<uint32_t>(warp - 2) * 4096u;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (long long id = blockIdx.x; ok && id < p.tiles_total; id += gridDim.x) {
            const TileCoord t = decode_tile(p, id);
            const size_t row = static_cast<size_t>(t.tm) * kBM + quadrant * 32 + lane;
            const bool row_ok = row < static_cast<size_t>(p.m);
            const int col0 = t.tn * BN;
            const size_t batch_offset =
                p.batched ? static_cast<size_t>(t.z) * p.m * static_cast<size_t>(p.n) : 0;
            // The first chunk's second operands are requested before the accumulator is
            // awaited, each later chunk's while the one before it is processed.
            Aux<E> aux;
            if (prefetch && p.n - (col0 + column_half * 32) > 0) {
                load_aux<E>(aux, p, batch_offset, row - lane, col0 + column_half * 32,
                            min(32, p.n - (col0 + column_half * 32)), lane);
            }
            if (!sm100::mbar_wait(acc_full_bar(acc), acc_phase, abort)) {
                ok = false;
                break;
            }
            sm100::tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + static_cast<uint32_t>(acc * BN) +
                                    (static_cast<uint32_t>(quadrant * 32) << 16);
#pragma unroll 1
            for (int c = column_half * 32; c < BN; c += 64) {
                const bool last = c + 64 >= BN;
                const int col = col0 + c;
                const int valid = min(32, p.n - col);  // warp-uniform
                Aux<E> next = aux;
                if (prefetch && !last && p.n - (col + 64) > 0) {
                    load_aux<E>(next, p, batch_offset, row - lane, col + 64,
                                min(32, p.n - (col + 64)), lane);
                }
                const float bias_lane = load_bias_lane<E>(p, col, lane);
                uint32_t raw[32];
                if (valid > 0) {
                    sm100::tmem_ld_32x32(t_addr + c, raw);
                    sm100::tmem_ld_wait();
                }
                if (last) {
                    // This warp's reads of the accumulator are complete: hand it back.
                    sm100::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        sm100::mbar_arrive(acc_empty_bar(acc));
                    }
                }
                if (valid > 0) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(raw[j]);
                    }
                    if (coalesced) {
                        store_chunk<E>(p, stage, batch_offset, t.z, row - lane, col, v, valid,
                                       lane, aux, bias_lane);
                    } else if (row_ok) {
                        store_segment<E>(p, batch_offset, t.z, row, col, v, valid);
                    }
                }
                aux = next;
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1u;
            }
        }
    }

    // ---- teardown ----
    __syncthreads();
    if (abort_flag != 0) {
        if (threadIdx.x == 0) {
            atomicExch(&g_gemm_error, 1);
        }
        // Let any TMA copy still in flight land before shared memory is released.
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- the CTA-pair kernel: 256 x 256 tiles --------------------------------------------------
//
// Two CTAs of a cluster work on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (M = 256, N = 256): CTA r of the pair loads rows
// [128 r, 128 r + 128) of the A tile and the same range of the B tile (its half
// of N), so each SM moves 32 KB per k-block instead of the 48 KB of a 128 x 256
// single-CTA tile, and its tensor memory receives its own 128 rows of D. The
// leader (rank 0) issues every MMA; commits reach both CTAs' barriers; the
// peer's TMA transactions and epilogue arrivals are counted on the leader's
// barriers. Roles per CTA are those of fb_gemm_tc.

constexpr int kPairBN = 256;
constexpr int kPairStageA = kBM * kBK * 2;          // 16 KB
constexpr int kPairStageB = 128 * kBK * 2;          // 16 KB: half of the 256 B rows
constexpr int kPairStage = kPairStageA + kPairStageB;
constexpr int kPairStages = kRingBytes / kPairStage;  // 6
constexpr int kPairSmemBytes = kPairStages * kPairStage + kEpilogueWarps * 4096 + 1024 + 256;
constexpr int kPairGroupM = 4;  // rows of 256-row tiles handed out together

__device__ __forceinline__ TileCoord decode_pair_tile(const GemmParams& p, long long id) {
    const long long per = static_cast<long long>(p.tiles_m) * p.tiles_n;
    TileCoord c;
    c.z = id / per;
    const long long r = id - c.z * per;
    const long long group_span = static_cast<long long>(kPairGroupM) * p.tiles_n;
    const long long g = r / group_span;
    const int first_m = static_cast<int>(g) * kPairGroupM;
    const int rows_here = min(kPairGroupM, p.tiles_m - first_m);
    const long long in_group = r - g * group_span;
    c.tm = first_m + static_cast<int>(in_group % rows_here);
    c.tn = static_cast<int>(in_group / rows_here);
    return c;
}

// Epilogue warps per CTA of the pair kernel: two per TMEM lane quadrant, 4 KB of
// staging each. (Four per quadrant were measured for the element-wise FP16
// epilogues and were slower: 96 registers per thread spill.)
template <Epilogue E>
__host__ __device__ constexpr int pair_epilogue_warps() {
    return 8;
}

template <Layout L, Epilogue E>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * pair_epilogue_warps<E>(), 1)
    fb_gemm_pair(const __grid_constant__ GemmParams p) {
    constexpr int kEpi = pair_epilogue_warps<E>();
    constexpr int kColumnStep = 32 * (kEpi / 4);            // between a warp's chunks
    constexpr uint32_t kSlotBytes = kEpilogueWarps * 4096 / kEpi;
    constexpr bool kAMn = L == Layout::kTN;
    constexpr bool kBMn = L != Layout::kNT;
    constexpr bool kIsTn = L == Layout::kTN;
    constexpr uint32_t kIdesc = sm100::instr_desc_f16(256, kPairBN, kAMn, kBMn);
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging = smem_base + kPairStages * kPairStage;
    const uint32_t bars = staging + kEpilogueWarps * 4096;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kPairStages + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * kPairStages + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * kPairStages + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t rank = sm100::cluster_cta_rank();
    const bool leader = rank == 0;
    const long long pair = blockIdx.x / 2;
    const long long pairs = gridDim.x / 2;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kPairStages; ++s) {
            sm100::mbar_init(full_bar(s), 1);
            sm100::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            sm100::mbar_init(acc_full_bar(a), 1);
            sm100::mbar_init(acc_empty_bar(a), 2 * kEpi);
        }
        sm100::mbar_fence_init();
        sm100::tma_prefetch_descriptor(&p.map_a);
        sm100::tma_prefetch_descriptor(&p.map_b);
    }
    if (warp == 1) {
        sm100::tmem_alloc_pair(sm100::smem_u32(&tmem_base_slot), kTmemCols);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    // Both CTAs' barriers exist before either touches the other's.
    sm100::cluster_sync_all();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;
    // Everything above ran while the previous kernel in the stream may still have been
    // finishing; global memory is touched only from here on.
    fb::dependency_wait();
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }

    if (warp == 0) {
        // ---- TMA producer (both CTAs) ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long id = pair; ok && id < p.tiles_total; id += pairs) {
                const TileCoord t = decode_pair_tile(p, id);
                const bool split_k = kIsTn && !p.batched;
                const int k0 = split_k ? static_cast<int>(t.z) * p.split_len : 0;
                const int k1 = split_k ? min(p.k, k0 + p.split_len) : p.k;
                const int batch = p.batched ? static_cast<int>(t.z) : 0;
                const int row_a = t.tm * 256 + static_cast<int>(rank) * 128;
                const int row_b = t.tn * kPairBN + static_cast<int>(rank) * 128;
                for (int kk = k0; kk < k1; kk += kBK) {
                    if (!sm100::mbar_wait(empty_bar(stage), phase ^ 1u, abort)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * kPairStage;
                    const uint32_t b_dst = a_dst + kPairStageA;
                    if (leader) {
                        // The leader's barrier counts both CTAs' bytes.
                        sm100::mbar_expect_tx(full_bar(stage), 2 * kPairStage);
                    }
                    const uint32_t bar = sm100::map_to_cta(full_bar(stage), 0);
                    if constexpr (!kAMn) {
                        if (p.batched) {
                            sm100::tma_load_3d_pair(a_dst, &p.map_a, bar, kk, row_a, batch);
                        } else {
                            sm100::tma_load_2d_pair(a_dst, &p.map_a, bar, kk, row_a);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (p.batched) {
                                sm100::tma_load_3d_pair(a_dst + j * 8192, &p.map_a, bar,
                                                        row_a + 64 * j, kk, batch);
                            } else {
                                sm100::tma_load_2d_pair(a_dst + j * 8192, &p.map_a, bar,
                                                        row_a + 64 * j, kk);
                            }
                        }
                    }
                    if constexpr (!kBMn) {
                        if (p.batched) {
                            sm100::tma_load_3d_pair(b_dst, &p.map_b, bar, kk, row_b, batch);
                        } else {
                            sm100::tma_load_2d_pair(b_dst, &p.map_b, bar, kk, row_b);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (p.batched) {
                                sm100::tma_load_3d_pair(b_dst + j * 8192, &p.map_b, bar,
                                                        row_b + 64 * j, kk, batch);
                            } else {
                                sm100::tma_load_2d_pair(b_dst + j * 8192, &p.map_b, bar,
                                                        row_b + 64 * j, kk);
                            }
                        }
                    }
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (leader only) ----
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (long long id = pair; ok && id < p.tiles_total; id += pairs) {
                const TileCoord t = decode_pair_tile(p, id);
                const bool split_k = kIsTn && !p.batched;
                const int k0 = split_k ? static_cast<int>(t.z) * p.split_len : 0;
                const int k1 = split_k ? min(p.k, k0 + p.split_len) : p.k;
                if (!sm100::mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort)) {
                    ok = false;
                    break;
                }
                sm100::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairBN);
                uint32_t accumulate = 0;
                for (int kk = k0; kk < k1; kk += kBK) {
                    if (!sm100::mbar_wait(full_bar(stage), phase, abort)) {
                        ok = false;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                    const uint32_t a_addr = smem_base + stage * kPairStage;
                    const uint32_t b_addr = a_addr + kPairStageA;
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks) {
                        const uint64_t a_desc =
                            kAMn ? sm100::smem_desc_sw128(a_addr + ks * 2048, 8192, 1024)
                                 : sm100::smem_desc_sw128(a_addr + ks * 32, 16, 1024);
                        const uint64_t b_desc =
                            kBMn ? sm100::smem_desc_sw128(b_addr + ks * 2048, 8192, 1024)
                                 : sm100::smem_desc_sw128(b_addr + ks * 32, 16, 1024);
                        sm100::mma_f16_ss_pair(d_tmem, a_desc, b_desc, kIdesc, accumulate);
                        accumulate = 1;
                    }
                    sm100::mma_commit_pair(empty_bar(stage), 3);
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                sm100::mma_commit_pair(acc_full_bar(acc), 3);
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---- epilogue warps (both CTAs) ----
        const int quadrant = warp % 4;
        const int column_part = (warp - 2) / 4;
        const bool coalesced = chunk_path_ok<E>(p);
        const bool prefetch = coalesced && aux_slots<E>() > 1;
        constexpr bool kAhead = kEpi == 8;  // room to keep the next chunk's operands too
        const uint32_t stage = staging + static_cast<uint32_t>(warp - 2) * kSlotBytes;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        // A chunk's second operands (residual, pre-activations) are requested while the
        // chunk before it is processed. For the dGELU epilogue the first chunk of a tile
        // counts as following the last chunk of the tile before, so only this CTA's very
        // first chunk waits for its operands with nothing else to do; the others request
        // a tile's first operands before they wait for its accumulator.
        Aux<E> aux;
        bool aux_requested = false;
        for (long long id = pair; ok && id < p.tiles_total; id += pairs) {
            const TileCoord t = decode_pair_tile(p, id);
            const size_t row = static_cast<size_t>(t.tm) * 256 + rank * 128 + quadrant * 32 + lane;
            const bool row_ok = row < static_cast<size_t>(p.m);
            const int col0 = t.tn * kPairBN;
            const size_t batch_offset =
                p.batched ? static_cast<size_t>(t.z) * p.m * static_cast<size_t>(p.n) : 0;
            if (prefetch && !aux_requested && p.n - (col0 + column_part * 32) > 0) {
                load_aux<E>(aux, p, batch_offset, row - lane, col0 + column_part * 32,
                            min(32, p.n - (col0 + column_part * 32)), lane);
            }
            aux_requested = false;
            float bias_next = load_bias_lane<E>(p, col0 + column_part * 32, lane);
            if (!sm100::mbar_wait(acc_full_bar(acc), acc_phase, abort)) {
                ok = false;
                break;
            }
            sm100::tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + static_cast<uint32_t>(acc * kPairBN) +
                                    (static_cast<uint32_t>(quadrant * 32) << 16);
            const uint32_t leader_empty = sm100::map_to_cta(acc_empty_bar(acc), 0);
            // The warp's chunks, software-pipelined: chunk i+1's accumulators are being
            // read from tensor memory into the other register set while chunk i is
            // worked on.
            constexpr int kChunks = kPairBN / kColumnStep;
            // The epilogues with second operands already hold a chunk of those ahead; a
            // second accumulator set in flight as well would not fit in registers.
            constexpr bool kPipelined =
                !(E == Epilogue::kBiasResidual || E == Epilogue::kTnStore ||
                  E == Epilogue::kTnPartial || E == Epilogue::kDGelu);
            uint32_t raw[2][32];
            auto chunk_column = [&](int i) { return column_part * 32 + i * kColumnStep; };
            auto chunk_valid = [&](int i) { return min(32, p.n - (col0 + chunk_column(i))); };
            if (kPipelined && chunk_valid(0) > 0) {
                sm100::tmem_ld_32x32(t_addr + chunk_column(0), raw[0]);
            }
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                const bool last = i + 1 == kChunks;
                const int c = chunk_column(i);
                const int col = col0 + c;
                const int valid = chunk_valid(i);
                const float bias_lane = bias_next;
                if (!last) {
                    bias_next = load_bias_lane<E>(p, col + kColumnStep, lane);
                }
                Aux<E> next = aux;
                if (kAhead && prefetch && !last && chunk_valid(i + 1) > 0) {
                    load_aux<E>(next, p, batch_offset, row - lane, col + kColumnStep,
                                chunk_valid(i + 1), lane);
                }
                // (Only where the operands are few registers: with the FP32 residual's 32
                // registers held through the last chunk as well, the kernel was slower.)
                if (E == Epilogue::kDGelu && kAhead && prefetch && last &&
                    id + pairs < p.tiles_total) {
                    // The next tile's first chunk.
                    const TileCoord t2 = decode_pair_tile(p, id + pairs);
                    const size_t row2 =
                        static_cast<size_t>(t2.tm) * 256 + rank * 128 + quadrant * 32;
                    const int col2 = t2.tn * kPairBN + column_part * 32;
                    const size_t offset2 =
                        p.batched ? static_cast<size_t>(t2.z) * p.m * static_cast<size_t>(p.n) : 0;
                    if (p.n - col2 > 0) {
                        load_aux<E>(next, p, offset2, row2, col2, min(32, p.n - col2), lane);
                        aux_requested = true;
                    }
                }
                const int kSet = kPipelined ? (i & 1) : 0;  // static once unrolled
                if (!kPipelined && valid > 0) {
                    sm100::tmem_ld_32x32(t_addr + c, raw[0]);
                }
                sm100::tmem_ld_wait();
                // The loaded registers are "rewritten" by empty volatile statements so
                // that nothing reading them can be scheduled above the wait.
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    asm volatile(""
                                 : "+r"(raw[kSet][j]), "+r"(raw[kSet][j + 1]),
                                   "+r"(raw[kSet][j + 2]), "+r"(raw[kSet][j + 3]),
                                   "+r"(raw[kSet][j + 4]), "+r"(raw[kSet][j + 5]),
                                   "+r"(raw[kSet][j + 6]), "+r"(raw[kSet][j + 7]));
                }
                if (kPipelined && !last && chunk_valid(i + 1) > 0) {
                    sm100::tmem_ld_32x32(t_addr + chunk_column(i + 1), raw[(i + 1) & 1]);
                }
                if (last) {
                    // Every read of this accumulator has completed: hand it back.
                    sm100::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        sm100::mbar_arrive_cluster(leader_empty);
                    }
                }
                if (valid > 0) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(raw[kSet][j]);
                    }
                    if (coalesced) {
                        store_chunk<E>(p, stage, batch_offset, t.z, row - lane, col, v, valid,
                                       lane, aux, bias_lane);
                    } else if (row_ok) {
                        store_segment<E>(p, batch_offset, t.z, row, col, v, valid);
                    }
                }
                if (kAhead) {
                    aux = next;
                } else if (prefetch && !last && chunk_valid(i + 1) > 0) {
                    load_aux<E>(aux, p, batch_offset, row - lane, col + kColumnStep,
                                chunk_valid(i + 1), lane);
                }
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1u;
            }
        }
        // Asynchronous output stores must have landed before the kernel is over.
        if (p.tma_out != 0 && lane == 0) {
            store_wait_all();
        }
    }

    // ---- teardown: neither CTA leaves while the other may still signal it ----
    __syncthreads();
    if (abort_flag != 0) {
        if (threadIdx.x == 0) {
            atomicExch(&g_gemm_error, 1);
        }
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
        __syncthreads();
    }
    sm100::tc_fence_before_sync();
    sm100::cluster_sync_all();
    if (warp == 1) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---- plain CUDA-core kernel, for debugging the pipeline only -------------------------
//
// Selected with FLINT_B200_GEMM=simt in the environment; never the default.

template <Layout L, Epilogue E>
__global__ void __launch_bounds__(256)
    fb_gemm_simt(GemmParams p, const __half* __restrict__ x, const __half* __restrict__ w) {
    const long long total = static_cast<long long>(p.batches) * p.m * p.n;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += gridDim.x * 256LL) {
        const long long b = i / (static_cast<long long>(p.m) * p.n);
        const long long r = i - b * p.m * p.n;
        const int row = static_cast<int>(r / p.n);
        const int col = static_cast<int>(r % p.n);
        const __half* xb = x + b * p.m * p.k;
        const __half* wb = w + b * p.n * p.k;
        float acc = 0.0f;
        for (int kk = 0; kk < p.k; ++kk) {
            float a;
            float c;
            if (L == Layout::kTN) {
                a = __half2float(xb[static_cast<size_t>(kk) * p.m + row]);
            } else {
                a = __half2float(xb[static_cast<size_t>(row) * p.k + kk]);
            }
            if (L == Layout::kNT) {
                c = __half2float(wb[static_cast<size_t>(col) * p.k + kk]);
            } else {
                c = __half2float(wb[static_cast<size_t>(kk) * p.n + col]);
            }
            acc = fmaf(a, c, acc);
        }
        const size_t at = static_cast<size_t>(b) * p.m * p.n + static_cast<size_t>(row) * p.n + col;
        if (E == Epilogue::kBias || E == Epilogue::kBiasGelu || E == Epilogue::kBiasResidual) {
            acc = __fadd_rn(acc, p.bias[col]);
        }
        if (E == Epilogue::kScale) {
            acc = __fmul_rn(acc, p.scale);
        }
        if (E == Epilogue::kDGelu) {
            acc = __fmul_rn(acc, gelu_tanh_grad(__half2float(static_cast<const __half*>(p.aux_in)[at])));
        }
        if (E == Epilogue::kBiasResidual) {
            static_cast<float*>(p.y)[at] = __fadd_rn(static_cast<const float*>(p.aux_in)[at], acc);
        } else if (E == Epilogue::kTnStore) {
            float* out = static_cast<float*>(p.y) + at;
            *out = p.accumulate ? __fadd_rn(*out, acc) : acc;
        } else if (E == Epilogue::kBiasGelu) {
            static_cast<__half*>(p.aux_out)[at] = __float2half_rn(acc);
            static_cast<__half*>(p.y)[at] = __float2half_rn(gelu_tanh(acc));
        } else {
            static_cast<__half*>(p.y)[at] = __float2half_rn(acc);
        }
    }
}

// y = (old +) p0 + p1 + ... in split order.
__global__ void __launch_bounds__(256)
    fb_gemm_tn_reduce(float4* __restrict__ y, const float4* __restrict__ partials, size_t quads,
                      int splits, int accumulate) {
    fb::dependency_wait();
    fb::dependency_release();
    for (size_t i = size_t{blockIdx.x} * 256 + threadIdx.x; i < quads;
         i += size_t{gridDim.x} * 256) {
        float4 s = partials[i];
        for (int k = 1; k < splits; ++k) {
            const float4 v = partials[static_cast<size_t>(k) * quads + i];
            s = make_float4(__fadd_rn(s.x, v.x), __fadd_rn(s.y, v.y), __fadd_rn(s.z, v.z),
                            __fadd_rn(s.w, v.w));
        }
        if (accumulate) {
            const float4 o = y[i];
            s = make_float4(__fadd_rn(o.x, s.x), __fadd_rn(o.y, s.y), __fadd_rn(o.z, s.z),
                            __fadd_rn(o.w, s.w));
        }
        y[i] = s;
    }
}

// ---- host side ----------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

cudaError_t encode_fn(EncodeTiled* out) {
    static EncodeTiled cached = nullptr;
    if (cached == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        const cudaError_t e =
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
        if (e != cudaSuccess) {
            return e;
        }
        if (status != cudaDriverEntryPointSuccess || fn == nullptr) {
            return cudaErrorNotSupported;
        }
        cached = reinterpret_cast<EncodeTiled>(fn);
    }
    *out = cached;
    return cudaSuccess;
}

// A row-major FP16 matrix [outer][inner] (inner contiguous), optionally
// repeated `batches` times back to back; boxes are 64 inner elements (one
// 128-byte swizzle row) by box_outer rows.
cudaError_t make_map(CUtensorMap* map, const void* base, size_t inner, size_t outer,
                     size_t batches, bool batched, int box_outer) {
    EncodeTiled encode = nullptr;
    cudaError_t e = encode_fn(&encode);
    if (e != cudaSuccess) {
        return e;
    }
    const cuuint64_t dims[3] = {inner, outer, batches};
    const cuuint64_t strides[2] = {inner * 2, inner * outer * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_outer), 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, batched ? 3 : 2,
                              const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

bool use_simt() {
    static int cached = -1;
    if (cached < 0) {
        const char* v = std::getenv("FLINT_B200_GEMM");
        cached = (v != nullptr && std::strcmp(v, "simt") == 0) ? 1 : 0;
    }
    return cached == 1;
}

int pick_bn(size_t n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

template <Layout L, Epilogue E, int BN>
cudaError_t launch_tc(GemmParams& p, const void* x, const void* w, int sms, cudaStream_t stream) {
    using R = Ring<BN>;
    constexpr bool kAMn = L == Layout::kTN;
    constexpr bool kBMn = L != Layout::kNT;
    const bool batched = p.batched != 0;
    cudaError_t e;
    if (kAMn) {
        e = make_map(&p.map_a, x, p.m, p.k, p.batches, batched, kBK);
    } else {
        e = make_map(&p.map_a, x, p.k, p.m, p.batches, batched, kBM);
    }
    if (e != cudaSuccess) {
        return e;
    }
    if (kBMn) {
        e = make_map(&p.map_b, w, p.n, p.k, p.batches, batched, kBK);
    } else {
        e = make_map(&p.map_b, w, p.k, p.n, p.batches, batched, BN);
    }
    if (e != cudaSuccess) {
        return e;
    }
    p.tiles_m = (p.m + kBM - 1) / kBM;
    p.tiles_n = (p.n + BN - 1) / BN;
    const long long z = L == Layout::kTN && !batched ? p.splits : p.batches;
    p.tiles_total = static_cast<long long>(p.tiles_m) * p.tiles_n * z;

    static std::atomic<bool> configured[64] = {};
    auto kernel = fb_gemm_tc<L, E, BN>;
    e = fb::allow_shared_memory(kernel, R::kSmemBytes, configured);
    if (e != cudaSuccess) {
        return e;
    }
    const unsigned grid = static_cast<unsigned>(std::min<long long>(p.tiles_total, sms));
    return fb::launch_dependent(kernel, dim3(grid), dim3(kThreads), R::kSmemBytes, stream, p);
}

bool pair_disabled() {
    static int cached = -1;
    if (cached < 0) {
        const char* v = std::getenv("FLINT_B200_GEMM");
        cached = (v != nullptr && std::strcmp(v, "single") == 0) ? 1 : 0;
    }
    return cached == 1;
}

// The CTA-pair kernel pays off once both CTAs of a pair have rows to work on
// and the tile is full width.
bool use_pair(const GemmParams& p) {
    return !pair_disabled() && p.m > 128 && p.n > 128;
}

template <Layout L, Epilogue E>
cudaError_t launch_pair(GemmParams& p, const void* x, const void* w, int sms, cudaStream_t stream) {
    constexpr bool kAMn = L == Layout::kTN;
    constexpr bool kBMn = L != Layout::kNT;
    const bool batched = p.batched != 0;
    cudaError_t e;
    if (kAMn) {
        e = make_map(&p.map_a, x, p.m, p.k, p.batches, batched, kBK);
    } else {
        e = make_map(&p.map_a, x, p.k, p.m, p.batches, batched, kBM);
    }
    if (e != cudaSuccess) {
        return e;
    }
    if (kBMn) {
        e = make_map(&p.map_b, w, p.n, p.k, p.batches, batched, kBK);
    } else {
        e = make_map(&p.map_b, w, p.k, p.n, p.batches, batched, 128);
    }
    if (e != cudaSuccess) {
        return e;
    }
    // FP16 outputs of unbatched calls leave through TMA stores when the rows are 16-byte
    // multiples (the tensor map's requirement; the same rule as the coalesced path).
    constexpr bool kHalfOut = E == Epilogue::kNone || E == Epilogue::kBias ||
                              E == Epilogue::kBiasGelu || E == Epilogue::kDGelu ||
                              E == Epilogue::kScale;
    p.tma_out = 0;
    if (kHalfOut && L != Layout::kTN && !batched && p.n % 8 == 0) {
        e = fb::encode_rows_map(&p.map_y, p.y, p.m, p.n, 2, 32, 32, 64);
        if (e == cudaSuccess && E == Epilogue::kBiasGelu) {
            e = fb::encode_rows_map(&p.map_pre, p.aux_out, p.m, p.n, 2, 32, 32, 64);
        }
        if (e != cudaSuccess) {
            return e;
        }
        p.tma_out = 1;
    }
    p.tiles_m = (p.m + 255) / 256;
    p.tiles_n = (p.n + kPairBN - 1) / kPairBN;
    const long long z = L == Layout::kTN && !batched ? p.splits : p.batches;
    p.tiles_total = static_cast<long long>(p.tiles_m) * p.tiles_n * z;

    static std::atomic<bool> configured[64] = {};
    auto kernel = fb_gemm_pair<L, E>;
    e = fb::allow_shared_memory(kernel, kPairSmemBytes, configured);
    if (e != cudaSuccess) {
        return e;
    }
    const long long pairs = std::min<long long>(p.tiles_total, sms / 2);
    return fb::launch_dependent(kernel, dim3(static_cast<unsigned>(2 * pairs)),
                                dim3(64 + 32 * pair_epilogue_warps<E>()), kPairSmemBytes, stream, p);
}

template <Layout L, Epilogue E>
cudaError_t launch_any(GemmParams& p, const void* x, const void* w, cudaStream_t stream) {
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) {
        return e;
    }
    if (use_simt()) {
        const long long total = static_cast<long long>(p.batches) * p.m * p.n;
        const unsigned grid =
            static_cast<unsigned>(std::min<long long>((total + 255) / 256, sms * 32LL));
        fb_gemm_simt<L, E><<<grid, 256, 0, stream>>>(p, static_cast<const __half*>(x),
                                                     static_cast<const __half*>(w));
        return fb::after_launch();
    }
    if (use_pair(p)) {
        return launch_pair<L, E>(p, x, w, sms, stream);
    }
    switch (pick_bn(static_cast<size_t>(p.n))) {
    case 256:
        return launch_tc<L, E, 256>(p, x, w, sms, stream);
    case 128:
        return launch_tc<L, E, 128>(p, x, w, sms, stream);
    default:
        return launch_tc<L, E, 64>(p, x, w, sms, stream);
    }
}

GemmParams base_params(void* y, size_t m, size_t n, size_t k, size_t batches, bool batched) {
    GemmParams p;
    std::memset(&p, 0, sizeof p);
    p.y = y;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.batches = static_cast<int>(batches);
    p.batched = batched ? 1 : 0;
    p.splits = 1;
    p.split_len = static_cast<int>((k + kBK - 1) / kBK * kBK);
    p.scale = 1.0f;
    return p;
}

}  // namespace

// ---- internal launchers (declared in gemm.h) --------------------------------------------

TnSplit tn_split(size_t m, size_t n, size_t k, int sms) {
    // Tiles and the CTAs (or CTA pairs) that run at once, for the kernel this shape gets.
    const bool pair = !pair_disabled() && m > 128 && n > 128;
    const long long tiles =
        pair ? static_cast<long long>((m + 255) / 256) * static_cast<long long>((n + 255) / 256)
             : static_cast<long long>((m + kBM - 1) / kBM) *
                   static_cast<long long>((n + pick_bn(n) - 1) / pick_bn(n));
    const long long slots = pair ? std::max(1, sms / 2) : sms;
    const int most = static_cast<int>(std::min<size_t>(16, std::max<size_t>(1, k / 1024)));
    int want = 1;
    double best = 0.0;
    for (int s = 1; s <= most; ++s) {
        const long long blocks = tiles * s;
        const long long waves = (blocks + slots - 1) / slots;
        const double fill = static_cast<double>(blocks) / static_cast<double>(waves * slots);
        if (fill > best) {
            best = fill;
            want = s;
        }
        if (fill >= 0.75) {
            want = s;
            break;
        }
    }
    const size_t per = (k + want - 1) / want;
    TnSplit r;
    r.len = static_cast<int>((per + kBK - 1) / kBK * kBK);
    r.count = static_cast<int>((k + r.len - 1) / r.len);
    return r;
}

cudaError_t gemm_nt(Epilogue e, void* y, void* pre, const void* x, const void* w,
                    const void* bias, const void* residual, size_t m, size_t n, size_t k,
                    cudaStream_t stream) {
    GemmParams p = base_params(y, m, n, k, 1, false);
    p.bias = static_cast<const float*>(bias);
    p.aux_out = pre;
    p.aux_in = residual;
    switch (e) {
    case Epilogue::kNone:
        return launch_any<Layout::kNT, Epilogue::kNone>(p, x, w, stream);
    case Epilogue::kBias:
        return launch_any<Layout::kNT, Epilogue::kBias>(p, x, w, stream);
    case Epilogue::kBiasGelu:
        return launch_any<Layout::kNT, Epilogue::kBiasGelu>(p, x, w, stream);
    case Epilogue::kBiasResidual:
        return launch_any<Layout::kNT, Epilogue::kBiasResidual>(p, x, w, stream);
    default:
        return cudaErrorInvalidValue;
    }
}

cudaError_t gemm_nn(Epilogue e, void* y, const void* x, const void* w, const void* pre, size_t m,
                    size_t n, size_t k, cudaStream_t stream) {
    GemmParams p = base_params(y, m, n, k, 1, false);
    p.aux_in = pre;
    if (e == Epilogue::kDGelu) {
        return launch_any<Layout::kNN, Epilogue::kDGelu>(p, x, w, stream);
    }
    return launch_any<Layout::kNN, Epilogue::kNone>(p, x, w, stream);
}

cudaError_t gemm_tn(void* y, const void* x, const void* w, size_t m, size_t n, size_t k,
                    bool accumulate, void* workspace, cudaStream_t stream) {
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) {
        return e;
    }
    GemmParams p = base_params(y, m, n, k, 1, false);
    p.accumulate = accumulate ? 1 : 0;
    const TnSplit s = use_simt() ? TnSplit{1, p.split_len} : tn_split(m, n, k, sms);
    if (s.count == 1) {
        return launch_any<Layout::kTN, Epilogue::kTnStore>(p, x, w, stream);
    }
    p.splits = s.count;
    p.split_len = s.len;
    p.partials = static_cast<float*>(workspace);
    e = launch_any<Layout::kTN, Epilogue::kTnPartial>(p, x, w, stream);
    if (e != cudaSuccess) {
        return e;
    }
    const size_t quads = m * n / 4;
    const unsigned grid =
        static_cast<unsigned>(std::min<size_t>((quads + 255) / 256, static_cast<size_t>(sms) * 8));
    return fb::launch_dependent(fb_gemm_tn_reduce, dim3(grid), dim3(256), 0, stream,
                                static_cast<float4*>(y), static_cast<const float4*>(workspace),
                                quads, s.count, p.accumulate);
}

cudaError_t gemm_batched(Layout l, void* y, const void* x, const void* w, size_t batches,
                         size_t m, size_t n, size_t k, float scale, cudaStream_t stream) {
    GemmParams p = base_params(y, m, n, k, batches, true);
    p.scale = scale;
    switch (l) {
    case Layout::kNT:
        return launch_any<Layout::kNT, Epilogue::kScale>(p, x, w, stream);
    case Layout::kNN:
        return launch_any<Layout::kNN, Epilogue::kNone>(p, x, w, stream);
    default:
        return launch_any<Layout::kTN, Epilogue::kNone>(p, x, w, stream);
    }
}

cudaError_t gemm_error_flag(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_gemm_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    }
    return e;
}

}  // namespace fb
