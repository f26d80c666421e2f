// Deterministic reductions over rows: flint_bias_gradient, flint_layernorm_backward,
// flint_embedding_backward and their workspace queries.
//
// Column sums (a bias gradient, LayerNorm's dgamma/dbeta, the position table's
// gradient) share one two-pass scheme whose addition order depends only on the
// matrix shape, never on the GPU: rows are cut into chunks of 256; inside a
// chunk, lane-row y (0..7) adds rows y, y+8, ... with a compensated FP32 sum,
// the eight lane-rows are merged in order of y, and the chunk's (sum, error)
// pair per column goes to the workspace as two FP32 rows; a second pass merges
// the chunks (lane l takes chunks l, l+32, ..., then a butterfly) and writes
// sum + error. There are no floating-point atomics anywhere.
// Reference for the order and the workspace layout:
// src/kernels/bias_gradient.cu:82-178, src/kernels/layernorm_backward.cu:119-233,
// src/kernels/embedding_backward.cu:131-345 and embedding_backward.cuh:31-79.
//
// Argument checks follow src/api/bias_gradient.cpp:11-67,
// src/api/layernorm.cpp:55-119 and src/api/embedding.cpp:55-134.
#include <algorithm>
#include <atomic>
#include <cstdint>

#include <cuda.h>
#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"
#include "flint/flint_b200.h"

namespace {

using fb::Comp;

constexpr size_t kChunkRows = 256;
constexpr int kLaneRows = 8;    // interleaved row streams per chunk
constexpr int kTilePieces = 32; // 8-column pieces per CTA tile
constexpr size_t kMaxCols = size_t{65535} * 256;            // 16,776,960
constexpr size_t kMaxBiasRows = size_t{0x7fffffff} * 256;   // 549,755,813,632
constexpr size_t kMaxRows8 = size_t{0x7fffffff} * 8;

constexpr size_t column_sum_workspace(size_t rows, size_t cols) {
    return (rows + kChunkRows - 1) / kChunkRows * cols * 8;
}

enum class Source { kHalf, kHalfTimesXhat, kFloat };

// First pass. CTA (chunk, tile) with 32 x 9 threads: warps 0-7 add (thread
// (px, ly) owns the 8 columns of piece tile*32+px and the row stream ly), warp 8
// fetches.
//
// The chunk's rows reach the CTA through shared memory: lane l of the fetching
// warp issues one bulk asynchronous copy per row segment (32 rows per stage, a
// ring of stages, each completing on its own mbarrier), so whole stages are in
// flight per CTA while every adding thread still takes its stream's rows
// strictly in row order. (A thread that loaded its own rows would add each one as
// it arrived, paying one memory latency per row.) The additions run on packed
// FP32 pairs: columns (0,1), (2,3), (4,5), (6,7) of the piece.
template <Source kSource>
struct Staging {
    static constexpr int kMainBytes = kSource == Source::kFloat ? 32 : 16;  // per piece and row
    static constexpr int kXBytes = kSource == Source::kHalfTimesXhat ? 32 : 0;
    static constexpr int kRows = 32;                                        // rows per stage
    static constexpr int kMainStage = kRows * kTilePieces * kMainBytes;
    static constexpr int kStage = kMainStage + kRows * kTilePieces * kXBytes;
    static constexpr int kStages = kSource == Source::kHalf ? 4 : 2;
    static constexpr int kBytes = kStages * kStage + 128;
};
// After the last stage the ring's memory holds the eight streams' sums for the merge.
static_assert(Staging<Source::kHalf>::kStages * Staging<Source::kHalf>::kStage >=
                  2 * kLaneRows * kTilePieces * 8 * 4,
              "the merge buffers must fit in the ring");

__device__ int g_reduction_error = 0;

__device__ __forceinline__ uint32_t shared_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Bounded mbarrier wait: false (and the flag set) after about a second of SM clocks.
__device__ __forceinline__ bool staged_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
    const long long start = clock64();
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done = 0;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done != 0) {
            return true;
        }
        if ((spin & 63u) == 63u && (*abort != 0 || clock64() - start > 2000000000LL)) {
            *abort = 1;
            return false;
        }
    }
}

// Tensor maps of the source (and of x for the dgamma sums): one TMA tensor load
// then brings a whole 32-row stage. `use` is 0 for matrices whose row count does
// not fit a tensor map; those stages are fetched row by row.
struct ColumnMaps {
    CUtensorMap main;
    CUtensorMap x;
    int use;
};

// kPlain: a stream adds its rows with ordinary FP32 adds (one instruction per pair
// instead of seven); the eight streams, the chunks and the lanes are still merged with
// compensated adds in the same fixed order. This is not the reference's pinned
// arithmetic (the public entry points never use it); the model built on the fused
// attention kernels does, where it makes these kernels bandwidth-bound. In that variant
// the FP16-times-xhat kernel (LayerNorm's dgamma) also sums the FP16 values themselves
// (dbeta) from the same staged rows, with the operations the plain FP16 kernel would
// use, and writes those partial sums as a second block right behind the first one.
template <Source kSource, bool kPlain>
__global__ void __launch_bounds__(kTilePieces * (kLaneRows + 1))
    fb_column_partials(const __grid_constant__ ColumnMaps maps, float4* __restrict__ partial,
                       const void* __restrict__ src, const float4* __restrict__ x,
                       const float* __restrict__ mean, const float* __restrict__ rstd, size_t rows,
                       int pieces) {
    using S = Staging<kSource>;
    extern __shared__ unsigned char staging_raw[];
    __shared__ float sh_mean[kSource == Source::kHalfTimesXhat ? kChunkRows : 1];
    __shared__ float sh_rstd[kSource == Source::kHalfTimesXhat ? kChunkRows : 1];
    __shared__ alignas(8) unsigned long long barriers[2 * S::kStages];
    __shared__ int abort_flag;
    const int px = threadIdx.x;
    const int ly = threadIdx.y;  // 0-7 add, 8 fetches
    const int first_piece = blockIdx.y * kTilePieces;
    const int piece = first_piece + px;
    const int width = min(kTilePieces, pieces - first_piece);  // pieces this tile holds
    const size_t first = size_t{blockIdx.x} * kChunkRows;
    const int chunk_rows = static_cast<int>(rows - first < kChunkRows ? rows - first : kChunkRows);
    const int stages_total = (chunk_rows + S::kRows - 1) / S::kRows;
    const uint32_t staging = (shared_address(staging_raw) + 127u) & ~127u;
    const uint32_t bar0 = shared_address(barriers);
    auto full_bar = [&](int slot) { return bar0 + 8u * slot; };
    auto empty_bar = [&](int slot) { return bar0 + 8u * (S::kStages + slot); };

    if (ly == 0 && px == 0) {
        abort_flag = 0;
        for (int i = 0; i < S::kStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full_bar(i)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(i)),
                         "r"(kLaneRows)
                         : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    fb::dependency_wait();
    if (ly == 0 && px == 0) {
        fb::dependency_release();
    }
    if constexpr (kSource == Source::kHalfTimesXhat) {
        const int t = ly * kTilePieces + px;
        if (t < chunk_rows) {
            sh_mean[t] = mean[first + t];
            sh_rstd[t] = rstd[first + t];
        }
    }
    __syncthreads();
    volatile int* abort = &abort_flag;
    bool ok = true;
    int issued = 0;  // fetching warp: stages whose copies have been started
    fb::Comp2 acc[4];
    constexpr bool kAlsoPlainSums = kPlain && kSource == Source::kHalfTimesXhat;
    fb::F2 also[4] = {0, 0, 0, 0};

    if (ly == kLaneRows) {
        // ---- fetching warp: lane l copies row l of each stage (and its x segment) ----
        const uint32_t main_bytes = static_cast<uint32_t>(width) * S::kMainBytes;
        const uint32_t x_bytes = static_cast<uint32_t>(width) * S::kXBytes;
        for (int k = 0; k < stages_total; ++k) {
            const int slot = k % S::kStages;
            if (k >= S::kStages &&
                !staged_wait(empty_bar(slot), static_cast<uint32_t>(k / S::kStages - 1) & 1u,
                             abort)) {
                ok = false;
                break;
            }
            issued = k + 1;
            const int here = min(S::kRows, chunk_rows - k * S::kRows);
            if (maps.use != 0) {
                // One tensor load per operand: the box is always delivered whole (zeros
                // past the matrix's edges, which the adding warps never read).
                if (px == 0) {
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                     full_bar(slot)),
                                 "r"(static_cast<uint32_t>(S::kStage))
                                 : "memory");
                    const int column = first_piece * 8;
                    const int row = static_cast<int>(first) + k * S::kRows;
                    const uint32_t dst = staging + slot * S::kStage;
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                        " [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&maps.main)),
                          "r"(full_bar(slot)), "r"(column), "r"(row)
                        : "memory");
                    if constexpr (S::kXBytes != 0) {
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                            " [%0], [%1, {%3, %4}], [%2];"
                            ::"r"(dst + S::kMainStage), "l"(reinterpret_cast<uint64_t>(&maps.x)),
                              "r"(full_bar(slot)), "r"(column), "r"(row)
                            : "memory");
                    }
                }
                continue;
            }
            if (px == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                 full_bar(slot)),
                             "r"(static_cast<uint32_t>(here) * (main_bytes + x_bytes))
                             : "memory");
            }
            if (px < here) {
                const size_t at =
                    (first + static_cast<size_t>(k) * S::kRows + px) * pieces + first_piece;
                const uint32_t dst =
                    staging + slot * S::kStage + px * (kTilePieces * S::kMainBytes);
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                    ::"r"(dst), "l"(static_cast<const unsigned char*>(src) + at * S::kMainBytes),
                      "r"(main_bytes), "r"(full_bar(slot))
                    : "memory");
                if constexpr (S::kXBytes != 0) {
                    const uint32_t xdst = staging + slot * S::kStage + S::kMainStage +
                                          px * (kTilePieces * S::kXBytes);
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                        ::"r"(xdst),
                          "l"(reinterpret_cast<const unsigned char*>(x) + at * S::kXBytes),
                          "r"(x_bytes), "r"(full_bar(slot))
                        : "memory");
                }
            }
        }
    } else {
        // ---- adding warps ----
        auto load16 = [](uint4& q, uint32_t at) {
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                         : "r"(at));
        };
        auto pair_of = [](uint32_t lo, uint32_t hi) {
            return static_cast<fb::F2>(lo) | (static_cast<fb::F2>(hi) << 32);
        };
        for (int k = 0; k < stages_total; ++k) {
            const int slot = k % S::kStages;
            if (!staged_wait(full_bar(slot), static_cast<uint32_t>(k / S::kStages) & 1u, abort)) {
                ok = false;
                break;
            }
            const int here = min(S::kRows, chunk_rows - k * S::kRows);
            const uint32_t stage = staging + slot * S::kStage;
            if (px < width) {
#pragma unroll
                for (int j = 0; j < S::kRows / kLaneRows; ++j) {
                    const int row = ly + kLaneRows * j;  // row inside the stage
                    if (row >= here) {
                        break;
                    }
                    fb::F2 v[4];
                    const uint32_t at =
                        stage + row * (kTilePieces * S::kMainBytes) + px * S::kMainBytes;
                    uint4 a;
                    load16(a, at);
                    if constexpr (kSource == Source::kFloat) {
                        uint4 b;
                        load16(b, at + 16);
                        v[0] = pair_of(a.x, a.y);
                        v[1] = pair_of(a.z, a.w);
                        v[2] = pair_of(b.x, b.y);
                        v[3] = pair_of(b.z, b.w);
                    } else {
                        float f[8];
                        fb::unpack8(f, a);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            v[c] = fb::f2_pack(f[2 * c], f[2 * c + 1]);
                        }
                    }
                    if constexpr (kSource == Source::kHalfTimesXhat) {
                        uint4 x0;
                        uint4 x1;
                        const uint32_t xat = stage + S::kMainStage +
                                             row * (kTilePieces * S::kXBytes) + px * S::kXBytes;
                        load16(x0, xat);
                        load16(x1, xat + 16);
                        const fb::F2 xs[4] = {pair_of(x0.x, x0.y), pair_of(x0.z, x0.w),
                                              pair_of(x1.x, x1.y), pair_of(x1.z, x1.w)};
                        const float m = sh_mean[k * S::kRows + row];
                        const float rs = sh_rstd[k * S::kRows + row];
                        const fb::F2 m2 = fb::f2_pack(m, m);
                        const fb::F2 rs2 = fb::f2_pack(rs, rs);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const fb::F2 xhat = fb::f2_mul(fb::f2_sub(xs[c], m2), rs2);
                            if constexpr (kPlain) {
                                acc[c].s = fb::f2_fma(v[c], xhat, acc[c].s);
                                also[c] = fb::f2_add(also[c], v[c]);
                            } else {
                                fb::comp_add_product2(acc[c], v[c], xhat);
                            }
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            if constexpr (kPlain) {
                                acc[c].s = fb::f2_add(acc[c].s, v[c]);
                            } else {
                                fb::comp_add2(acc[c], v[c]);
                            }
                        }
                    }
                }
            }
            // This warp is done with the slot; the fetching warp refills it once all eight are.
            __syncwarp();
            if (px == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(slot))
                             : "memory");
            }
        }
    }
    if (!ok && px == 0) {
        atomicExch(&g_reduction_error, 1);
    }
    __syncthreads();
    if (abort_flag != 0) {
        // A wait gave up (the flag was written before the barrier above, so every thread
        // sees the same value). The error word is set; this CTA writes no sums. Before it
        // leaves, the fetching warp waits, again with a limit, for the copies it started
        // into the ring: shared memory must not be handed to another CTA with a copy
        // still on its way.
        if (ly == kLaneRows && px == 0) {
            for (int k = max(0, issued - S::kStages); k < issued; ++k) {
                int unused = 0;
                staged_wait(full_bar(k % S::kStages), static_cast<uint32_t>(k / S::kStages) & 1u,
                            &unused);
            }
        }
        return;
    }
    // Every stage has been consumed: the ring's memory now carries the eight streams'
    // (sum, error) pairs to stream 0, which merges them in stream order.
    float* sh_s = reinterpret_cast<float*>(staging_raw + (staging - shared_address(staging_raw)));
    float* sh_e = sh_s + kLaneRows * kTilePieces * 8;
    const size_t block_quads = size_t{gridDim.x} * pieces * 4;  // float4s in one block of partials
#pragma unroll
    for (int set = 0; set < (kAlsoPlainSums ? 2 : 1); ++set) {
        if (set == 1) {
            __syncthreads();  // stream 0 has read the first set
        }
        if (ly < kLaneRows) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float lo, hi;
                fb::f2_unpack(set == 0 ? acc[c].s : also[c], lo, hi);
                sh_s[(ly * kTilePieces + px) * 8 + 2 * c] = lo;
                sh_s[(ly * kTilePieces + px) * 8 + 2 * c + 1] = hi;
                fb::f2_unpack(set == 0 ? acc[c].e : fb::F2{0}, lo, hi);
                sh_e[(ly * kTilePieces + px) * 8 + 2 * c] = lo;
                sh_e[(ly * kTilePieces + px) * 8 + 2 * c + 1] = hi;
            }
        }
        __syncthreads();
        if (ly != 0 || piece >= pieces) {
            continue;
        }
        Comp total[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            total[j].s = sh_s[px * 8 + j];
            total[j].e = sh_e[px * 8 + j];
        }
        for (int other = 1; other < kLaneRows; ++other) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                fb::comp_merge(total[j], sh_s[(other * kTilePieces + px) * 8 + j],
                               sh_e[(other * kTilePieces + px) * 8 + j]);
            }
        }
        // Chunk c occupies rows 2c (sums) and 2c+1 (errors) of a [2*chunks, cols] FP32 matrix.
        float4* out = partial + set * block_quads + size_t{blockIdx.x} * pieces * 4 + size_t(piece) * 2;
        out[0] = make_float4(total[0].s, total[1].s, total[2].s, total[3].s);
        out[1] = make_float4(total[4].s, total[5].s, total[6].s, total[7].s);
        out += size_t(pieces) * 2;
        out[0] = make_float4(total[0].e, total[1].e, total[2].e, total[3].e);
        out[1] = make_float4(total[4].e, total[5].e, total[6].e, total[7].e);
    }
}

// Second pass: a warp per 4 columns.
constexpr int kFinishWarps = 8;

// The sums of columns [4 quad, 4 quad + 4) over all chunks, by one warp.
__device__ __forceinline__ void finish_quad(float4* __restrict__ out,
                                            const float4* __restrict__ partial, size_t chunks,
                                            int quads, int quad, bool accumulate) {
    const int lane = threadIdx.x % 32;
    Comp total[4];
    for (size_t chunk = lane; chunk < chunks; chunk += 32) {
        const float4* row = partial + chunk * quads * 2;
        const float4 s = row[quad];
        const float4 e = row[quads + quad];
        fb::comp_merge(total[0], s.x, e.x);
        fb::comp_merge(total[1], s.y, e.y);
        fb::comp_merge(total[2], s.z, e.z);
        fb::comp_merge(total[3], s.w, e.w);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float os[4];
        float oe[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            os[j] = __shfl_xor_sync(fb::kFullMask, total[j].s, off);
            oe[j] = __shfl_xor_sync(fb::kFullMask, total[j].e, off);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            fb::comp_merge(total[j], os[j], oe[j]);
        }
    }
    if (lane != 0) {
        return;
    }
    float4 result = make_float4(fb::comp_value(total[0]), fb::comp_value(total[1]),
                                fb::comp_value(total[2]), fb::comp_value(total[3]));
    if (accumulate) {
        const float4 old = out[quad];
        result = make_float4(__fadd_rn(old.x, result.x), __fadd_rn(old.y, result.y),
                             __fadd_rn(old.z, result.z), __fadd_rn(old.w, result.w));
    }
    out[quad] = result;
}

__global__ void __launch_bounds__(32 * kFinishWarps)
    fb_column_finish(float4* __restrict__ out, const float4* __restrict__ partial, size_t chunks,
                     int quads, bool accumulate) {
    fb::dependency_wait();
    fb::dependency_release();
    const int quad = blockIdx.x * kFinishWarps + threadIdx.x / 32;
    if (quad < quads) {
        finish_quad(out, partial, chunks, quads, quad, accumulate);
    }
}

// Several second passes in one launch: job j owns blocks [first_block[j], first_block[j + 1]).
struct FinishJobs {
    float4* out[fb::ColumnFinishList::kMost];
    const float4* partial[fb::ColumnFinishList::kMost];
    int quads[fb::ColumnFinishList::kMost];
    int first_block[fb::ColumnFinishList::kMost + 1];
    unsigned accumulate;  // bit j
    int count;
};

__global__ void __launch_bounds__(32 * kFinishWarps)
    fb_column_finish_many(const __grid_constant__ FinishJobs jobs, size_t chunks) {
    fb::dependency_wait();
    fb::dependency_release();
    int j = 0;
    while (j + 1 < jobs.count && static_cast<int>(blockIdx.x) >= jobs.first_block[j + 1]) {
        ++j;
    }
    const int quad =
        (static_cast<int>(blockIdx.x) - jobs.first_block[j]) * kFinishWarps + threadIdx.x / 32;
    if (quad < jobs.quads[j]) {
        finish_quad(jobs.out[j], jobs.partial[j], chunks, jobs.quads[j], quad,
                    ((jobs.accumulate >> j) & 1u) != 0);
    }
}

template <Source kSource, bool kPlain = false>
cudaError_t launch_partials(void* workspace, const void* src, const void* x, const void* mean,
                            const void* rstd, size_t rows, size_t cols, cudaStream_t stream) {
    const unsigned chunks = static_cast<unsigned>((rows + kChunkRows - 1) / kChunkRows);
    const int pieces = static_cast<int>(cols / 8);
    const unsigned tiles = static_cast<unsigned>((pieces + kTilePieces - 1) / kTilePieces);
    constexpr int kDynamic = Staging<kSource>::kBytes;
    static std::atomic<bool> configured[64] = {};  // per instantiation and device
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        return e;
    }
    if (device >= 64 || !configured[device].load(std::memory_order_relaxed)) {
        e = cudaFuncSetAttribute(fb_column_partials<kSource, kPlain>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamic);
        if (e != cudaSuccess) {
            return e;
        }
        if (device < 64) {
            configured[device].store(true, std::memory_order_relaxed);
        }
    }
    ColumnMaps maps;
    maps.use = rows < (size_t{1} << 31) ? 1 : 0;
    if (maps.use != 0) {
        using S = Staging<kSource>;
        e = fb::encode_rows_map(&maps.main, src, rows, cols, S::kMainBytes / 8, kTilePieces * 8,
                                S::kRows);
        if (e == cudaSuccess && S::kXBytes != 0) {
            e = fb::encode_rows_map(&maps.x, x, rows, cols, 4, kTilePieces * 8, S::kRows);
        }
        if (e != cudaSuccess) {
            return e;
        }
    }
    return fb::launch_dependent(fb_column_partials<kSource, kPlain>, dim3(chunks, tiles),
                                dim3(kTilePieces, kLaneRows + 1), kDynamic, stream, maps,
                                static_cast<float4*>(workspace), src, static_cast<const float4*>(x),
                                static_cast<const float*>(mean), static_cast<const float*>(rstd),
                                rows, pieces);
}

cudaError_t launch_finish(void* out, const void* workspace, size_t rows, size_t cols,
                          bool accumulate, cudaStream_t stream) {
    const size_t chunks = (rows + kChunkRows - 1) / kChunkRows;
    const int quads = static_cast<int>(cols / 4);
    const unsigned blocks = static_cast<unsigned>((quads + kFinishWarps - 1) / kFinishWarps);
    return fb::launch_dependent(fb_column_finish, dim3(blocks), dim3(32 * kFinishWarps), 0, stream,
                                static_cast<float4*>(out), static_cast<const float4*>(workspace),
                                chunks, quads, accumulate);
}

// ---- LayerNorm backward: dx -----------------------------------------------------

constexpr int kWarpsPerBlock = 8;

// A warp per row, lane l owning the 8-column pieces l, l+32, ... kPieces > 0:
// the lane keeps its pieces of dy and x in registers (rows up to 256*kPieces
// wide) and the row is read once; kPieces == 0 re-reads the row for the
// second pass.
template <int kPieces>
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
    fb_layernorm_backward_dx(float4* __restrict__ dx, const uint4* __restrict__ dy,
                             const float4* __restrict__ x, const float* __restrict__ mean,
                             const float* __restrict__ rstd, const float4* __restrict__ gamma,
                             size_t rows, int pieces, bool accumulate, uint4* __restrict__ dx_half) {
    fb::dependency_wait();
    fb::dependency_release();
    const size_t row = size_t{blockIdx.x} * kWarpsPerBlock + threadIdx.x / 32;
    if (row >= rows) {
        return;
    }
    const int lane = threadIdx.x % 32;
    const uint4* dyr = dy + row * pieces;
    const float4* xr = x + row * pieces * 2;
    float4* dxr = dx + row * pieces * 2;
    const float m = mean[row];
    const float rs = rstd[row];
    const float n = static_cast<float>(pieces * 8);

    float g_sum = 0.0f;
    float gx_sum = 0.0f;
    if constexpr (kPieces > 0) {
        float g[kPieces][8];
        float xh[kPieces][8];
#pragma unroll
        for (int k = 0; k < kPieces; ++k) {
            const int i = lane + 32 * k;
            if (i < pieces) {
                float d[8];
                float xs[8];
                float gs[8];
                fb::unpack8(d, dyr[i]);
                fb::load8(xs, xr + 2 * i);
                fb::load8(gs, gamma + 2 * i);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    g[k][j] = __fmul_rn(d[j], gs[j]);
                    xh[k][j] = __fmul_rn(__fsub_rn(xs[j], m), rs);
                    g_sum = __fadd_rn(g_sum, g[k][j]);
                    gx_sum = __fadd_rn(gx_sum, __fmul_rn(g[k][j], xh[k][j]));
                }
            }
        }
        const float g_mean = __fdiv_rn(fb::warp_sum_rn(g_sum), n);
        const float gx_mean = __fdiv_rn(fb::warp_sum_rn(gx_sum), n);
#pragma unroll
        for (int k = 0; k < kPieces; ++k) {
            const int i = lane + 32 * k;
            if (i < pieces) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j] = __fmul_rn(rs, __fsub_rn(__fsub_rn(g[k][j], g_mean),
                                                   __fmul_rn(xh[k][j], gx_mean)));
                }
                if (accumulate) {
                    float old[8];
                    fb::load8(old, dxr + 2 * i);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        o[j] = __fadd_rn(old[j], o[j]);
                    }
                }
                fb::store8(dxr + 2 * i, o);
                if (dx_half != nullptr) {
                    dx_half[row * pieces + i] = fb::pack8(o);  // the same values, rounded once
                }
            }
        }
    } else {
        for (int i = lane; i < pieces; i += 32) {
            float d[8];
            float xs[8];
            float gs[8];
            fb::unpack8(d, dyr[i]);
            fb::load8(xs, xr + 2 * i);
            fb::load8(gs, gamma + 2 * i);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float g = __fmul_rn(d[j], gs[j]);
                g_sum = __fadd_rn(g_sum, g);
                gx_sum = __fadd_rn(gx_sum, __fmul_rn(g, __fmul_rn(__fsub_rn(xs[j], m), rs)));
            }
        }
        const float g_mean = __fdiv_rn(fb::warp_sum_rn(g_sum), n);
        const float gx_mean = __fdiv_rn(fb::warp_sum_rn(gx_sum), n);
        for (int i = lane; i < pieces; i += 32) {
            float d[8];
            float xs[8];
            float gs[8];
            fb::unpack8(d, dyr[i]);
            fb::load8(xs, xr + 2 * i);
            fb::load8(gs, gamma + 2 * i);
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float g = __fmul_rn(d[j], gs[j]);
                const float xhat = __fmul_rn(__fsub_rn(xs[j], m), rs);
                o[j] = __fmul_rn(rs, __fsub_rn(__fsub_rn(g, g_mean), __fmul_rn(xhat, gx_mean)));
            }
            if (accumulate) {
                float old[8];
                fb::load8(old, dxr + 2 * i);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j] = __fadd_rn(old[j], o[j]);
                }
            }
            fb::store8(dxr + 2 * i, o);
            if (dx_half != nullptr) {
                dx_half[row * pieces + i] = fb::pack8(o);
            }
        }
    }
}

// ---- embedding backward: bucket the rows by token -----------------------------------
//
// A stable least-significant-digit radix sort of (token, row) pairs by the
// 16-bit token, in two passes of 8 bits. Rows start in ascending order and both
// passes are stable, so a token's rows end up ascending, which fixes the order
// of its sum. Per pass: count digits per tile of 2,048 rows, one exclusive scan
// over (digit, tile), then a ranked scatter. Integer counting only.

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr size_t kSortTileRows = 2048;
constexpr int kRowsPerWarp = static_cast<int>(kSortTileRows) / kSortWarps;
constexpr int kDigits = 256;
constexpr unsigned kNoDigit = 0xffffffffu;

struct EmbeddingLayout {
    size_t sorted_tokens, sorted_rows, offsets, pass_tokens, pass_rows, counts, bytes;
};

constexpr size_t align16(size_t v) { return (v + 15) / 16 * 16; }

// Byte offsets of the workspace's parts: position partials first, then the
// sorted tokens (u16) and rows (u32), offsets[vocab + 1] (u32), the first
// pass's tokens and rows, and 256 u32 counters per tile.
EmbeddingLayout embedding_layout(size_t sequences, size_t length, size_t vocab, size_t width) {
    const size_t rows = sequences * length;
    const size_t tiles = (rows + kSortTileRows - 1) / kSortTileRows;
    EmbeddingLayout l{};
    size_t at = align16(column_sum_workspace(sequences, length * width));
    l.sorted_tokens = at;
    at += align16(rows * 2);
    l.sorted_rows = at;
    at += align16(rows * 4);
    l.offsets = at;
    at += align16((vocab + 1) * 4);
    l.pass_tokens = at;
    at += align16(rows * 2);
    l.pass_rows = at;
    at += align16(rows * 4);
    l.counts = at;
    at += align16(tiles * kDigits * 4);
    l.bytes = at;
    return l;
}

// The lowest lane of a group of lanes that share a digit.
__device__ __forceinline__ bool rank_leader(unsigned peers, int lane) {
    return lane == __ffs(peers) - 1;
}

__device__ __forceinline__ unsigned digit_at(const uint16_t* tokens, size_t i, size_t rows,
                                             int shift) {
    return i < rows ? (static_cast<unsigned>(tokens[i]) >> shift) & (kDigits - 1) : kNoDigit;
}

// counts[digit * tiles + tile] = rows of this tile with that digit.
__global__ void __launch_bounds__(kSortThreads)
    fb_sort_count(unsigned* __restrict__ counts, const uint16_t* __restrict__ tokens, size_t rows,
                  int shift) {
    __shared__ unsigned histogram[kDigits];
    histogram[threadIdx.x] = 0;
    __syncthreads();
    const size_t base = size_t{blockIdx.x} * kSortTileRows;
    for (int i = threadIdx.x; i < static_cast<int>(kSortTileRows); i += kSortThreads) {
        const unsigned digit = digit_at(tokens, base + i, rows, shift);
        if (digit != kNoDigit) {
            atomicAdd(&histogram[digit], 1u);  // integer: the total is order-independent
        }
    }
    __syncthreads();
    counts[size_t{threadIdx.x} * gridDim.x + blockIdx.x] = histogram[threadIdx.x];
}

// In-place exclusive prefix sum of `entries` counters by one CTA of 1,024 threads.
__global__ void __launch_bounds__(1024) fb_sort_scan(unsigned* __restrict__ counts, size_t entries) {
    __shared__ unsigned warp_totals[32];
    __shared__ unsigned carry_shared;
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    if (threadIdx.x == 0) {
        carry_shared = 0;
    }
    __syncthreads();
    for (size_t base = 0; base < entries; base += 1024) {
        const size_t i = base + threadIdx.x;
        const unsigned v = i < entries ? counts[i] : 0;
        unsigned inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const unsigned o = __shfl_up_sync(fb::kFullMask, inc, off);
            if (lane >= off) {
                inc += o;
            }
        }
        if (lane == 31) {
            warp_totals[warp] = inc;
        }
        __syncthreads();
        if (warp == 0) {
            unsigned w = warp_totals[lane];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned o = __shfl_up_sync(fb::kFullMask, w, off);
                if (lane >= off) {
                    w += o;
                }
            }
            warp_totals[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const unsigned carry = carry_shared;
        const unsigned before = warp == 0 ? 0 : warp_totals[warp - 1];
        if (i < entries) {
            counts[i] = carry + before + inc - v;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry_shared = carry + warp_totals[31];
        }
        __syncthreads();
    }
}

// Moves a tile's (token, row) pairs to their positions for this digit. Warp w
// handles rows [256 w, 256 w + 256) of the tile, 32 at a time in order, so
// equal digits keep their input order.
__global__ void __launch_bounds__(kSortThreads)
    fb_sort_scatter(uint16_t* __restrict__ out_tokens, unsigned* __restrict__ out_rows,
                    const uint16_t* __restrict__ in_tokens, const unsigned* __restrict__ in_rows,
                    const unsigned* __restrict__ starts, size_t rows, int shift) {
    __shared__ unsigned next[kSortWarps][kDigits];
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    for (int w = 0; w < kSortWarps; ++w) {
        next[w][threadIdx.x] = 0;
    }
    __syncthreads();
    const size_t first = size_t{blockIdx.x} * kSortTileRows + size_t(warp) * kRowsPerWarp;
    // Each warp's digit counts.
    for (int step = 0; step < kRowsPerWarp / 32; ++step) {
        const unsigned digit = digit_at(in_tokens, first + step * 32 + lane, rows, shift);
        if (digit != kNoDigit) {
            atomicAdd(&next[warp][digit], 1u);
        }
    }
    __syncthreads();
    // Thread d turns digit d's per-warp counts into per-warp start positions.
    unsigned position = starts[size_t{threadIdx.x} * gridDim.x + blockIdx.x];
    for (int w = 0; w < kSortWarps; ++w) {
        const unsigned c = next[w][threadIdx.x];
        next[w][threadIdx.x] = position;
        position += c;
    }
    __syncthreads();
    for (int step = 0; step < kRowsPerWarp / 32; ++step) {
        const size_t i = first + step * 32 + lane;
        const unsigned digit = digit_at(in_tokens, i, rows, shift);
        const unsigned peers = __match_any_sync(fb::kFullMask, digit);
        if (digit != kNoDigit) {
            const unsigned rank = __popc(peers & ((1u << lane) - 1u));
            const unsigned at = next[warp][digit] + rank;
            out_tokens[at] = in_tokens[i];
            out_rows[at] = in_rows == nullptr ? static_cast<unsigned>(i) : in_rows[i];
        }
        __syncwarp();
        if (digit != kNoDigit && rank_leader(peers, lane)) {
            next[warp][digit] += __popc(peers);
        }
        __syncwarp();
    }
}

// offsets[v] = number of sorted tokens below v, for v = 0..vocab (binary search).
__global__ void __launch_bounds__(256)
    fb_token_offsets(unsigned* __restrict__ offsets, const uint16_t* __restrict__ sorted_tokens,
                     size_t rows, unsigned vocab) {
    const unsigned v = blockIdx.x * 256 + threadIdx.x;
    if (v > vocab) {
        return;
    }
    size_t lo = 0;
    size_t hi = rows;
    while (lo < hi) {
        const size_t mid = lo + (hi - lo) / 2;
        if (sorted_tokens[mid] < v) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    offsets[v] = static_cast<unsigned>(lo);
}

// One CTA per word-table row v; each thread owns float4 columns q, q+128, ...
// and adds token v's rows of dx in ascending row order with a compensated sum.
constexpr int kWordThreads = 128;

__global__ void __launch_bounds__(kWordThreads)
    fb_word_gradient(float4* __restrict__ dwte, const float4* __restrict__ dx,
                     const unsigned* __restrict__ sorted_rows,
                     const unsigned* __restrict__ offsets, unsigned quads, bool accumulate) {
    const size_t v = blockIdx.x;
    const unsigned begin = offsets[v];
    const unsigned end = offsets[v + 1];
    if (begin == end && accumulate) {
        return;
    }
    for (unsigned q = threadIdx.x; q < quads; q += kWordThreads) {
        float4* out = dwte + v * quads + q;
        if (begin == end) {
            *out = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            continue;
        }
        Comp acc[4];
        for (unsigned k = begin; k < end; ++k) {
            const float4 d = dx[size_t{sorted_rows[k]} * quads + q];
            fb::comp_add(acc[0], d.x);
            fb::comp_add(acc[1], d.y);
            fb::comp_add(acc[2], d.z);
            fb::comp_add(acc[3], d.w);
        }
        float4 r = make_float4(fb::comp_value(acc[0]), fb::comp_value(acc[1]),
                               fb::comp_value(acc[2]), fb::comp_value(acc[3]));
        if (accumulate) {
            const float4 old = *out;
            r = make_float4(__fadd_rn(old.x, r.x), __fadd_rn(old.y, r.y), __fadd_rn(old.z, r.z),
                            __fadd_rn(old.w, r.w));
        }
        *out = r;
    }
}

flint_status check_column_dims(const char* name, size_t rows, size_t cols, bool allow_zero_cols,
                               size_t max_rows) {
    if ((cols == 0 && !allow_zero_cols) || cols % 8 != 0 || cols > kMaxCols) {
        if (allow_zero_cols) {
            return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                            "%s: cols (%zu) must be a multiple of 8 up to %zu", name, cols,
                            kMaxCols);
        }
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: cols (%zu) must be a multiple of 8 from 8 to %zu", name, cols,
                        kMaxCols);
    }
    if (rows == 0 || rows > max_rows) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: rows (%zu) must be from 1 to %zu", name,
                        rows, max_rows);
    }
    return FLINT_OK;
}

flint_status check_embedding_dims(const char* name, size_t sequences, size_t length, size_t vocab,
                                  size_t width) {
    constexpr size_t kMaxVocab = size_t{1} << 16;
    constexpr size_t kMaxSortRows = 0xffffffffu;
    if (width == 0 || width % 8 != 0 || width > kMaxCols) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: width (%zu) must be a multiple of 8 from 8 to %zu", name, width,
                        kMaxCols);
    }
    if (vocab == 0 || vocab > kMaxVocab) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: vocab (%zu) must be from 1 to %zu",
                        name, vocab, kMaxVocab);
    }
    if (length == 0 || length > kMaxCols / width) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: length (%zu) must be from 1 to %zu, so that length x width (%zu) "
                        "is at most %zu",
                        name, length, kMaxCols / width, width, kMaxCols);
    }
    if (sequences == 0 || sequences > kMaxSortRows / length) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: sequences (%zu) must be from 1 to %zu, so that sequences x length "
                        "is at most %zu rows",
                        name, sequences, kMaxSortRows / length, kMaxSortRows);
    }
    return FLINT_OK;
}

}  // namespace

namespace fb {

cudaError_t reductions_error_flag(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_reduction_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_reduction_error, &zero, sizeof(int));
    }
    return e;
}

// Internal launchers, also used by the model assembly.
size_t column_partial_bytes(size_t rows, size_t cols) { return column_sum_workspace(rows, cols); }

cudaError_t launch_column_finishes(const ColumnFinishList& list, size_t rows, cudaStream_t stream) {
    if (list.count == 0) {
        return cudaSuccess;
    }
    FinishJobs jobs = {};
    jobs.count = list.count;
    int blocks = 0;
    for (int j = 0; j < list.count; ++j) {
        const ColumnFinishList::Job& job = list.jobs[j];
        jobs.out[j] = static_cast<float4*>(job.out);
        jobs.partial[j] = static_cast<const float4*>(job.partial);
        jobs.quads[j] = static_cast<int>(job.cols / 4);
        jobs.first_block[j] = blocks;
        jobs.accumulate |= job.accumulate ? 1u << j : 0u;
        blocks += (jobs.quads[j] + kFinishWarps - 1) / kFinishWarps;
    }
    jobs.first_block[list.count] = blocks;
    const size_t chunks = (rows + kChunkRows - 1) / kChunkRows;
    return fb::launch_dependent(fb_column_finish_many, dim3(static_cast<unsigned>(blocks)),
                                dim3(32 * kFinishWarps), 0, stream, jobs, chunks);
}

namespace {
// The second pass now, or noted for launch_column_finishes.
cudaError_t finish_or_defer(void* out, const void* workspace, size_t rows, size_t cols,
                            bool accumulate, cudaStream_t stream, ColumnFinishList* later) {
    if (later == nullptr) {
        return launch_finish(out, workspace, rows, cols, accumulate, stream);
    }
    return later->add(out, workspace, cols, accumulate) ? cudaSuccess : cudaErrorInvalidValue;
}
}  // namespace

cudaError_t launch_bias_gradient(void* dbias, const void* dy, size_t rows, size_t cols,
                                 bool accumulate, void* workspace, cudaStream_t stream,
                                 bool plain, ColumnFinishList* later) {
    cudaError_t e =
        plain ? launch_partials<Source::kHalf, true>(workspace, dy, nullptr, nullptr, nullptr, rows,
                                                     cols, stream)
              : launch_partials<Source::kHalf>(workspace, dy, nullptr, nullptr, nullptr, rows, cols,
                                               stream);
    if (e != cudaSuccess) {
        return e;
    }
    return finish_or_defer(dbias, workspace, rows, cols, accumulate, stream, later);
}

cudaError_t launch_layernorm_backward(void* dx, void* dgamma, void* dbeta, const void* dy,
                                      const void* x, const void* mean, const void* rstd,
                                      const void* gamma, size_t rows, size_t cols,
                                      bool accumulate_dx, bool accumulate_params, void* workspace,
                                      cudaStream_t stream, void* dx_half, bool plain,
                                      ColumnFinishList* later) {
    cudaError_t e = cudaSuccess;
    if (plain) {
        // One pass over dy serves both parameter gradients: dgamma's partial sums fill the
        // first block of the workspace, dbeta's the second (the caller provides twice the
        // public workspace size for this variant).
        e = launch_partials<Source::kHalfTimesXhat, true>(workspace, dy, x, mean, rstd, rows, cols,
                                                          stream);
        if (e != cudaSuccess) {
            return e;
        }
        e = finish_or_defer(dgamma, workspace, rows, cols, accumulate_params, stream, later);
        if (e != cudaSuccess) {
            return e;
        }
        e = finish_or_defer(dbeta,
                            static_cast<unsigned char*>(workspace) + column_sum_workspace(rows, cols),
                            rows, cols, accumulate_params, stream, later);
        if (e != cudaSuccess) {
            return e;
        }
    } else {
        // dbeta first; its second pass is done with the workspace before dgamma's
        // partial sums reuse it (stream order).
        e = launch_bias_gradient(dbeta, dy, rows, cols, accumulate_params, workspace, stream,
                                 false);
        if (e != cudaSuccess) {
            return e;
        }
        e = launch_partials<Source::kHalfTimesXhat>(workspace, dy, x, mean, rstd, rows, cols,
                                                    stream);
        if (e != cudaSuccess) {
            return e;
        }
        e = launch_finish(dgamma, workspace, rows, cols, accumulate_params, stream);
        if (e != cudaSuccess) {
            return e;
        }
    }
    const int pieces = static_cast<int>(cols / 8);
    const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto* dxq = static_cast<float4*>(dx);
    const auto* dyq = static_cast<const uint4*>(dy);
    const auto* xq = static_cast<const float4*>(x);
    const auto* mf = static_cast<const float*>(mean);
    const auto* rf = static_cast<const float*>(rstd);
    const auto* gq = static_cast<const float4*>(gamma);
    if (pieces <= 32) {
        e = fb::launch_dependent(fb_layernorm_backward_dx<1>, dim3(blocks), dim3(32 * kWarpsPerBlock), 0,
                                 stream, dxq, dyq, xq, mf, rf, gq, rows, pieces, accumulate_dx,
                                 static_cast<uint4*>(dx_half));
    } else if (pieces <= 96) {
        e = fb::launch_dependent(fb_layernorm_backward_dx<3>, dim3(blocks), dim3(32 * kWarpsPerBlock), 0,
                                 stream, dxq, dyq, xq, mf, rf, gq, rows, pieces, accumulate_dx,
                                 static_cast<uint4*>(dx_half));
    } else if (pieces <= 192) {
        e = fb::launch_dependent(fb_layernorm_backward_dx<6>, dim3(blocks), dim3(32 * kWarpsPerBlock), 0,
                                 stream, dxq, dyq, xq, mf, rf, gq, rows, pieces, accumulate_dx,
                                 static_cast<uint4*>(dx_half));
    } else {
        e = fb::launch_dependent(fb_layernorm_backward_dx<0>, dim3(blocks), dim3(32 * kWarpsPerBlock), 0,
                                 stream, dxq, dyq, xq, mf, rf, gq, rows, pieces, accumulate_dx,
                                 static_cast<uint4*>(dx_half));
    }
    return e;
}

cudaError_t launch_embedding_backward(void* dwte, void* dwpe, const void* dx, const void* tokens,
                                      size_t sequences, size_t length, size_t vocab, size_t width,
                                      bool accumulate_wte, bool accumulate_wpe, void* workspace,
                                      cudaStream_t stream) {
    const size_t rows = sequences * length;
    const EmbeddingLayout l = embedding_layout(sequences, length, vocab, width);
    auto* base = static_cast<unsigned char*>(workspace);
    auto* sorted_tokens = reinterpret_cast<uint16_t*>(base + l.sorted_tokens);
    auto* sorted_rows = reinterpret_cast<unsigned*>(base + l.sorted_rows);
    auto* offsets = reinterpret_cast<unsigned*>(base + l.offsets);
    auto* pass_tokens = reinterpret_cast<uint16_t*>(base + l.pass_tokens);
    auto* pass_rows = reinterpret_cast<unsigned*>(base + l.pass_rows);
    auto* counts = reinterpret_cast<unsigned*>(base + l.counts);
    const auto* in_tokens = static_cast<const uint16_t*>(tokens);

    const unsigned tiles = static_cast<unsigned>((rows + kSortTileRows - 1) / kSortTileRows);
    const size_t entries = size_t{tiles} * kDigits;
    for (int pass = 0; pass < 2; ++pass) {
        const int shift = 8 * pass;
        const uint16_t* from_tokens = pass == 0 ? in_tokens : pass_tokens;
        const unsigned* from_rows = pass == 0 ? nullptr : pass_rows;
        uint16_t* to_tokens = pass == 0 ? pass_tokens : sorted_tokens;
        unsigned* to_rows = pass == 0 ? pass_rows : sorted_rows;
        fb_sort_count<<<tiles, kSortThreads, 0, stream>>>(counts, from_tokens, rows, shift);
        cudaError_t e = fb::after_launch();
        if (e != cudaSuccess) {
            return e;
        }
        fb_sort_scan<<<1, 1024, 0, stream>>>(counts, entries);
        e = fb::after_launch();
        if (e != cudaSuccess) {
            return e;
        }
        fb_sort_scatter<<<tiles, kSortThreads, 0, stream>>>(to_tokens, to_rows, from_tokens,
                                                            from_rows, counts, rows, shift);
        e = fb::after_launch();
        if (e != cudaSuccess) {
            return e;
        }
    }
    fb_token_offsets<<<static_cast<unsigned>((vocab + 1 + 255) / 256), 256, 0, stream>>>(
        offsets, sorted_tokens, rows, static_cast<unsigned>(vocab));
    cudaError_t e = fb::after_launch();
    if (e != cudaSuccess) {
        return e;
    }
    fb_word_gradient<<<static_cast<unsigned>(vocab), kWordThreads, 0, stream>>>(
        static_cast<float4*>(dwte), static_cast<const float4*>(dx), sorted_rows, offsets,
        static_cast<unsigned>(width / 4), accumulate_wte);
    e = fb::after_launch();
    if (e != cudaSuccess) {
        return e;
    }
    // The position table: dx viewed as sequences x (length * width), FP32.
    const size_t cols = length * width;
    e = launch_partials<Source::kFloat>(base, dx, nullptr, nullptr, nullptr, sequences, cols,
                                        stream);
    if (e != cudaSuccess) {
        return e;
    }
    return launch_finish(dwpe, base, sequences, cols, accumulate_wpe, stream);
}

}  // namespace fb

namespace {
// ---- a bias gradient that needs no workspace from the caller -------------------------------
//
// Some hosts cannot hand this library a workspace: a plug-in living inside an
// application that owns every byte of device memory and gives none away after
// start-up, or a serving loop whose latency budget rules out cudaMalloc (it
// synchronises the whole device). For them the partial sums of the first pass go
// into this fixed array, which is part of the library's image: every GPU that
// loads the library carries these 4 MiB until the process exits.
constexpr size_t kStaticScratchBytes = size_t{4} << 20;
static __device__ __align__(256) unsigned char g_bias_gradient_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not an address
// a kernel can use; the device address comes from cudaGetSymbolAddress, asked
// once per device while that device is current.
// Host threads may make their first calls at the same time: the cache slots are
// atomics, and two threads that both miss simply store the same address.
cudaError_t static_scratch(void** pointer) {
    constexpr int kMaxDevices = 64;
    static std::atomic<void*> cached[kMaxDevices] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        return e;
    }
    const bool slot = device >= 0 && device < kMaxDevices;
    if (slot) {
        void* known = cached[device].load(std::memory_order_relaxed);
        if (known != nullptr) {
            *pointer = known;
            return cudaSuccess;
        }
    }
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, g_bias_gradient_scratch);
    if (e != cudaSuccess) {
        return e;
    }
    if (slot) {
        cached[device].store(address, std::memory_order_relaxed);
    }
    *pointer = address;
    return cudaSuccess;
}

}  // namespace

extern "C" {

flint_status flint_bias_gradient_workspace(size_t rows, size_t cols, size_t* bytes) {
    constexpr const char* name = "flint_bias_gradient_workspace";
    if (bytes == nullptr) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: bytes is null", name);
    }
    FB_TRY(check_column_dims(name, rows, cols, true, kMaxBiasRows));
    *bytes = column_sum_workspace(rows, cols);
    return FLINT_OK;
}

flint_status flint_bias_gradient(void* dbias, const void* dy, size_t rows, size_t cols,
                                 int accumulate, void* workspace, size_t workspace_bytes,
                                 flint_stream stream) {
    constexpr const char* name = "flint_bias_gradient";
    FB_TRY(check_column_dims(name, rows, cols, true, kMaxBiasRows));
    if (cols == 0) {
        return FLINT_OK;
    }
    const size_t needed = column_sum_workspace(rows, cols);
    if (workspace_bytes < needed) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: needs %zu bytes of workspace, given %zu", name, needed,
                        workspace_bytes);
    }
    const fb::Span spans[] = {
        {"dbias", dbias, cols * 4},
        {"workspace", workspace, needed},
        {"dy", dy, rows * cols * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 2));
    FB_CUDA(fb::launch_bias_gradient(dbias, dy, rows, cols, accumulate != 0, workspace, stream,
                                     false));
    return FLINT_OK;
}

flint_status flint_b200_bias_gradient_static(void* dbias, const void* dy, size_t rows, size_t cols,
                                             int accumulate, flint_stream stream) {
    constexpr const char* name = "flint_b200_bias_gradient_static";
    FB_TRY(check_column_dims(name, rows, cols, true, kMaxBiasRows));
    if (cols == 0) {
        return FLINT_OK;
    }
    const size_t needed = column_sum_workspace(rows, cols);
    if (needed > kStaticScratchBytes) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: rows (%zu) x cols (%zu) needs %zu bytes of scratch, and the built-in "
                        "scratch holds %zu; use flint_bias_gradient with a workspace",
                        name, rows, cols, needed, kStaticScratchBytes);
    }
    // Arguments are judged before any CUDA call, like everywhere else in the library.
    const fb::Span spans[] = {
        {"dbias", dbias, cols * 4},
        {"dy", dy, rows * cols * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 1));
    void* scratch = nullptr;
    FB_CUDA(static_scratch(&scratch));
    // The first pass overwrites every partial sum the second pass reads, so what an
    // earlier call left in the array never matters and nothing needs clearing.
    FB_CUDA(fb::launch_bias_gradient(dbias, dy, rows, cols, accumulate != 0, scratch, stream,
                                     false));
    return FLINT_OK;
}

flint_status flint_layernorm_backward_workspace(size_t rows, size_t cols, size_t* bytes) {
    constexpr const char* name = "flint_layernorm_backward_workspace";
    if (bytes == nullptr) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: bytes is null", name);
    }
    FB_TRY(check_column_dims(name, rows, cols, false, kMaxRows8));
    *bytes = column_sum_workspace(rows, cols);
    return FLINT_OK;
}

flint_status flint_layernorm_backward(void* dx, void* dgamma, void* dbeta, const void* dy,
                                      const void* x, const void* mean, const void* rstd,
                                      const void* gamma, size_t rows, size_t cols,
                                      int accumulate_dx, int accumulate_params, void* workspace,
                                      size_t workspace_bytes, flint_stream stream) {
    constexpr const char* name = "flint_layernorm_backward";
    FB_TRY(check_column_dims(name, rows, cols, false, kMaxRows8));
    const size_t needed = column_sum_workspace(rows, cols);
    if (workspace_bytes < needed) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: needs %zu bytes of workspace, given %zu", name, needed,
                        workspace_bytes);
    }
    const fb::Span spans[] = {
        {"dx", dx, rows * cols * 4},       {"dgamma", dgamma, cols * 4},
        {"dbeta", dbeta, cols * 4},        {"workspace", workspace, needed},
        {"dy", dy, rows * cols * 2},       {"x", x, rows * cols * 4},
        {"mean", mean, rows * 4},          {"rstd", rstd, rows * 4},
        {"gamma", gamma, cols * 4},
    };
    FB_TRY(fb::check_spans(name, spans, 4));
    FB_CUDA(fb::launch_layernorm_backward(dx, dgamma, dbeta, dy, x, mean, rstd, gamma, rows, cols,
                                          accumulate_dx != 0, accumulate_params != 0, workspace,
                                          stream, nullptr, false));
    return FLINT_OK;
}

flint_status flint_embedding_backward_workspace(size_t sequences, size_t length, size_t vocab,
                                                size_t width, size_t* bytes) {
    constexpr const char* name = "flint_embedding_backward_workspace";
    if (bytes == nullptr) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT, "%s: bytes is null", name);
    }
    FB_TRY(check_embedding_dims(name, sequences, length, vocab, width));
    *bytes = embedding_layout(sequences, length, vocab, width).bytes;
    return FLINT_OK;
}

flint_status flint_embedding_backward(void* dwte, void* dwpe, const void* dx, const void* tokens,
                                      size_t sequences, size_t length, size_t vocab, size_t width,
                                      int accumulate_wte, int accumulate_wpe, void* workspace,
                                      size_t workspace_bytes, flint_stream stream) {
    constexpr const char* name = "flint_embedding_backward";
    FB_TRY(check_embedding_dims(name, sequences, length, vocab, width));
    const size_t needed = embedding_layout(sequences, length, vocab, width).bytes;
    if (workspace_bytes < needed) {
        return fb::fail(FLINT_ERROR_INVALID_ARGUMENT,
                        "%s: needs %zu bytes of workspace, given %zu", name, needed,
                        workspace_bytes);
    }
    const size_t rows = sequences * length;
    const fb::Span spans[] = {
        {"dwte", dwte, vocab * width * 4},   {"dwpe", dwpe, length * width * 4},
        {"workspace", workspace, needed},    {"dx", dx, rows * width * 4},
        {"tokens", tokens, rows * 2},
    };
    FB_TRY(fb::check_spans(name, spans, 3));
    FB_CUDA(fb::launch_embedding_backward(dwte, dwpe, dx, tokens, sequences, length, vocab, width,
                                          accumulate_wte != 0, accumulate_wpe != 0, workspace,
                                          stream));
    return FLINT_OK;
}

}  // extern "C"
