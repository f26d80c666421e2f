// Fused causal attention for head width 64 on the 5th-generation tensor cores
// (extension; the reference materialises scores and probabilities instead,
// src/api/gpt2.cpp:495-530 and :559-618, and lists flash attention as planned).
//
// Three kernels, all warp-specialised like the GEMM (warp 0 = TMA producer,
// warp 1 = tcgen05.mma issuer, the rest compute on accumulators read from
// tensor memory), all persistent (one CTA per SM over a work-ordered item list):
//   forward   items of (head, two adjacent 128-query tiles) sharing the K and V
//             tiles that stream through a ring: S = Q K^T into TMEM, base-2
//             softmax in registers, P written back over S as FP16 pairs and read
//             from tensor memory as the A operand of O += P V, which accumulates
//             in TMEM over the row of key tiles (rescaled only when the running
//             maximum moves by more than 2^8); the two query tiles alternate on
//             the tensor pipe, one's softmax under the other's MMAs
//   dK/dV     items of (head, 128 keys) over 64-query sub-steps from the diagonal
//             on: S^T and dP^T = V dO^T recomputed with K and V in tensor memory,
//             P^T and dS^T written back over them, dV += P^T dO and
//             dK += dS^T Q accumulated in TMEM
//   dQ        items of (head, 128 queries) over 64-key sub-steps:
//             dQ += dS K accumulated in TMEM
// dQ has its own kernel so that no gradient needs atomics: every output element
// is produced by one CTA in a fixed order, so results are deterministic.
//
// Q, K, V, O and their gradients are addressed through strided 4-D tensor maps
// (column, row, head, sequence), so the same kernels read the heads layout
// [B, H, T, 64] or GPT-2's packed qkv rows [B*T, 3*H*64] without a split/merge
// pass. Softmax runs in base 2: t = s * scale * log2(e), p = 2^(t - max).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>

#include <cuda.h>
#include <cuda_fp16.h>

#include "attention.h"
#include "common.h"
#include "device_utils.cuh"
#include "flint/flint_b200.h"
#include "sm100.cuh"

namespace fb {
namespace {

constexpr int kTile = 128;     // queries and keys per tile
constexpr int kHead = 64;      // head width
constexpr int kTileBytes = kTile * kHead * 2;  // 16 KB: one Q/K/V/dO tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ int g_attention_error = 0;

struct AttnParams {
    CUtensorMap map_q, map_k, map_v, map_do;          // 128-row boxes
    CUtensorMap map_q64, map_k64, map_v64, map_do64;  // 64-row boxes (backward sub-steps)
    // Outputs and row statistics are addressed directly.
    void* out0;            // forward: O; dkv: dK; dq: dQ
    void* out1;            // dkv: dV
    long long out_row, out_head, out_seq;  // element strides of out0/out1
    float* lse;            // [seqs * heads, length]
    const float* delta;    // [seqs * heads, length]
    int length, heads, seqs, blocks;
    float scale;           // applied to the raw scores
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
          "r"(c3)
        : "memory");
}

// Untiled bulk copy global -> shared (both 16-byte aligned, bytes a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// 2^x on the special-function unit (relative error about 2^-22, flushes denormals).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// How far (in base-2 exponent units) a tile's maximum may exceed the reference exponent
// before the forward kernel moves the reference and rescales its accumulator:
// probabilities then stay below 2^8, well inside FP16.
constexpr float kLazyShift = 8.0f;

// 2^x for two values at once on the FMA pipe, for the share of the forward kernel's
// exponentials that the special-function unit has no time for: x = n + f with n the
// nearest integer (taken from the low mantissa bits of x + 1.5 * 2^23), 2^f by a
// degree-4 polynomial on [-0.5, 0.5] (relative error 2.7e-6, two orders below the FP16
// rounding of the probabilities), n added into the exponent field. x must be at most
// 127 - 1; anything below -120 counts as -120 (2^-120 is zero in FP16).
__device__ __forceinline__ void exp2_pair_fma(fb::F2 x, float& lo, float& hi) {
    float x0, x1;
    fb::f2_unpack(x, x0, x1);
    const fb::F2 clamped = fb::f2_pack(fmaxf(x0, -120.0f), fmaxf(x1, -120.0f));
    const fb::F2 magic = fb::f2_pack(12582912.0f, 12582912.0f);
    const fb::F2 z = fb::f2_add(clamped, magic);
    const fb::F2 f = fb::f2_sub(clamped, fb::f2_sub(z, magic));
    fb::F2 poly = fb::f2_fma(f, fb::f2_pack(0.009570090100169182f, 0.009570090100169182f),
                             fb::f2_pack(0.05591785907745361f, 0.05591785907745361f));
    poly = fb::f2_fma(poly, f, fb::f2_pack(0.2402474582195282f, 0.2402474582195282f));
    poly = fb::f2_fma(poly, f, fb::f2_pack(0.6931217908859253f, 0.6931217908859253f));
    poly = fb::f2_fma(poly, f, fb::f2_pack(0.9999992847442627f, 0.9999992847442627f));
    float p0, p1, z0, z1;
    fb::f2_unpack(poly, p0, p1);
    fb::f2_unpack(z, z0, z1);
    lo = __int_as_float(__float_as_int(p0) + (__float_as_int(z0) << 23));
    hi = __int_as_float(__float_as_int(p1) + (__float_as_int(z1) << 23));
}

// Of every four pairs of exponentials in the forward kernel, how many take the FMA pipe.
#ifndef FB_ATTN_FMA_EXP_OF_4
#define FB_ATTN_FMA_EXP_OF_4 1
#endif

// Two exponentials; `pair` (a compile-time constant after unrolling) picks the pipe.
#ifndef FB_ATTN_BWD_FMA_EXP_OF_4
#define FB_ATTN_BWD_FMA_EXP_OF_4 1
#endif
__device__ __forceinline__ void exp2_two(int pair, float x0, float x1, float& e0, float& e1) {
    if ((pair & 3) < FB_ATTN_BWD_FMA_EXP_OF_4) {
        exp2_pair_fma(fb::f2_pack(x0, x1), e0, e1);
    } else {
        e0 = fast_exp2(x0);
        e1 = fast_exp2(x1);
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Named barrier between the two warps that share a TMEM lane quadrant (the two
// halves of the same 32 rows); barrier 0 is __syncthreads, 1..4 are the quadrants'.
__device__ __forceinline__ void quadrant_sync(int quadrant) {
    asm volatile("bar.sync %0, 64;" ::"r"(quadrant + 1) : "memory");
}

// Descriptors for the three ways a tile is read.
// K-major tile [128 rows][64 cols] (rows = M or N index): 16-column step = 32 bytes.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kstep) {
    return sm100::smem_desc_sw128(tile + kstep * 32, 16, 1024);
}
// MN-major view of the same memory: rows are the K index, 16 rows = 2,048 bytes;
// 64-column blocks (panels) are `lbo` bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kstep, uint32_t lbo) {
    return sm100::smem_desc_sw128(tile + kstep * 2048, lbo, 1024);
}

constexpr uint32_t kIdescS = sm100::instr_desc_f16(128, 128, false, false);   // Q K^T, dO V^T
constexpr uint32_t kIdescPV = sm100::instr_desc_f16(128, 64, false, true);    // P V, dS K

__device__ __forceinline__ void finish(int abort_value, uint32_t tmem_base, uint32_t cols,
                                       int warp) {
    __syncthreads();
    if (abort_value != 0) {
        if (threadIdx.x == 0) {
            atomicExch(&g_attention_error, 1);
        }
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc(tmem_base, cols);
    }
}

// ---- forward ---------------------------------------------------------------------------
//
// Persistent CTAs, one per SM, each taking items of (128-query tile, two heads) in rounds
// from a list ordered by work (the last query tile, which sees the most keys, first). The
// two heads' tiles ("tile 0" and "tile 1" below) have the same number of key tiles and take
// turns on everything, so the CTA's work is one sequence of steps n = 0, 1, 2, ... that runs
// on across items: step n belongs to tile n & 1.
//   tensor pipe   S(n) = Q K^T into score buffer n % 3 (three 128-column buffers), issued
//                 three steps ahead of the P V that frees the buffer: O(tile) += P(n) V.
//   softmax       eight warps per tile, two threads per row: read 64 scores each, take the
//                 row maximum, form the probabilities in base 2 and write them back as FP16
//                 pairs over the first 32 columns they read, where they are the A operand
//                 (from tensor memory) of P V. A quarter of the exponentials run as a
//                 polynomial on the FMA pipe, the rest on the special-function unit.
// A tile's softmax therefore never waits for its own P V: the next scores are already
// there, and the two tiles' softmax phases overlap each other and the MMAs. O accumulates
// in tensor memory over the whole row of key tiles; the exponent the probabilities are
// taken against moves only when a tile's maximum exceeds it by more than 2^kLazyShift, and
// only then does the thread wait for the previous P V, read O back, rescale and rewrite it.
// The tensor pipe runs one thread's MMAs in issue order, which is what lets S(n + 3)
// overwrite the columns that P(n) occupies: it is issued after the P V that reads them.
// Every K and V tile passes through one ring in the order the MMAs use them: K(0), K(1),
// K(2), then V(n), K(n + 3) alternately. The query tiles are double-buffered by item.
// Tensor memory: score buffers at 0, 128, 256; O of tile 0 at 384, of tile 1 at 448.

constexpr int kFwdThreads = 576;  // TMA warp, MMA warp, 2 x 8 softmax warps
constexpr int kFwdSlots = 8;      // ring of K and V tiles
constexpr int kFwdSmem = 1024 + kTileBytes * (4 + kFwdSlots) + 256;

struct FwdBarriers {
    uint32_t base;
    __device__ uint32_t q_full(int b) const { return base + 8u * b; }
    __device__ uint32_t q_empty(int b) const { return base + 16 + 8u * b; }
    __device__ uint32_t s_full(int b) const { return base + 32 + 8u * b; }
    __device__ uint32_t p_ready(int b) const { return base + 56 + 8u * b; }
    __device__ uint32_t pv_done(int t) const { return base + 80 + 8u * t; }
    __device__ uint32_t slot_full(int s) const { return base + 96 + 8u * s; }
    __device__ uint32_t slot_empty(int s) const { return base + 96 + 8u * (kFwdSlots + s); }
};

// Where a role stands in the CTA's sequence of steps: item number `round` of this CTA,
// key tile j of the item, query tile t.
struct FwdCursor {
    int round, j, t;
    int qb;      // the item's query tile (it has qb + 1 key tiles); -1 past the last item
    int pair;    // which pair of heads
};

__global__ void __launch_bounds__(kFwdThreads, 1)
    fb_attention_forward(const __grid_constant__ AttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_tiles = base;                       // [item parity][tile]
    const uint32_t ring = base + 4 * kTileBytes;
    const FwdBarriers bar{ring + kFwdSlots * kTileBytes};
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float pair_max[2][2][2][kTile];  // [query tile][iteration parity][column half][row]

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x / 32), 0);
    const int lane = threadIdx.x % 32;
    const int bh_count = p.heads * p.seqs;
    const int head_pairs = (bh_count + 1) / 2;
    const int items = p.blocks * head_pairs;
    const int first_item = static_cast<int>(blockIdx.x);
    const int stride = static_cast<int>(gridDim.x);
    // Rounds of gridDim.x items, dealt alternately in ascending and descending CTA order.
    auto item_of = [&](int round) {
        const int slot = (round & 1) != 0 ? stride - 1 - first_item : first_item;
        return round * stride + slot;
    };
    // The cursor at the first step of this CTA's item number `round` (the divisions are
    // done here, once per item, not in the roles' inner loops).
    auto enter = [&](int round) {
        const int item = item_of(round);
        FwdCursor c{round, 0, 0, -1, 0};
        if (item < items) {
            c.qb = p.blocks - 1 - item / head_pairs;
            c.pair = item % head_pairs;
        }
        return c;
    };
    auto valid = [](const FwdCursor& c) { return c.qb >= 0; };
    // The (sequence, head) a tile of the item works on. With an odd number of heads in all,
    // the last item's second tile repeats the first one's head and stores nothing.
    auto head_of = [&](const FwdCursor& c, int t) { return min(2 * c.pair + t, bh_count - 1); };
    auto advance = [&](FwdCursor& c) {
        c.t ^= 1;
        if (c.t == 0 && ++c.j > c.qb) {
            c = enter(c.round + 1);
        }
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int b = 0; b < 2; ++b) {
            sm100::mbar_init(bar.q_full(b), 1);
            sm100::mbar_init(bar.q_empty(b), 1);
            sm100::mbar_init(bar.pv_done(b), 1);
        }
        for (int b = 0; b < 3; ++b) {
            sm100::mbar_init(bar.s_full(b), 1);
            sm100::mbar_init(bar.p_ready(b), 8);   // one arrival per softmax warp of the tile
        }
        for (int s = 0; s < kFwdSlots; ++s) {
            sm100::mbar_init(bar.slot_full(s), 1);
            sm100::mbar_init(bar.slot_empty(s), 1);
        }
        sm100::mbar_fence_init();
    }
    if (warp == 1) {
        sm100::tmem_alloc(sm100::smem_u32(&tmem_slot), 512);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t tmem_o = tmem + 384;   // + 64 t
    volatile int* abort = &abort_flag;
    fb::dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto load = [&](const CUtensorMap* map, const FwdCursor& c) {
                if (!sm100::mbar_wait(bar.slot_empty(slot), phase ^ 1u, abort)) {
                    ok = false;
                    return;
                }
                const int bh = head_of(c, c.t);
                sm100::mbar_expect_tx(bar.slot_full(slot), kTileBytes);
                tma_load_4d(ring + slot * kTileBytes, map, bar.slot_full(slot), 0, c.j * kTile,
                            bh % p.heads, bh / p.heads);
                if (++slot == kFwdSlots) {
                    slot = 0;
                    phase ^= 1u;
                }
            };
            FwdCursor keys = enter(0);     // the next K tile to fetch
            FwdCursor values = enter(0);   // the next V tile, three steps behind
            for (int ahead = 0; ok && valid(values); ++ahead) {
                if (ahead >= 3) {
                    load(&p.map_v, values);
                    advance(values);
                }
                if (ok && valid(keys)) {
                    if (keys.j == 0 && keys.t == 0) {
                        // A new item: its two query tiles go into the buffer of its parity,
                        // free once the item two rounds back has issued its last scores.
                        const int b = keys.round & 1;
                        if (keys.round >= 2 &&
                            !sm100::mbar_wait(bar.q_empty(b), ((keys.round >> 1) - 1) & 1, abort)) {
                            break;
                        }
                        sm100::mbar_expect_tx(bar.q_full(b), 2 * kTileBytes);
                        for (int t = 0; t < 2; ++t) {
                            const int bh = head_of(keys, t);
                            tma_load_4d(q_tiles + (2 * b + t) * kTileBytes, &p.map_q, bar.q_full(b), 0,
                                        keys.qb * kTile, bh % p.heads, bh / p.heads);
                        }
                    }
                    load(&p.map_k, keys);
                    advance(keys);
                }
            }
        }
    } else if (warp == 1) {
        // The whole warp runs this loop, so that its state stays warp-uniform (the MMA's
        // descriptors then need no per-thread to uniform register moves); one elected lane
        // issues.
        int slot = 0;
        uint32_t phase = 0;
        bool ok = true;
        // Waits for the ring's next tile and returns its address (0 after an abort).
        auto next_tile = [&]() -> uint32_t {
            if (!sm100::mbar_wait(bar.slot_full(slot), phase, abort)) {
                ok = false;
                return 0u;
            }
            sm100::tc_fence_after_sync();
            return ring + slot * kTileBytes;
        };
        // To be called by the elected lane after the MMAs that read the tile.
        auto release_tile = [&]() { sm100::mma_commit(bar.slot_empty(slot)); };
        auto step_ring = [&]() {
            if (++slot == kFwdSlots) {
                slot = 0;
                phase ^= 1u;
            }
        };
        FwdCursor ahead = enter(0);   // the next scores to issue
        uint32_t issued = 0;        // their step number
        auto issue_scores = [&]() {
            if (!ok || !valid(ahead)) {
                return;
            }
            const int b = ahead.round & 1;
            if (ahead.j == 0 && ahead.t == 0 &&
                !sm100::mbar_wait(bar.q_full(b), (ahead.round >> 1) & 1, abort)) {
                ok = false;
                return;
            }
            const uint32_t k_tile = next_tile();
            if (k_tile == 0) {
                return;
            }
            const uint64_t q_desc = desc_kmajor(q_tiles + (2 * b + ahead.t) * kTileBytes, 0);
            const uint64_t k_desc = desc_kmajor(k_tile, 0);
            const uint32_t s_at = tmem + 128u * (issued % 3);
            const bool last_of_item = ahead.t == 1 && ahead.j == ahead.qb;
            if (sm100::elect_one()) {
                sm100::mma_f16_ss_at<0>(s_at, q_desc, 0, k_desc, 0, kIdescS);
                sm100::mma_f16_ss_at<1>(s_at, q_desc, 2, k_desc, 2, kIdescS);
                sm100::mma_f16_ss_at<1>(s_at, q_desc, 4, k_desc, 4, kIdescS);
                sm100::mma_f16_ss_at<1>(s_at, q_desc, 6, k_desc, 6, kIdescS);
                sm100::mma_commit(bar.s_full(issued % 3));
                release_tile();
                if (last_of_item) {
                    sm100::mma_commit(bar.q_empty(b));
                }
            }
            __syncwarp();
            step_ring();
            ++issued;
            advance(ahead);
        };
        issue_scores();
        issue_scores();
        issue_scores();
        uint32_t n = 0;
        for (FwdCursor at = enter(0); ok && valid(at); advance(at), ++n) {
            if (!sm100::mbar_wait(bar.p_ready(n % 3), (n / 3) & 1, abort)) {
                break;
            }
            const uint32_t v_tile = next_tile();
            if (v_tile == 0) {
                break;
            }
            // O(tile) (+)= P V; keys 64 half + [0, 64) sit in columns 64 half + [0, 32) of
            // the score buffer. An MN-major step of 16 keys is 2,048 bytes.
            const uint64_t v_desc = desc_mnmajor(v_tile, 0, 16);
            const uint32_t p_at = tmem + 128u * (n % 3);
            const uint32_t o_at = tmem_o + 64u * at.t;
            if (sm100::elect_one()) {
                sm100::mma_f16_ts_at<-1>(o_at, p_at, v_desc, 0, kIdescPV, at.j > 0);
#pragma unroll
                for (int ks = 1; ks < 8; ++ks) {
                    sm100::mma_f16_ts_at<1>(o_at, p_at + (ks >> 2) * 64 + (ks & 3) * 8, v_desc,
                                            ks * 128, kIdescPV);
                }
                sm100::mma_commit(bar.pv_done(at.t));
                release_tile();
            }
            __syncwarp();
            step_ring();
            issue_scores();   // into the buffer this P V frees
        }
    } else {
        // Two threads per query row: this one owns score columns [64 half, 64 half + 64)
        // and output columns [32 half, 32 half + 32) of query tile `tile`.
        const int tile = (warp - 2) / 8;
        const int quadrant = warp % 4;
        const int half = ((warp - 2) % 8) / 4;
        const int row = quadrant * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        const uint32_t my_output = tmem_o + 64u * tile + lane_base + half * 32;
        const int pair_barrier = tile * 4 + quadrant;
        const float scale2 = p.scale * kLog2e;
        const fb::F2 scale_pair = fb::f2_pack(scale2, scale2);
        uint32_t before = 0;   // key tiles of this CTA's earlier items
        bool ok = true;
        for (FwdCursor item = enter(0); ok && valid(item); item = enter(item.round + 1)) {
            const int qb = item.qb;
            const int bh = head_of(item, tile);
            const bool stores = 2 * item.pair + tile < bh_count;
            const int q_index = qb * kTile + row;
            float m = -INFINITY;  // reference exponent of the row (base 2), shared by the pair
            fb::F2 l = 0;         // this thread's share of the row sum, in two partial sums
            for (int j = 0; ok && j <= qb; ++j) {
                const uint32_t n = 2 * (before + j) + tile;   // this step's number
                if (!sm100::mbar_wait(bar.s_full(n % 3), (n / 3) & 1, abort)) {
                    ok = false;
                    break;
                }
                const int parity = j & 1;
                const uint32_t my_scores = tmem + 128u * (n % 3) + lane_base + half * 64;
                sm100::tc_fence_after_sync();
                uint32_t raw[64];
                sm100::tmem_ld_32x32(my_scores, reinterpret_cast<uint32_t(&)[32]>(raw[0]));
                sm100::tmem_ld_32x32(my_scores + 32, reinterpret_cast<uint32_t(&)[32]>(raw[32]));
                sm100::tmem_ld_wait();
                if (j == qb) {
                    // The diagonal tile: keys after the query count as minus infinity.
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        raw[i] = (half * 64 + i <= row) ? raw[i] : 0xff800000u;
                    }
                }
                float top[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    top[t] = max3(__uint_as_float(raw[t]), __uint_as_float(raw[4 + t]),
                                  __uint_as_float(raw[8 + t]));
                }
#pragma unroll
                for (int i = 12; i < 60; i += 8) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        top[t] = max3(top[t], __uint_as_float(raw[i + t]),
                                      __uint_as_float(raw[i + 4 + t]));
                    }
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    top[t] = fmaxf(top[t], __uint_as_float(raw[60 + t]));
                }
                // The scale is positive, so the maximum may be scaled after it is taken.
                const float local = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) * scale2;
                pair_max[tile][parity][half][row] = local;
                quadrant_sync(pair_barrier);
                const float mx = fmaxf(m, fmaxf(local, pair_max[tile][parity][half ^ 1][row]));
                const bool moved = mx - m > kLazyShift;   // always on the first tile (m = -inf)
                float alpha = 1.0f;
                if (moved) {
                    alpha = fast_exp2(m - mx);
                    m = mx;
                    l = fb::f2_mul(l, fb::f2_pack(alpha, alpha));
                }
                if (j > 0 && __any_sync(0xffffffffu, moved)) {
                    // The previous key tile's P V must have finished (it cannot be more than
                    // one behind: the next one needs this step's probabilities).
                    if (!sm100::mbar_wait(bar.pv_done(tile), (before + j - 1) & 1, abort)) {
                        ok = false;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                    const fb::F2 a2 = fb::f2_pack(alpha, alpha);
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t acc[16];
                        sm100::tmem_ld_32x16(my_output + c * 16, acc);
                        sm100::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            float lo, hi;
                            fb::f2_unpack(fb::f2_mul(fb::f2_pack(__uint_as_float(acc[i]),
                                                                 __uint_as_float(acc[i + 1])), a2),
                                          lo, hi);
                            acc[i] = __float_as_uint(lo);
                            acc[i + 1] = __float_as_uint(hi);
                        }
                        sm100::tmem_st_32x16(my_output + c * 16, acc);
                    }
                }
                const fb::F2 shift = fb::f2_pack(-m, -m);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float lo, hi;
                        const fb::F2 x =
                            fb::f2_fma(fb::f2_pack(__uint_as_float(raw[32 * c + 2 * i]),
                                                   __uint_as_float(raw[32 * c + 2 * i + 1])),
                                       scale_pair, shift);
                        if ((i & 3) < FB_ATTN_FMA_EXP_OF_4) {
                            exp2_pair_fma(x, lo, hi);
                        } else {
                            fb::f2_unpack(x, lo, hi);
                            lo = fast_exp2(lo);
                            hi = fast_exp2(hi);
                        }
                        l = fb::f2_add(l, fb::f2_pack(lo, hi));
                        packed[i] = fb::pack2(lo, hi);
                    }
                    sm100::tmem_st_32x16(my_scores + c * 16, packed);
                }
                sm100::tmem_st_wait();
                sm100::tc_fence_before_sync();
                // A parity wait is only right while the barrier is neither behind nor ahead by
                // more than the phase waited for. After the item's last step the thread waits
                // for that step's P V; the MMA warp may still be one P V short of it, so the
                // last but one is awaited first, and here, before this warp's arrival lets the
                // last one be issued at all (afterwards a slow warp could find both complete
                // and wait for a parity that no longer comes).
                if (j == qb && qb > 0 &&
                    !sm100::mbar_wait(bar.pv_done(tile), (before + qb - 1) & 1, abort)) {
                    ok = false;
                    break;
                }
                __syncwarp();
                if (lane == 0) {
                    sm100::mbar_arrive(bar.p_ready(n % 3));
                }
            }
            if (!ok || !sm100::mbar_wait(bar.pv_done(tile), (before + qb) & 1, abort)) {
                ok = false;
                break;
            }
            before += qb + 1;
            sm100::tc_fence_after_sync();
            uint32_t acc[32];
            sm100::tmem_ld_32x32(my_output, acc);
            sm100::tmem_ld_wait();
            // The accumulator is overwritten by the next item's first P V, which needs the
            // probabilities this thread writes after it has got here.
            sm100::tc_fence_before_sync();
            // The row sum is the two threads' shares added together.
            float l_lo, l_hi;
            fb::f2_unpack(l, l_lo, l_hi);
            const float mine = l_lo + l_hi;
            const int parity = (qb + 1) & 1;   // not the slot the last key tile used
            pair_max[tile][parity][half][row] = mine;
            quadrant_sync(pair_barrier);
            const float total = mine + pair_max[tile][parity][half ^ 1][row];
            quadrant_sync(pair_barrier);     // both have read before either writes a maximum there
            if (stores && q_index < p.length) {
                const float inv = 1.0f / total;
                const int head = bh % p.heads;
                const int seq = bh / p.heads;
                __half* out = static_cast<__half*>(p.out0) + seq * p.out_seq + head * p.out_head +
                              static_cast<long long>(q_index) * p.out_row + half * 32;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[i] = __uint_as_float(acc[c * 8 + i]) * inv;
                    }
                    *reinterpret_cast<uint4*>(out + c * 8) = fb::pack8(v);
                }
                if (half == 0) {
                    p.lse[static_cast<size_t>(bh) * p.length + q_index] = (m + log2f(total)) * kLn2;
                }
            }
        }
    }
    // A persistent CTA lets the next kernel in only when its own work is done.
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }
    finish(abort_flag, tmem, 512, warp);
}

// ---- backward: delta = rowsum(dO * O) ----------------------------------------------------------

struct View {
    const __half* base;
    long long row, head, seq;
};

// Eight lanes per row (16 bytes of dO and of O each), four rows per warp and step.
__global__ void __launch_bounds__(256)
    fb_attention_delta(float* __restrict__ delta, View d_o, View o, int length, int heads,
                       int seqs) {
    fb::dependency_wait();
    fb::dependency_release();
    const long long rows = static_cast<long long>(length) * heads * seqs;
    const int lane = threadIdx.x % 32;
    const int piece = lane % 8;  // which 8 of the row's 64 values
    const long long first = (blockIdx.x * 8LL + threadIdx.x / 32) * 4 + lane / 8;
    const long long stride = gridDim.x * 8LL * 4;
    for (long long r0 = first; r0 - lane / 8 < rows; r0 += stride) {
        const bool valid = r0 < rows;
        const long long r = valid ? r0 : rows - 1;
        const int t = static_cast<int>(r % length);
        const long long bh = r / length;
        const int head = static_cast<int>(bh % heads);
        const long long seq = bh / heads;
        const uint4 a = *reinterpret_cast<const uint4*>(d_o.base + seq * d_o.seq + head * d_o.head +
                                                        t * d_o.row + 8 * piece);
        const uint4 b = *reinterpret_cast<const uint4*>(o.base + seq * o.seq + head * o.head +
                                                        t * o.row + 8 * piece);
        float fa[8];
        float fo[8];
        fb::unpack8(fa, a);
        fb::unpack8(fo, b);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s = fmaf(fa[i], fo[i], s);
        }
        s += __shfl_xor_sync(fb::kFullMask, s, 4);
        s += __shfl_xor_sync(fb::kFullMask, s, 2);
        s += __shfl_xor_sync(fb::kFullMask, s, 1);
        if (valid && piece == 0) {
            delta[r] = s;
        }
    }
}

// ---- backward: shared pieces --------------------------------------------------------------------
//
// Both gradient kernels keep every A operand in tensor memory (TS-form MMAs): the
// resident tile pair is copied there once per CTA, and the probabilities / score
// gradients the compute warps produce are written back as FP16 pairs over the
// accumulator columns they were read from. Shared memory then only feeds the B
// operands (the streamed 64-row tiles): an SS-form MMA with N = 64 needs 6 KB of
// operands per instruction and is bound by the shared-memory rate (measured 49
// clocks against 32 of tensor work), and the P/dS stores shared the same banks.

constexpr int kBwdThreads = 576;  // TMA warp, MMA warp, 16 compute warps
constexpr int kPart = 16;         // accumulator columns per compute thread and sub-step
constexpr int kBwdComputeWarps = 16;
constexpr int kSub = 64;          // streamed rows (queries for dK/dV, keys for dQ) per sub-step
constexpr int kSubBytes = kSub * kHead * 2;  // 8 KB: one streamed tile
constexpr int kBwdStages = 4;
constexpr int kStatBytes = kSub * 4;  // one sub-step's log-sum-exp or delta values
// resident pair (2 x 16 KB) + ring of tile pairs (4 x 16 KB) + row statistics + barriers
constexpr int kBwdUsed = 1024 + 2 * kTileBytes + kBwdStages * 2 * kSubBytes +
                         kBwdStages * 2 * kStatBytes + 256;
// The kernels are persistent, one CTA per SM, and each CTA wants all of tensor memory:
// asking for more than half an SM's shared memory keeps two from landing on one SM
// (which happens when CTAs become resident one SM at a time, behind an earlier kernel,
// and leaves other SMs idle while the pair takes turns).
constexpr int kBwdSmem = kBwdUsed > 120 * 1024 ? kBwdUsed : 120 * 1024;
constexpr uint32_t kIdescSub = sm100::instr_desc_f16(128, 64, false, false);  // A Bsub^T

struct BwdBarriers {
    uint32_t base;
    __device__ uint32_t resident() const { return base; }
    __device__ uint32_t done() const { return base + 8; }
    __device__ uint32_t a_ready() const { return base + 16; }
    __device__ uint32_t scores_full(int b) const { return base + 32 + 8u * b; }
    __device__ uint32_t operands_ready(int b) const { return base + 48 + 8u * b; }
    __device__ uint32_t stage_full(int s) const { return base + 64 + 8u * s; }
    __device__ uint32_t stage_empty(int s) const { return base + 96 + 8u * s; }
};

// The compute warps arrive once per warp (after __syncwarp, by lane 0).
__device__ __forceinline__ void init_bwd_barriers(const BwdBarriers& b) {
    sm100::mbar_init(b.resident(), 1);
    sm100::mbar_init(b.done(), 1);
    sm100::mbar_init(b.a_ready(), kBwdComputeWarps);
    for (int i = 0; i < 2; ++i) {
        sm100::mbar_init(b.scores_full(i), 1);
        sm100::mbar_init(b.operands_ready(i), kBwdComputeWarps);
    }
    for (int s = 0; s < kBwdStages; ++s) {
        sm100::mbar_init(b.stage_full(s), 1);
        sm100::mbar_init(b.stage_empty(s), 1);
    }
    sm100::mbar_fence_init();
}

// Copies this thread's share of a row of a resident 128 x 64 FP16 tile (swizzled as TMA
// wrote it) into tensor memory as an A operand: the 16 head columns [16 part, 16 part + 16)
// become 8 columns of FP16 pairs at `dst` + 8 part.
__device__ __forceinline__ void tile_row_to_tmem(uint32_t dst, uint32_t tile, int row, int part) {
    uint32_t r[8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int chunk = part * 2 + i;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[4 * i]), "=r"(r[4 * i + 1]), "=r"(r[4 * i + 2]), "=r"(r[4 * i + 3])
                     : "r"(tile + row * 128 + ((chunk ^ (row & 7)) << 4)));
    }
    sm100::tmem_st_32x8(dst + 8 * part, r);
}

// 16 FP32 values -> 8 words of FP16 pairs (the lower-indexed value in the low half).
__device__ __forceinline__ void pack_pairs(uint32_t (&w)[8], const float (&v)[kPart]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        w[i] = fb::pack2(v[2 * i], v[2 * i + 1]);
    }
}

// One arrival for the warp, after every lane's tensor-memory stores have completed.
__device__ __forceinline__ void warp_arrive_after_stores(uint32_t bar, int lane) {
    sm100::tmem_st_wait();
    sm100::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
        sm100::mbar_arrive(bar);
    }
}

// The 64-bit descriptor of a 128-byte-swizzled tile moved by `bytes` (a multiple of
// 16; shared memory is small enough that the address field never carries).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
    return desc + (bytes >> 4);
}

// ---- backward: dK and dV ------------------------------------------------------------------------
//
// Persistent CTAs, one per SM, each taking (head, 128 keys) items round-robin from a
// list ordered by work (key tile 0 first); an item is 64 queries per sub-step from the
// diagonal on. Scores are formed transposed, S^T = K Q^T and dP^T = V dO^T with keys on
// the TMEM lanes (A = K, V from tensor memory), so P^T and dS^T are already the A
// operands of dV += P^T dO and dK += dS^T Q. Accumulator pairs are double-buffered: the
// MMA warp issues sub-step h+1's score MMAs before it waits for sub-step h's
// probabilities. Items overlap too: the producer fetches the next item's K/V as soon as
// this item's were copied to tensor memory, the compute warps install them right after
// their last sub-step, and the MMA warp issues the next item's first score MMAs while the
// compute warps write this item's dK/dV out. Barrier phases and the tile ring simply
// continue from item to item (an item has an even number of sub-steps).
// Tensor memory: S^T at 0/64, dP^T at 128/192 (P^T and dS^T overwrite 4 x 8 columns of
// each), dV 256, dK 320, K 384, V 416.

__global__ void __launch_bounds__(kBwdThreads, 1)
    fb_attention_dkv(const __grid_constant__ AttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t k_tile = base;
    const uint32_t v_tile = base + kTileBytes;
    const uint32_t ring = base + 2 * kTileBytes;                   // stage: Q_h then dO_h
    const uint32_t stats = ring + kBwdStages * 2 * kSubBytes;      // stage: lse[64] then delta[64]
    const BwdBarriers bar{stats + kBwdStages * 2 * kStatBytes};
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x / 32), 0);
    const int lane = threadIdx.x % 32;
    const int bh_count = p.heads * p.seqs;
    const int items = bh_count * p.blocks;
    const int first_item = static_cast<int>(blockIdx.x);
    const int stride = static_cast<int>(gridDim.x);
    // Items are dealt in rounds of gridDim.x, alternately in ascending and descending CTA
    // order (the list is sorted by work, so this evens the CTAs' totals out); a result
    // >= items ends the list, and only the last round can be short.
    auto item_of = [&](int round) {
        const int slot = (round & 1) != 0 ? stride - 1 - first_item : first_item;
        return round * stride + slot;
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        init_bwd_barriers(bar);
    }
    if (warp == 1) {
        sm100::tmem_alloc(sm100::smem_u32(&tmem_slot), 512);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    auto tmem_st = [&](int b) { return tmem + 64u * b; };
    auto tmem_dpt = [&](int b) { return tmem + 128u + 64u * b; };
    const uint32_t tmem_dv = tmem + 256, tmem_dk = tmem + 320;
    const uint32_t tmem_k = tmem + 384, tmem_v = tmem + 416;
    volatile int* abort = &abort_flag;
    fb::dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int round = 0;
            for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
                const int kb = item / bh_count;
                const int bh = item % bh_count;
                const int head = bh % p.heads;
                const int seq = bh / p.heads;
                const int steps = 2 * (p.blocks - kb);
                // The K/V buffers are free once the item before was copied to tensor memory.
                if (round > 0 && !sm100::mbar_wait(bar.a_ready(), (round - 1) & 1, abort)) {
                    break;
                }
                sm100::mbar_expect_tx(bar.resident(), 2 * kTileBytes);
                tma_load_4d(k_tile, &p.map_k, bar.resident(), 0, kb * kTile, head, seq);
                tma_load_4d(v_tile, &p.map_v, bar.resident(), 0, kb * kTile, head, seq);
                for (int h = 0; h < steps; ++h) {
                    if (!sm100::mbar_wait(bar.stage_empty(stage), phase ^ 1u, abort)) {
                        ok = false;
                        break;
                    }
                    const int q0 = kb * kTile + h * kSub;
                    const uint32_t dst = ring + stage * 2 * kSubBytes;
                    // Row statistics of the queries that exist (length is a multiple of 8,
                    // so the byte count is a multiple of 32); the rest of the slot is never
                    // used.
                    const int present = min(kSub, p.length - q0);
                    const uint32_t stat_bytes =
                        present > 0 ? static_cast<uint32_t>(present) * 4u : 0u;
                    sm100::mbar_expect_tx(bar.stage_full(stage), 2 * kSubBytes + 2 * stat_bytes);
                    tma_load_4d(dst, &p.map_q64, bar.stage_full(stage), 0, q0, head, seq);
                    tma_load_4d(dst + kSubBytes, &p.map_do64, bar.stage_full(stage), 0, q0, head,
                                seq);
                    if (stat_bytes != 0) {
                        const size_t at = static_cast<size_t>(bh) * p.length + q0;
                        const uint32_t slot = stats + stage * 2 * kStatBytes;
                        bulk_load(slot, p.lse + at, stat_bytes, bar.stage_full(stage));
                        bulk_load(slot + kStatBytes, p.delta + at, stat_bytes,
                                  bar.stage_full(stage));
                    }
                    if (++stage == kBwdStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // The whole warp runs this loop so that its state stays warp-uniform; one elected
        // lane issues the MMAs and commits.
        {
            // Descriptors of stage 0's tiles; a stage is 16 KB further, a K-major k-step 32
            // bytes, an MN-major one 2,048.
            const uint64_t q_desc = sm100::smem_desc_sw128(ring, 16, 1024);
            const uint64_t do_desc = sm100::smem_desc_sw128(ring + kSubBytes, 16, 1024);
            uint32_t before = 0;  // sub-steps of earlier items (always even)
            bool ok = true;
            int round = 0;
            for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
                const int steps = 2 * (p.blocks - item / bh_count);
                ok = sm100::mbar_wait(bar.a_ready(), round & 1, abort);
                sm100::tc_fence_after_sync();
                // S^T and dP^T of sub-step g into accumulator pair g & 1.
                auto issue_scores = [&](int g) -> bool {
                    const uint32_t count = before + g;
                    const int stage = count % kBwdStages;
                    if (!sm100::mbar_wait(bar.stage_full(stage), (count / kBwdStages) & 1, abort)) {
                        return false;
                    }
                    sm100::tc_fence_after_sync();
                    const uint64_t q_sub = desc_advance(q_desc, stage * 2 * kSubBytes);
                    const uint64_t do_sub = desc_advance(do_desc, stage * 2 * kSubBytes);
                    if (sm100::elect_one()) {
                        const uint32_t st_at = tmem_st(g & 1), dpt_at = tmem_dpt(g & 1);
                        sm100::mma_f16_ts_at<0>(st_at, tmem_k, q_sub, 0, kIdescSub);
                        sm100::mma_f16_ts_at<1>(st_at, tmem_k + 8, q_sub, 2, kIdescSub);
                        sm100::mma_f16_ts_at<1>(st_at, tmem_k + 16, q_sub, 4, kIdescSub);
                        sm100::mma_f16_ts_at<1>(st_at, tmem_k + 24, q_sub, 6, kIdescSub);
                        sm100::mma_f16_ts_at<0>(dpt_at, tmem_v, do_sub, 0, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dpt_at, tmem_v + 8, do_sub, 2, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dpt_at, tmem_v + 16, do_sub, 4, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dpt_at, tmem_v + 24, do_sub, 6, kIdescSub);
                        sm100::mma_commit(bar.scores_full(g & 1));
                    }
                    __syncwarp();
                    return true;
                };
                ok = ok && issue_scores(0);
                for (int h = 0; ok && h < steps; ++h) {
                    const int b = h & 1;
                    const uint32_t count = before + h;
                    if (h + 1 < steps && !issue_scores(h + 1)) {
                        ok = false;
                        break;
                    }
                    if (!sm100::mbar_wait(bar.operands_ready(b), (count >> 1) & 1, abort)) {
                        ok = false;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                    const int stage = count % kBwdStages;
                    const uint64_t q_sub = desc_advance(q_desc, stage * 2 * kSubBytes);
                    const uint64_t do_sub = desc_advance(do_desc, stage * 2 * kSubBytes);
                    // dV += P^T dO and dK += dS^T Q over this sub-step's 64 queries; queries
                    // 16 part + [0, 16) sit in columns 16 part + [0, 8) of the accumulator.
                    if (sm100::elect_one()) {
                        const uint32_t st_at = tmem_st(b), dpt_at = tmem_dpt(b);
                        sm100::mma_f16_ts_at<-1>(tmem_dv, st_at, do_sub, 0, kIdescPV, h != 0);
                        sm100::mma_f16_ts_at<1>(tmem_dv, st_at + 16, do_sub, 128, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dv, st_at + 32, do_sub, 256, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dv, st_at + 48, do_sub, 384, kIdescPV);
                        sm100::mma_f16_ts_at<-1>(tmem_dk, dpt_at, q_sub, 0, kIdescPV, h != 0);
                        sm100::mma_f16_ts_at<1>(tmem_dk, dpt_at + 16, q_sub, 128, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dk, dpt_at + 32, q_sub, 256, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dk, dpt_at + 48, q_sub, 384, kIdescPV);
                        sm100::mma_commit(bar.stage_empty(stage));
                        if (h + 1 == steps) {
                            sm100::mma_commit(bar.done());
                        }
                    }
                    __syncwarp();
                }
                before += steps;
            }
        }
    } else {
        const int quadrant = warp % 4;
        const int part = (warp - 2) / 4;                 // which 16 of the 64 query columns
        const int row = quadrant * 32 + lane;            // key row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        const float scale2 = p.scale * kLog2e;
        // K and V of an item become the A operands of its score MMAs. Called when every
        // score MMA of the item before has completed (its last scores_full was awaited).
        auto install = [&](int round) -> bool {
            if (!sm100::mbar_wait(bar.resident(), round & 1, abort)) {
                return false;
            }
            tile_row_to_tmem(tmem_k + lane_base, k_tile, row, part);
            tile_row_to_tmem(tmem_v + lane_base, v_tile, row, part);
            warp_arrive_after_stores(bar.a_ready(), lane);
            return true;
        };
        uint32_t before = 0;
        int round = 0;
        bool ok = first_item < items && install(0);
        for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
            const int kb = item / bh_count;
            const int bh = item % bh_count;
            const int head = bh % p.heads;
            const int seq = bh / p.heads;
            const int steps = 2 * (p.blocks - kb);
            const int k_index = kb * kTile + row;
            for (int h = 0; ok && h < steps; ++h) {
                const int b = h & 1;
                const uint32_t count = before + h;
                const int stage = count % kBwdStages;
                const int q0 = kb * kTile + h * kSub + part * kPart;  // first query of my columns
                // stage_full covers the statistics; scores_full the two accumulators (and,
                // the tensor pipe being in order, that the MMAs which read this pair's
                // previous P^T and dS^T have finished).
                if (!sm100::mbar_wait(bar.scores_full(b), (count >> 1) & 1, abort)) {
                    ok = false;
                    break;
                }
                sm100::tc_fence_after_sync();
                const uint32_t my_scores = tmem_st(b) + lane_base + part * kPart;
                const uint32_t my_weights = tmem_dpt(b) + lane_base + part * kPart;
                uint32_t s_raw[kPart];
                uint32_t dp_raw[kPart];
                sm100::tmem_ld_32x16(my_scores, s_raw);
                sm100::tmem_ld_32x16(my_weights, dp_raw);
                if (!sm100::mbar_wait(bar.stage_full(stage), (count / kBwdStages) & 1, abort)) {
                    ok = false;
                    break;
                }
                // My 16 queries' statistics: every lane reads the same addresses (broadcast).
                const uint32_t stat = stats + stage * 2 * kStatBytes + part * kPart * 4;
                float lse2[kPart];
                float dlt[kPart];
#pragma unroll
                for (int c = 0; c < kPart / 4; ++c) {
                    float a0, a1, a2, a3;
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(a0), "=f"(a1), "=f"(a2), "=f"(a3)
                                 : "r"(stat + c * 16));
                    lse2[4 * c] = a0 * kLog2e;
                    lse2[4 * c + 1] = a1 * kLog2e;
                    lse2[4 * c + 2] = a2 * kLog2e;
                    lse2[4 * c + 3] = a3 * kLog2e;
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(dlt[4 * c]), "=f"(dlt[4 * c + 1]), "=f"(dlt[4 * c + 2]),
                                   "=f"(dlt[4 * c + 3])
                                 : "r"(stat + kStatBytes + c * 16));
                }
                sm100::tmem_ld_wait();
                float pv[kPart];
                float dsv[kPart];
                if (h < 2 || kb * kTile + (h + 1) * kSub > p.length) {
                    // The diagonal tile (a key is visible to the queries at or after it) or
                    // a sub-step with absent queries, whose statistics slots were not
                    // filled: both tests select rather than multiply.
                    const int first_visible = h < 2 ? k_index : 0;
#pragma unroll
                    for (int i = 0; i < kPart; ++i) {
                        const bool visible = first_visible <= q0 + i && q0 + i < p.length;
                        const float e =
                            fast_exp2(fmaf(__uint_as_float(s_raw[i]), scale2, -lse2[i]));
                        pv[i] = visible ? e : 0.0f;
                        dsv[i] = visible ? e * (__uint_as_float(dp_raw[i]) - dlt[i]) : 0.0f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kPart; i += 2) {
                        exp2_two(i / 2, fmaf(__uint_as_float(s_raw[i]), scale2, -lse2[i]),
                                 fmaf(__uint_as_float(s_raw[i + 1]), scale2, -lse2[i + 1]), pv[i],
                                 pv[i + 1]);
                        dsv[i] = pv[i] * (__uint_as_float(dp_raw[i]) - dlt[i]);
                        dsv[i + 1] = pv[i + 1] * (__uint_as_float(dp_raw[i + 1]) - dlt[i + 1]);
                    }
                }
                // P^T and dS^T go back over the first 8 of the 16 columns this thread read.
                uint32_t packed[8];
                pack_pairs(packed, pv);
                sm100::tmem_st_32x8(my_scores, packed);
                pack_pairs(packed, dsv);
                sm100::tmem_st_32x8(my_weights, packed);
                warp_arrive_after_stores(bar.operands_ready(b), lane);
            }
            before += steps;
            if (!ok) {
                break;
            }
            // The next item's K/V go in now, so that its first score MMAs run while this
            // item's gradients are written out.
            if (item_of(round + 1) < items && !install(round + 1)) {
                ok = false;
                break;
            }
            if (!sm100::mbar_wait(bar.done(), round & 1, abort)) {
                ok = false;
                break;
            }
            sm100::tc_fence_after_sync();
            // Rows of dV/dK are keys; this thread writes 16 of the 64 columns. dS was kept
            // unscaled, so the score scale is applied to dK here.
            uint32_t dv_raw[kPart];
            uint32_t dk_raw[kPart];
            sm100::tmem_ld_32x16(tmem_dv + lane_base + part * kPart, dv_raw);
            sm100::tmem_ld_32x16(tmem_dk + lane_base + part * kPart, dk_raw);
            sm100::tmem_ld_wait();
            if (k_index < p.length) {
                const long long at = seq * p.out_seq + head * p.out_head +
                                     static_cast<long long>(k_index) * p.out_row + part * kPart;
                __half* dk_out = static_cast<__half*>(p.out0) + at;
                __half* dv_out = static_cast<__half*>(p.out1) + at;
#pragma unroll
                for (int c = 0; c < kPart / 8; ++c) {
                    float a[8];
                    float bv[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        a[i] = __uint_as_float(dk_raw[c * 8 + i]) * p.scale;
                        bv[i] = __uint_as_float(dv_raw[c * 8 + i]);
                    }
                    *reinterpret_cast<uint4*>(dk_out + c * 8) = fb::pack8(a);
                    *reinterpret_cast<uint4*>(dv_out + c * 8) = fb::pack8(bv);
                }
            }
            sm100::tc_fence_before_sync();
        }
    }
    // A persistent CTA lets the next kernel in only when its own work is done: a
    // dependent that became resident earlier was measured to slow this kernel down.
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }
    finish(abort_flag, tmem, 512, warp);
}

// ---- backward: dQ ---------------------------------------------------------------------------------
//
// Persistent CTAs over (head, 128 queries) items, the last query tile (most keys)
// first; 64 keys per sub-step: S = Q K^T and dP = dO V^T (A = Q, dO from tensor
// memory) into double-buffered accumulators, dS written back over dP as FP16 pairs,
// dQ += dS K accumulated in TMEM. Items overlap as in the dK/dV kernel.
// Tensor memory: S at 0/64, dP at 128/192, dQ 256, Q 320, dO 352.

__global__ void __launch_bounds__(kBwdThreads, 1)
    fb_attention_dq(const __grid_constant__ AttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_tile = base;
    const uint32_t do_tile = base + kTileBytes;
    const uint32_t ring = base + 2 * kTileBytes;                   // stage: K_g then V_g
    const uint32_t stats = ring + kBwdStages * 2 * kSubBytes;      // unused here
    const BwdBarriers bar{stats + kBwdStages * 2 * kStatBytes};
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x / 32), 0);
    const int lane = threadIdx.x % 32;
    const int bh_count = p.heads * p.seqs;
    const int items = bh_count * p.blocks;
    const int first_item = static_cast<int>(blockIdx.x);
    const int stride = static_cast<int>(gridDim.x);
    // Items are dealt in rounds of gridDim.x, alternately in ascending and descending CTA
    // order (the list is sorted by work, so this evens the CTAs' totals out); a result
    // >= items ends the list, and only the last round can be short.
    auto item_of = [&](int round) {
        const int slot = (round & 1) != 0 ? stride - 1 - first_item : first_item;
        return round * stride + slot;
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        init_bwd_barriers(bar);
    }
    if (warp == 1) {
        sm100::tmem_alloc(sm100::smem_u32(&tmem_slot), 512);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    auto tmem_s = [&](int b) { return tmem + 64u * b; };
    auto tmem_dp = [&](int b) { return tmem + 128u + 64u * b; };
    const uint32_t tmem_dq = tmem + 256;
    const uint32_t tmem_q = tmem + 320, tmem_do = tmem + 352;
    volatile int* abort = &abort_flag;
    fb::dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int round = 0;
            for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
                const int qb = p.blocks - 1 - item / bh_count;
                const int bh = item % bh_count;
                const int head = bh % p.heads;
                const int seq = bh / p.heads;
                const int steps = 2 * (qb + 1);
                // The Q/dO buffers are free once the item before was copied to tensor memory.
                if (round > 0 && !sm100::mbar_wait(bar.a_ready(), (round - 1) & 1, abort)) {
                    break;
                }
                sm100::mbar_expect_tx(bar.resident(), 2 * kTileBytes);
                tma_load_4d(q_tile, &p.map_q, bar.resident(), 0, qb * kTile, head, seq);
                tma_load_4d(do_tile, &p.map_do, bar.resident(), 0, qb * kTile, head, seq);
                for (int g = 0; g < steps; ++g) {
                    if (!sm100::mbar_wait(bar.stage_empty(stage), phase ^ 1u, abort)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst = ring + stage * 2 * kSubBytes;
                    sm100::mbar_expect_tx(bar.stage_full(stage), 2 * kSubBytes);
                    tma_load_4d(dst, &p.map_k64, bar.stage_full(stage), 0, g * kSub, head, seq);
                    tma_load_4d(dst + kSubBytes, &p.map_v64, bar.stage_full(stage), 0, g * kSub,
                                head, seq);
                    if (++stage == kBwdStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // The whole warp runs this loop; one elected lane issues the MMAs and commits.
        {
            const uint64_t k_desc = sm100::smem_desc_sw128(ring, 16, 1024);
            const uint64_t v_desc = sm100::smem_desc_sw128(ring + kSubBytes, 16, 1024);
            uint32_t before = 0;  // sub-steps of earlier items (always even)
            bool ok = true;
            int round = 0;
            for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
                const int steps = 2 * (p.blocks - item / bh_count);
                ok = sm100::mbar_wait(bar.a_ready(), round & 1, abort);
                sm100::tc_fence_after_sync();
                auto issue_scores = [&](int g) -> bool {
                    const uint32_t count = before + g;
                    const int stage = count % kBwdStages;
                    if (!sm100::mbar_wait(bar.stage_full(stage), (count / kBwdStages) & 1, abort)) {
                        return false;
                    }
                    sm100::tc_fence_after_sync();
                    const uint64_t k_sub = desc_advance(k_desc, stage * 2 * kSubBytes);
                    const uint64_t v_sub = desc_advance(v_desc, stage * 2 * kSubBytes);
                    if (sm100::elect_one()) {
                        const uint32_t s_at = tmem_s(g & 1), dp_at = tmem_dp(g & 1);
                        sm100::mma_f16_ts_at<0>(s_at, tmem_q, k_sub, 0, kIdescSub);
                        sm100::mma_f16_ts_at<1>(s_at, tmem_q + 8, k_sub, 2, kIdescSub);
                        sm100::mma_f16_ts_at<1>(s_at, tmem_q + 16, k_sub, 4, kIdescSub);
                        sm100::mma_f16_ts_at<1>(s_at, tmem_q + 24, k_sub, 6, kIdescSub);
                        sm100::mma_f16_ts_at<0>(dp_at, tmem_do, v_sub, 0, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dp_at, tmem_do + 8, v_sub, 2, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dp_at, tmem_do + 16, v_sub, 4, kIdescSub);
                        sm100::mma_f16_ts_at<1>(dp_at, tmem_do + 24, v_sub, 6, kIdescSub);
                        sm100::mma_commit(bar.scores_full(g & 1));
                    }
                    __syncwarp();
                    return true;
                };
                ok = ok && issue_scores(0);
                for (int g = 0; ok && g < steps; ++g) {
                    const int b = g & 1;
                    const uint32_t count = before + g;
                    if (g + 1 < steps && !issue_scores(g + 1)) {
                        ok = false;
                        break;
                    }
                    if (!sm100::mbar_wait(bar.operands_ready(b), (count >> 1) & 1, abort)) {
                        ok = false;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                    const int stage = count % kBwdStages;
                    const uint64_t k_sub = desc_advance(k_desc, stage * 2 * kSubBytes);
                    // dQ += dS K over this sub-step's 64 keys (the K tile read MN-major).
                    if (sm100::elect_one()) {
                        const uint32_t dp_at = tmem_dp(b);
                        sm100::mma_f16_ts_at<-1>(tmem_dq, dp_at, k_sub, 0, kIdescPV, g != 0);
                        sm100::mma_f16_ts_at<1>(tmem_dq, dp_at + 16, k_sub, 128, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dq, dp_at + 32, k_sub, 256, kIdescPV);
                        sm100::mma_f16_ts_at<1>(tmem_dq, dp_at + 48, k_sub, 384, kIdescPV);
                        sm100::mma_commit(bar.stage_empty(stage));
                        if (g + 1 == steps) {
                            sm100::mma_commit(bar.done());
                        }
                    }
                    __syncwarp();
                }
                before += steps;
            }
        }
    } else {
        const int quadrant = warp % 4;
        const int part = (warp - 2) / 4;                 // which 16 of the 64 key columns
        const int row = quadrant * 32 + lane;            // query row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        const float scale2 = p.scale * kLog2e;
        // Q and dO of an item become the A operands of its score MMAs.
        auto install = [&](int round) -> bool {
            if (!sm100::mbar_wait(bar.resident(), round & 1, abort)) {
                return false;
            }
            tile_row_to_tmem(tmem_q + lane_base, q_tile, row, part);
            tile_row_to_tmem(tmem_do + lane_base, do_tile, row, part);
            warp_arrive_after_stores(bar.a_ready(), lane);
            return true;
        };
        uint32_t before = 0;
        int round = 0;
        bool ok = first_item < items && install(0);
        for (int item = item_of(0); ok && item < items; item = item_of(++round)) {
            const int qb = p.blocks - 1 - item / bh_count;
            const int bh = item % bh_count;
            const int head = bh % p.heads;
            const int seq = bh / p.heads;
            const int steps = 2 * (qb + 1);  // 64-key sub-steps up to and including the diagonal
            const int q_index = qb * kTile + row;
            const bool row_valid = q_index < p.length;
            float lse2 = INFINITY;
            float dlt = 0.0f;
            if (row_valid) {
                lse2 = p.lse[static_cast<size_t>(bh) * p.length + q_index] * kLog2e;
                dlt = p.delta[static_cast<size_t>(bh) * p.length + q_index];
            }
            for (int g = 0; ok && g < steps; ++g) {
                const int b = g & 1;
                const uint32_t count = before + g;
                if (!sm100::mbar_wait(bar.scores_full(b), (count >> 1) & 1, abort)) {
                    ok = false;
                    break;
                }
                sm100::tc_fence_after_sync();
                const uint32_t my_weights = tmem_dp(b) + lane_base + part * kPart;
                uint32_t s_raw[kPart];
                uint32_t dp_raw[kPart];
                sm100::tmem_ld_32x16(tmem_s(b) + lane_base + part * kPart, s_raw);
                sm100::tmem_ld_32x16(my_weights, dp_raw);
                sm100::tmem_ld_wait();
                const int k0 = g * kSub + part * kPart;  // first key of my columns
                float dsv[kPart];
                if (g + 2 >= steps) {
                    // The diagonal tile: keys after the query are masked.
#pragma unroll
                    for (int i = 0; i < kPart; ++i) {
                        const float e = fast_exp2(fmaf(__uint_as_float(s_raw[i]), scale2, -lse2));
                        dsv[i] =
                            (k0 + i <= q_index) ? e * (__uint_as_float(dp_raw[i]) - dlt) : 0.0f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kPart; i += 2) {
                        float e0, e1;
                        exp2_two(i / 2, fmaf(__uint_as_float(s_raw[i]), scale2, -lse2),
                                 fmaf(__uint_as_float(s_raw[i + 1]), scale2, -lse2), e0, e1);
                        dsv[i] = e0 * (__uint_as_float(dp_raw[i]) - dlt);
                        dsv[i + 1] = e1 * (__uint_as_float(dp_raw[i + 1]) - dlt);
                    }
                }
                // dS goes back over the first 8 of the 16 dP columns this thread just read.
                uint32_t packed[8];
                pack_pairs(packed, dsv);
                sm100::tmem_st_32x8(my_weights, packed);
                warp_arrive_after_stores(bar.operands_ready(b), lane);
            }
            before += steps;
            if (!ok) {
                break;
            }
            if (item_of(round + 1) < items && !install(round + 1)) {
                ok = false;
                break;
            }
            if (!sm100::mbar_wait(bar.done(), round & 1, abort)) {
                ok = false;
                break;
            }
            sm100::tc_fence_after_sync();
            uint32_t raw[kPart];
            sm100::tmem_ld_32x16(tmem_dq + lane_base + part * kPart, raw);
            sm100::tmem_ld_wait();
            if (row_valid) {
                __half* out = static_cast<__half*>(p.out0) + seq * p.out_seq + head * p.out_head +
                              static_cast<long long>(q_index) * p.out_row + part * kPart;
#pragma unroll
                for (int c = 0; c < kPart / 8; ++c) {
                    float a[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        a[i] = __uint_as_float(raw[c * 8 + i]) * p.scale;
                    }
                    *reinterpret_cast<uint4*>(out + c * 8) = fb::pack8(a);
                }
            }
            sm100::tc_fence_before_sync();
        }
    }
    // A persistent CTA lets the next kernel in only when its own work is done: a
    // dependent that became resident earlier was measured to slow this kernel down.
    if (threadIdx.x == 0) {
        fb::dependency_release();
    }
    finish(abort_flag, tmem, 512, warp);
}

// ---- host side ---------------------------------------------------------------------------------

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

// (column 0..63, row 0..length-1, head, sequence) view of an FP16 tensor.
cudaError_t make_map(CUtensorMap* map, const AttentionView& v, const AttentionShape& s,
                     int box_rows = kTile) {
    EncodeTiled encode = nullptr;
    const cudaError_t e = encode_fn(&encode);
    if (e != cudaSuccess) {
        return e;
    }
    const cuuint64_t dims[4] = {kHead, s.length, s.heads, s.sequences};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(v.row_stride) * 2,
                                   static_cast<cuuint64_t>(v.head_stride) * 2,
                                   static_cast<cuuint64_t>(v.sequence_stride) * 2};
    const cuuint32_t box[4] = {kHead, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(v.base),
                              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

AttnParams base_params(const AttentionShape& s, float scale) {
    AttnParams p;
    std::memset(&p, 0, sizeof p);
    p.length = static_cast<int>(s.length);
    p.heads = static_cast<int>(s.heads);
    p.seqs = static_cast<int>(s.sequences);
    p.blocks = static_cast<int>((s.length + kTile - 1) / kTile);
    p.scale = scale;
    return p;
}

}  // namespace

cudaError_t attention_forward(const AttentionView& o, float* lse, const AttentionView& q,
                              const AttentionView& k, const AttentionView& v,
                              const AttentionShape& shape, float scale, cudaStream_t stream) {
    AttnParams p = base_params(shape, scale);
    cudaError_t e = make_map(&p.map_q, q, shape);
    if (e == cudaSuccess) e = make_map(&p.map_k, k, shape);
    if (e == cudaSuccess) e = make_map(&p.map_v, v, shape);
    if (e != cudaSuccess) {
        return e;
    }
    p.out0 = const_cast<void*>(o.base);
    p.out_row = o.row_stride;
    p.out_head = o.head_stride;
    p.out_seq = o.sequence_stride;
    p.lse = lse;
    static std::atomic<bool> configured[64] = {};
    e = fb::allow_shared_memory(fb_attention_forward, kFwdSmem, configured);
    if (e != cudaSuccess) {
        return e;
    }
    int sms = 148;
    sm_count(&sms);
    const long long items = static_cast<long long>((shape.sequences * shape.heads + 1) / 2) * p.blocks;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(items, sms));
    return fb::launch_dependent(fb_attention_forward, dim3(grid), dim3(kFwdThreads), kFwdSmem, stream,
                                p);
}

cudaError_t attention_backward(const AttentionView& dq, const AttentionView& dk,
                               const AttentionView& dv, const AttentionView& d_o,
                               const AttentionView& o, const float* lse, float* delta,
                               const AttentionView& q, const AttentionView& k,
                               const AttentionView& v, const AttentionShape& shape, float scale,
                               cudaStream_t stream) {
    AttnParams p = base_params(shape, scale);
    cudaError_t e = make_map(&p.map_q, q, shape);
    if (e == cudaSuccess) e = make_map(&p.map_k, k, shape);
    if (e == cudaSuccess) e = make_map(&p.map_v, v, shape);
    if (e == cudaSuccess) e = make_map(&p.map_do, d_o, shape);
    if (e == cudaSuccess) e = make_map(&p.map_q64, q, shape, kSub);
    if (e == cudaSuccess) e = make_map(&p.map_k64, k, shape, kSub);
    if (e == cudaSuccess) e = make_map(&p.map_v64, v, shape, kSub);
    if (e == cudaSuccess) e = make_map(&p.map_do64, d_o, shape, kSub);
    if (e != cudaSuccess) {
        return e;
    }
    const long long rows = static_cast<long long>(shape.length) * shape.heads * shape.sequences;
    int sms = 148;
    sm_count(&sms);
    const unsigned delta_grid =
        static_cast<unsigned>(std::min<long long>((rows + 31) / 32, sms * 16LL));
    const View vdo{static_cast<const __half*>(d_o.base), d_o.row_stride, d_o.head_stride,
                   d_o.sequence_stride};
    const View vo{static_cast<const __half*>(o.base), o.row_stride, o.head_stride,
                  o.sequence_stride};
    e = fb::launch_dependent(fb_attention_delta, dim3(delta_grid), dim3(256), 0, stream, delta, vdo,
                             vo, p.length, p.heads, p.seqs);
    if (e != cudaSuccess) {
        return e;
    }
    p.lse = const_cast<float*>(lse);
    p.delta = delta;
    // One persistent CTA per SM (fewer when there are fewer items).
    const unsigned items = static_cast<unsigned>(shape.sequences * shape.heads * p.blocks);
    const unsigned bwd_grid = std::min(items, static_cast<unsigned>(sms));

    static std::atomic<bool> dkv_configured[64] = {};
    e = fb::allow_shared_memory(fb_attention_dkv, kBwdSmem, dkv_configured);
    if (e != cudaSuccess) {
        return e;
    }
    // dK and dV must share strides (they do in both supported layouts).
    p.out0 = const_cast<void*>(dk.base);
    p.out1 = const_cast<void*>(dv.base);
    p.out_row = dk.row_stride;
    p.out_head = dk.head_stride;
    p.out_seq = dk.sequence_stride;
    e = fb::launch_dependent(fb_attention_dkv, dim3(bwd_grid), dim3(kBwdThreads), kBwdSmem, stream,
                             p);
    if (e != cudaSuccess) {
        return e;
    }
    static std::atomic<bool> dq_configured[64] = {};
    e = fb::allow_shared_memory(fb_attention_dq, kBwdSmem, dq_configured);
    if (e != cudaSuccess) {
        return e;
    }
    p.out0 = const_cast<void*>(dq.base);
    p.out1 = nullptr;
    p.out_row = dq.row_stride;
    p.out_head = dq.head_stride;
    p.out_seq = dq.sequence_stride;
    return fb::launch_dependent(fb_attention_dq, dim3(bwd_grid), dim3(kBwdThreads), kBwdSmem, stream,
                                p);
}

// ---- diagnostic: MMA rate on an idle SM ----------------------------------------------------------

__device__ long long g_mma_clocks[2];

__global__ void __launch_bounds__(128, 1) fb_mma_clocks(int n, int a_in_tmem, int count) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (sm100::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar = base + 2 * kTileBytes;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x / 32), 0);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        sm100::mbar_init(bar, 1);
        sm100::mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 2 * kTileBytes / 4; i += blockDim.x) {
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + 4u * i), "r"(0u) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        sm100::tmem_alloc(sm100::smem_u32(&tmem_slot), 512);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (warp == 0) {
        const uint32_t idesc = n == 128 ? sm100::instr_desc_f16(128, 128, false, false)
                                        : sm100::instr_desc_f16(128, 64, false, false);
        const uint64_t a_desc = desc_kmajor(base, 0);
        const uint64_t b_desc = desc_kmajor(base + kTileBytes, 0);
        const long long start = clock64();
        long long issued = start;
        if (sm100::elect_one()) {
            for (int i = 0; i < count; ++i) {
                const uint32_t step = (i & 3) * 2;
                if (a_in_tmem != 0) {
                    sm100::mma_f16_ts_at<1>(tmem, tmem + 256 + (i & 3) * 8, b_desc, step, idesc);
                } else {
                    sm100::mma_f16_ss_at<1>(tmem, a_desc, step, b_desc, step, idesc);
                }
            }
            issued = clock64();
            sm100::mma_commit(bar);
        }
        __syncwarp();
        sm100::mbar_wait(bar, 0, &abort_flag);
        const long long completed = clock64();
        if (sm100::elect_one()) {
            g_mma_clocks[0] = issued - start;
            g_mma_clocks[1] = completed - start;
        }
        sm100::tc_fence_after_sync();
    }
    finish(abort_flag, tmem, 512, warp == 0 ? 1 : 0);
}

cudaError_t mma_clocks(int n, int a_in_tmem, int count, long long* issue, long long* complete,
                       cudaStream_t stream) {
    constexpr int kSmem = 1024 + 2 * kTileBytes + 64;
    static std::atomic<bool> configured[64] = {};
    cudaError_t e = fb::allow_shared_memory(fb_mma_clocks, kSmem, configured);
    if (e != cudaSuccess) {
        return e;
    }
    fb_mma_clocks<<<1, 128, kSmem, stream>>>(n, a_in_tmem, count);
    e = fb::after_launch();
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    long long host[2] = {0, 0};
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host, g_mma_clocks, sizeof host);
    *issue = host[0];
    *complete = host[1];
    return e;
}

cudaError_t attention_error_flag(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_attention_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_attention_error, &zero, sizeof(int));
    }
    return e;
}

}  // namespace fb

namespace {

constexpr flint_status kBad = FLINT_ERROR_INVALID_ARGUMENT;


flint_status check_attention_dims(const char* name, size_t batches, size_t length,
                                  size_t head_width, float scale) {
    if (head_width != 64) {
        return fb::fail(kBad, "%s: head_width (%zu) must be 64", name, head_width);
    }
    if (length % 8 != 0 || length > 1024) {
        return fb::fail(kBad, "%s: length (%zu) must be a multiple of 8 up to 1024", name, length);
    }
    if (batches > 65535) {
        return fb::fail(kBad, "%s: batches (%zu) can be up to 65535", name, batches);
    }
    if (!std::isfinite(scale) || scale <= 0.0f) {
        return fb::fail(kBad, "%s: scale (%g) must be finite and positive", name,
                        static_cast<double>(scale));
    }
    return FLINT_OK;
}

fb::AttentionView heads_view(const void* base, size_t batches, size_t length) {
    return fb::AttentionView{base, 64, static_cast<long long>(length) * 64,
                             static_cast<long long>(batches * length) * 64};
}

}  // namespace

extern "C" {

flint_status flint_b200_attention_forward(void* o, void* lse, const void* q, const void* k,
                                          const void* v, size_t batches, size_t length,
                                          size_t head_width, float scale, flint_stream stream) {
    constexpr const char* name = "flint_b200_attention_forward";
    FB_TRY(check_attention_dims(name, batches, length, head_width, scale));
    if (batches == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t bytes = batches * length * 64 * 2;
    const fb::Span spans[] = {
        {"o", o, bytes}, {"lse", lse, batches * length * 4}, {"q", q, bytes},
        {"k", k, bytes}, {"v", v, bytes},
    };
    FB_TRY(fb::check_spans(name, spans, 2));
    const fb::AttentionShape shape{1, batches, length};
    FB_CUDA(fb::attention_forward(heads_view(o, batches, length), static_cast<float*>(lse),
                                  heads_view(q, batches, length), heads_view(k, batches, length),
                                  heads_view(v, batches, length), shape, scale, stream));
    return FLINT_OK;
}

flint_status flint_b200_attention_backward(void* dq, void* dk, void* dv, const void* d_o,
                                           const void* o, const void* lse, void* delta,
                                           const void* q, const void* k, const void* v,
                                           size_t batches, size_t length, size_t head_width,
                                           float scale, flint_stream stream) {
    constexpr const char* name = "flint_b200_attention_backward";
    FB_TRY(check_attention_dims(name, batches, length, head_width, scale));
    if (batches == 0 || length == 0) {
        return FLINT_OK;
    }
    const size_t bytes = batches * length * 64 * 2;
    const size_t stats = batches * length * 4;
    const fb::Span spans[] = {
        {"dq", dq, bytes},   {"dk", dk, bytes}, {"dv", dv, bytes}, {"delta", delta, stats},
        {"d_o", d_o, bytes}, {"o", o, bytes},   {"lse", lse, stats}, {"q", q, bytes},
        {"k", k, bytes},     {"v", v, bytes},
    };
    FB_TRY(fb::check_spans(name, spans, 4));
    const fb::AttentionShape shape{1, batches, length};
    FB_CUDA(fb::attention_backward(heads_view(dq, batches, length), heads_view(dk, batches, length),
                                   heads_view(dv, batches, length), heads_view(d_o, batches, length),
                                   heads_view(o, batches, length), static_cast<const float*>(lse),
                                   static_cast<float*>(delta), heads_view(q, batches, length),
                                   heads_view(k, batches, length), heads_view(v, batches, length), shape, scale,
                                   stream));
    return FLINT_OK;
}

flint_status flint_b200_mma_clocks(int n, int a_in_tmem, int count, long long* issue_clocks,
                                   long long* complete_clocks, flint_stream stream) {
    constexpr const char* name = "flint_b200_mma_clocks";
    if (n != 64 && n != 128) {
        return fb::fail(kBad, "%s: n (%d) must be 64 or 128", name, n);
    }
    if (count < 1 || count > 4096) {
        return fb::fail(kBad, "%s: count (%d) must be between 1 and 4096", name, count);
    }
    if (issue_clocks == nullptr || complete_clocks == nullptr) {
        return fb::fail(kBad, "%s: a result pointer is null", name);
    }
    FB_CUDA(fb::mma_clocks(n, a_in_tmem, count, issue_clocks, complete_clocks, stream));
    return FLINT_OK;
}

}  // extern "C"
