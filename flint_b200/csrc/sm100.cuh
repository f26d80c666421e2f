// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM and
// attention kernels use: mbarriers with bounded waits, TMA tensor loads
// (each CTA always loads its own tiles), tensor-memory allocation, tcgen05.mma with
// shared-memory descriptors, tcgen05.commit and tcgen05.ld.
//
// Bit layouts of the descriptors follow the PTX ISA's "tcgen05 matrix
// descriptor" and "instruction descriptor" tables (the same fields CUTLASS's
// cute/arch/mma_sm100_desc.hpp names).
#pragma once

#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .b32 rx;\n"
        ".reg .pred px;\n"
        "elect.sync rx|px, %1;\n"
        "selp.u32 %0, 1, 0, px;\n"
        "}\n"
        : "=r"(pred)
        : "r"(0xffffffffu));
    return pred != 0;
}

// ---- mbarrier -----------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with this parity, but never forever: after about
// `limit_cycles` SM cycles, or once another thread of the CTA has raised
// *abort, it raises *abort itself and returns false. Callers then skip their
// remaining work and fall through to the CTA's teardown.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort,
                                          long long limit_cycles = 2000000000LL) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((spin & 63u) == 63u) {
            if (*abort != 0) {
                return false;
            }
            if (clock64() - start > limit_cycles) {
                *abort = 1;
                return false;
            }
        }
    }
}

// ---- TMA ---------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory -------------------------------------------------------------------

// Whole-warp calls. `columns` is a power of two from 32 to 512.
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     result_smem),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- descriptors ---------------------------------------------------------------------------

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose
// rows (K-major: one row per M/N index; MN-major: one row per K index) are
// 128 bytes long and packed, so eight rows form a 1,024-byte swizzle atom.
//   bits  0-13  start address >> 4
//   bits 16-29  leading-dimension byte offset >> 4 (MN-major: distance between
//               64-element column blocks; ignored for swizzled K-major)
//   bits 32-45  stride-dimension byte offset >> 4 (distance between 8-row groups)
//   bits 46-47  descriptor version, 1 on sm_100
//   bits 61-63  swizzle mode, 2 = 128 bytes
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= uint64_t{1} << 46;
    d |= uint64_t{2} << 61;
    return d;
}

// Instruction descriptor for kind::f16 with FP16 inputs and FP32 accumulation.
//   bits 4-5 D format (1 = F32), 7-9 A format (0 = F16), 10-12 B format,
//   bit 15 A is MN-major, bit 16 B is MN-major, bits 17-22 N >> 3, bits 24-28 M >> 4.
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n, bool a_mn_major,
                                                      bool b_mn_major) {
    return (1u << 4) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem] (A operand read from tensor memory).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same two instructions with the descriptors given as (low word + `step`, high word) and
// the accumulate flag fixed at compile time unless kAccumulate is negative (then `accumulate`
// decides): one integer addition per MMA in the issuing thread, which shares its scheduler
// with compute warps. `step` is in 16-byte units and must not carry out of the address field.
template <int kAccumulate>
__device__ __forceinline__ void mma_f16_ss_at(uint32_t d_tmem, uint64_t a_desc, uint32_t a_step,
                                              uint64_t b_desc, uint32_t b_step, uint32_t idesc,
                                              uint32_t accumulate = 0) {
    const uint32_t a_lo = static_cast<uint32_t>(a_desc) + a_step;
    const uint32_t b_lo = static_cast<uint32_t>(b_desc) + b_step;
    const uint32_t a_hi = static_cast<uint32_t>(a_desc >> 32);
    const uint32_t b_hi = static_cast<uint32_t>(b_desc >> 32);
    const uint32_t flag = kAccumulate < 0 ? accumulate : static_cast<uint32_t>(kAccumulate);
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 a, b;\n"
        "mov.b64 a, {%1, %2};\n"
        "mov.b64 b, {%3, %4};\n"
        "setp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(flag)
        : "memory");
}

template <int kAccumulate>
__device__ __forceinline__ void mma_f16_ts_at(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                              uint32_t b_step, uint32_t idesc,
                                              uint32_t accumulate = 0) {
    const uint32_t b_lo = static_cast<uint32_t>(b_desc) + b_step;
    const uint32_t b_hi = static_cast<uint32_t>(b_desc >> 32);
    const uint32_t flag = kAccumulate < 0 ? accumulate : static_cast<uint32_t>(kAccumulate);
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 b;\n"
        "mov.b64 b, {%2, %3};\n"
        "setp.ne.b32 p, %5, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], b, %4, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(flag)
        : "memory");
}

// The mbarrier gets one arrival when every tcgen05.mma issued so far by this
// thread has finished (including its reads of shared memory).
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// ---- CTA pairs (cta_group::2) -------------------------------------------------------------
//
// Two CTAs of a cluster share one tcgen05.mma: the even-ranked CTA (the leader)
// issues it, each CTA supplies its own 128 rows of A and its own half of B from
// its shared memory, and each CTA's tensor memory receives its 128 rows of D.
// Every CTA fetches its own operand tiles with its own TMA loads.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The shared::cluster address of `local` (a shared::cta address) in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

// An arrive on a barrier of another CTA of the cluster. CTA-scope release (the
// instruction's default): what the barrier hands over here is tensor memory, which the
// tcgen05 fences on either side order; a cluster-scope release would also wait for
// every earlier global and shared-memory write of the thread to become visible to the
// other SM (measured at about 2,400 clocks per arrive behind an epilogue's stores).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// TMA loads whose completion bytes may be counted on the pair leader's mbarrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1),
          "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     result_smem),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival on the mbarrier at this shared-memory offset in every CTA of
// `cta_mask`, once all MMAs issued so far have finished.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;"
        ::"r"(bar), "h"(cta_mask)
        : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators: thread i of the
// warp receives lane (base lane + i), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// The same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns (for FP16 operands: 32 values per lane,
// two per column, the lower-indexed one in the low half).
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}

// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

}  // namespace sm100
