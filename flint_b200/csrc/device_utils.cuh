// Device helpers shared by the bandwidth-bound kernels: compensated FP32
// sums with individually rounded operations, FP16 (un)packing of 128-bit
// words, and warp butterflies.
//
// The compensated sum is Knuth's TwoSum (the "Sum2" scheme of Ogita, Rump and
// Oishi): a rounded running sum plus the plain FP32 sum of the rounding errors
// it left behind. The exact operation order matters: callers compare results
// bit for bit with a plain FP32 restatement of the same order
// (reference: src/kernels/bias_gradient.cu:55-69).
#pragma once

#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace fb {

constexpr unsigned kFullMask = 0xffffffffu;

// Programmatic dependent launch (see fb::launch_dependent): dependency_wait() returns
// once every kernel this one depends on has completed and its writes are visible; it
// costs nothing in a kernel launched the ordinary way. dependency_release() lets the
// next kernel in the stream start its set-up early (it still waits, in its own
// dependency_wait(), for this kernel to finish).
__device__ __forceinline__ void dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void dependency_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

struct Comp {
    float s = 0.0f;  // rounded sum
    float e = 0.0f;  // sum of the rounding errors
};

// s + v = t + err exactly; err is accumulated into e. Every operation is an
// explicitly rounded add/sub so the compiler can neither fuse nor reassociate.
__device__ __forceinline__ void comp_add(Comp& a, float v) {
    const float t = __fadd_rn(a.s, v);
    const float vp = __fsub_rn(t, a.s);
    const float err = __fadd_rn(__fsub_rn(a.s, __fsub_rn(t, vp)), __fsub_rn(v, vp));
    a.e = __fadd_rn(a.e, err);
    a.s = t;
}

// Adds the product a*b together with the product's own rounding error (exact,
// from one fma).
__device__ __forceinline__ void comp_add_product(Comp& acc, float a, float b) {
    const float p = __fmul_rn(a, b);
    acc.e = __fadd_rn(acc.e, fmaf(a, b, -p));
    comp_add(acc, p);
}

// Two independent compensated sums side by side, on Blackwell's packed FP32
// instructions (add/sub/mul/fma.rn.f32x2): each half is rounded exactly like the
// scalar instruction, so the bits equal comp_add / comp_add_product applied to
// the halves separately, at half the instruction count.
using F2 = unsigned long long;  // two floats in a 64-bit register pair (.x low)

__device__ __forceinline__ F2 f2_pack(float lo, float hi) {
    F2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(F2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
    F2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ F2 f2_sub(F2 a, F2 b) {
    F2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
    F2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
    F2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

struct Comp2 {
    F2 s = 0;  // (+0, +0)
    F2 e = 0;
};

__device__ __forceinline__ void comp_add2(Comp2& a, F2 v) {
    const F2 t = f2_add(a.s, v);
    const F2 vp = f2_sub(t, a.s);
    const F2 err = f2_add(f2_sub(a.s, f2_sub(t, vp)), f2_sub(v, vp));
    a.e = f2_add(a.e, err);
    a.s = t;
}

__device__ __forceinline__ void comp_add_product2(Comp2& acc, F2 a, F2 b) {
    // The products are rounded by the scalar instruction: a packed multiply whose
    // result feeds a packed add was seen fused into one fma (a single rounding),
    // which an explicitly rounded scalar multiply never is.
    float a0, a1, b0, b1;
    f2_unpack(a, a0, a1);
    f2_unpack(b, b0, b1);
    const F2 p = f2_pack(__fmul_rn(a0, b0), __fmul_rn(a1, b1));
    // fma(a, b, -p) is the product's rounding error, exactly; (-0) - p negates p
    // exactly for every p, signed zeros included.
    const F2 minus_p = f2_sub(f2_pack(-0.0f, -0.0f), p);
    acc.e = f2_add(acc.e, f2_fma(a, b, minus_p));
    comp_add2(acc, p);
}

// Merges (bs, be) into a: the errors are added first, b's sum goes through
// TwoSum, then the errors are added back. Symmetric in its operands' bits.
__device__ __forceinline__ void comp_merge(Comp& a, float bs, float be) {
    const float errs = __fadd_rn(a.e, be);
    a.e = 0.0f;
    comp_add(a, bs);
    a.e = __fadd_rn(a.e, errs);
}

// The represented value. Once an inf went through TwoSum the error term is
// NaN, so a non-finite sum stands for itself.
__device__ __forceinline__ float comp_value(const Comp& a) {
    return isfinite(a.s) ? __fadd_rn(a.s, a.e) : a.s;
}

// Butterfly merge over the 32 lanes (xor 16, 8, 4, 2, 1); all lanes end with
// the same bits.
__device__ __forceinline__ Comp comp_warp_merge(Comp a) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float os = __shfl_xor_sync(kFullMask, a.s, off);
        const float oe = __shfl_xor_sync(kFullMask, a.e, off);
        comp_merge(a, os, oe);
    }
    return a;
}

__device__ __forceinline__ float warp_sum_rn(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v = __fadd_rn(v, __shfl_xor_sync(kFullMask, v, off));
    }
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(kFullMask, v, off));
    }
    return v;
}

// Eight FP16 values of a 16-byte word, widened exactly.
__device__ __forceinline__ void unpack8(float (&v)[8], const uint4& q) {
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        const float2 f = __half22float2(h);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    return make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
}

__device__ __forceinline__ void load8(float (&v)[8], const float4* p) {
    const float4 a = p[0];
    const float4 b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void store8(float4* p, const float (&v)[8]) {
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
}

}  // namespace fb
