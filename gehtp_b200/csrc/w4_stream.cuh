// Warp-level pieces of the streaming W4A16 matmul, used by the one-op kernels
// (ops_w4a16.cu): the strip-major unit -> mma.m16n8k16 fragments, one 64-deep scale group per call.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace gehtp {

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Activations are written by the preceding kernel of the stream, so they may
// only be read after griddepcontrol.wait. A read-only (.nc) load could be moved
// above the wait by the compiler; this one cannot.
__device__ __forceinline__ uint4 ld_ordered(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// (a & b) | c in one LOP3 (truth table 0xEA).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One packed word -> four fp16 pairs holding q - 8 (exact). The group scale is
// applied to the fp32 partial sum of the 64-deep group after the MMAs: the
// scale is constant along k inside a group and per output column, i.e. per
// accumulator row, so 4 FFMAs per group replace 16 half2 multiplies.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t MAGIC = 0x64006400u;          // 1024.0 in both halves
    const __half2 c1032 = __half2half2(__ushort_as_half(0x6408));   // 1032
    const __half2 c16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
    const __half2 cm72 = __half2half2(__ushort_as_half(0xd480));    // -72
    const uint32_t w8 = w >> 8;
    const uint32_t p0 = and_or(w, 0x000f000fu, MAGIC);    // 1024 + q
    const uint32_t p1 = and_or(w, 0x00f000f0u, MAGIC);    // 1024 + 16 q
    const uint32_t p2 = and_or(w8, 0x000f000fu, MAGIC);
    const uint32_t p3 = and_or(w8, 0x00f000f0u, MAGIC);
    __half2 h0 = __hsub2(*(__half2*)&p0, c1032);
    __half2 h1 = __hfma2(*(__half2*)&p1, c16th, cm72);
    __half2 h2 = __hsub2(*(__half2*)&p2, c1032);
    __half2 h3 = __hfma2(*(__half2*)&p3, c16th, cm72);
    a[0] = *(uint32_t*)&h0;
    a[1] = *(uint32_t*)&h1;
    a[2] = *(uint32_t*)&h2;
    a[3] = *(uint32_t*)&h3;
}

// Same with C = 0 (starts a fresh partial sum).
__device__ __forceinline__ void mma16816_first(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ void mma_group(float (&acc)[4], const uint32_t (&af)[4][4], uint4 b0,
                                          uint4 b1, float slo, float shi) {
    float gacc[4];
    mma16816_first(gacc, af[0], b0.x, b0.y);
    mma16816(gacc, af[1], b0.z, b0.w);
    mma16816(gacc, af[2], b1.x, b1.y);
    mma16816(gacc, af[3], b1.z, b1.w);
    acc[0] = fmaf(gacc[0], slo, acc[0]);     // rows g: columns 2t, 2t+1
    acc[1] = fmaf(gacc[1], slo, acc[1]);
    acc[2] = fmaf(gacc[2], shi, acc[2]);     // rows g+8
    acc[3] = fmaf(gacc[3], shi, acc[3]);
}

// SwiGLU on two accumulators with the op chain's roundings: gate -> fp16,
// sigmoid -> fp16, gate*sigmoid -> fp16, up -> fp16, product -> fp16
// (UNARY subtype 8 and two BINARY mul ops of the reference executor).
__device__ __forceinline__ uint16_t swiglu_chain(float gate_acc, float up_acc) {
    float gt = h2f(f2h(gate_acc));
    float sg = h2f(f2h(1.0f / (1.0f + expf(-gt))));
    float act = h2f(f2h(__fmul_rn(gt, sg)));
    float up = h2f(f2h(up_acc));
    return f2h(__fmul_rn(act, up));
}

// Two SwiGLU chains at once, packed: the same roundings through half2 conversions and fp16 multiplies (the fp32
// product of two fp16 values is exact, so one rounding to fp16 either way; 1 / x as the correctly rounded reciprocal
// is the IEEE quotient 1.0f / x). No branch, so that a caller's independent pairs overlap their latencies. A NaN
// anywhere in a chain reaches the result as a NaN: `nan` is set then, and the caller redoes such pairs with
// swiglu_chain, whose conversions turn a NaN into a signed infinity.
__device__ __forceinline__ uint32_t swiglu_pair_fast(float g0, float g1, float u0, float u1, bool& nan) {
    const __half2 gh = __floats2half2_rn(g0, g1);
    const float2 gf = __half22float2(gh);
    const __half2 sh = __floats2half2_rn(__frcp_rn(1.0f + expf(-gf.x)), __frcp_rn(1.0f + expf(-gf.y)));
    const __half2 out = __hmul2(__hmul2(gh, sh), __floats2half2_rn(u0, u1));
    nan |= __hisnan(__low2half(out)) || __hisnan(__high2half(out));
    return *(const uint32_t*)&out;
}

__device__ __forceinline__ uint32_t swiglu_chain2(float g0, float g1, float u0, float u1) {
    bool nan = false;
    const uint32_t r = swiglu_pair_fast(g0, g1, u0, u1, nan);
    return nan ? ((uint32_t)swiglu_chain(g0, u0) | ((uint32_t)swiglu_chain(g1, u1) << 16)) : r;
}

}  // namespace gehtp
