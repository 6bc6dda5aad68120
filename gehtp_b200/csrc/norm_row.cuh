// RMSNorm of one row per CTA, shared by the plain kernel and the tensor-parallel
// form that all-reduces one addend first.
#pragma once
#include "common.cuh"

namespace gehtp {

// Sum of squares in double, rms = float(sqrt(acc/n + 1e-6)), then x / rms,
// * gamma, + beta, each rounded separately in fp32, one fp16 rounding at the
// end (exec_rmsnorm2, oplist_exec.c:1817-1872). When `r` is given the row is
// f16(a + r) first (the residual add that precedes the norm in a decoder
// block) and that sum is also stored to sum_out. `row` holds width floats of
// shared memory; `part` BLOCK/32 doubles; all pointers are row-based.
template <int BLOCK>
__device__ __forceinline__ void rmsnorm_row(const uint16_t* a, const uint16_t* r, const uint16_t* __restrict__ g,
                                            const uint16_t* __restrict__ b, uint16_t* sum_out, uint16_t* y,
                                            uint32_t width, float* row, double* part, float* s_rms) {
    double acc = 0.0;
    if ((width & 7u) == 0 && ((((uintptr_t)a) | ((uintptr_t)r) | ((uintptr_t)sum_out)) & 15u) == 0) {
        // 8 values per 16-byte load
        for (uint32_t i = threadIdx.x * 8; i < width; i += BLOCK * 8) {
            uint4 qa = *(const uint4*)(a + i), qr = make_uint4(0, 0, 0, 0), qs;
            if (r) qr = *(const uint4*)(r + i);
            const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wr[4] = {qr.x, qr.y, qr.z, qr.w};
            uint32_t ws[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float v0 = h2f((uint16_t)(wa[k] & 0xffffu)), v1 = h2f((uint16_t)(wa[k] >> 16));
                if (r) {
                    uint16_t s0 = f2h(__fadd_rn(v0, h2f((uint16_t)(wr[k] & 0xffffu))));
                    uint16_t s1 = f2h(__fadd_rn(v1, h2f((uint16_t)(wr[k] >> 16))));
                    ws[k] = (uint32_t)s0 | ((uint32_t)s1 << 16);
                    v0 = h2f(s0); v1 = h2f(s1);
                }
                row[i + 2 * k] = v0;
                row[i + 2 * k + 1] = v1;
                acc += (double)v0 * (double)v0;
                acc += (double)v1 * (double)v1;
            }
            if (r && sum_out) { qs = make_uint4(ws[0], ws[1], ws[2], ws[3]); *(uint4*)(sum_out + i) = qs; }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < width; i += BLOCK) {
            float v = h2f(a[i]);
            if (r) {
                uint16_t s = f2h(__fadd_rn(v, h2f(r[i])));
                if (sum_out) sum_out[i] = s;
                v = h2f(s);
            }
            row[i] = v;
            acc += (double)v * (double)v;
        }
    }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < BLOCK / 32; w++) t += part[w];
        *s_rms = (float)sqrt(t / (double)width + 1e-6);
    }
    __syncthreads();
    const float rms = *s_rms;
    if ((width & 7u) == 0 && ((((uintptr_t)g) | ((uintptr_t)b) | ((uintptr_t)y)) & 15u) == 0) {
        // 8 outputs per thread and step: one 16-byte load of gamma (and beta), one 16-byte store
        for (uint32_t i = threadIdx.x * 8; i < width; i += BLOCK * 8) {
            const uint4 qg = __ldg((const uint4*)(g + i));
            uint4 qb = make_uint4(0, 0, 0, 0);
            if (b) qb = __ldg((const uint4*)(b + i));
            const uint32_t wg[4] = {qg.x, qg.y, qg.z, qg.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
            uint32_t wo[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float v0 = __fdiv_rn(row[i + 2 * k], rms), v1 = __fdiv_rn(row[i + 2 * k + 1], rms);
                v0 = __fadd_rn(__fmul_rn(v0, h2f((uint16_t)(wg[k] & 0xffffu))), b ? h2f((uint16_t)(wb[k] & 0xffffu)) : 0.0f);
                v1 = __fadd_rn(__fmul_rn(v1, h2f((uint16_t)(wg[k] >> 16))), b ? h2f((uint16_t)(wb[k] >> 16)) : 0.0f);
                wo[k] = (uint32_t)f2h(v0) | ((uint32_t)f2h(v1) << 16);
            }
            *(uint4*)(y + i) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
        }
        return;
    }
    for (uint32_t i = threadIdx.x; i < width; i += BLOCK) {
        float v = __fdiv_rn(row[i], rms);
        v = __fadd_rn(__fmul_rn(v, h2f(g[i])), b ? h2f(b[i]) : 0.0f);
        y[i] = f2h(v);
    }
}

}  // namespace gehtp
