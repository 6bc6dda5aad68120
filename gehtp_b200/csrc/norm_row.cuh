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
//
// The row is worked on by BLOCK consecutive threads numbered `tid` = 0..BLOCK-1 that meet at
// `sync()`: a whole CTA with __syncthreads, or a part of a larger CTA with a named barrier
// (a kernel that normalises several rows side by side). The partition of the
// sums over threads depends on BLOCK only, so both uses give the same bits. `a` and `r` are
// read with L2-only loads: they may have been written by other CTAs of the same launch.
// `load_a(i)` returns the 8 values a[i .. i+7] of the row: by default a 16-byte L2 load of `a`; a kernel that forms
// the row itself (the sum of a split-K GEMM's runs) passes its own and a null `a` - only the 16-byte paths
// use it, so such a caller must meet their conditions (width a multiple of 8, 16-byte aligned operands).
struct NormLoadGlobal {
    const uint16_t* a;
    __device__ __forceinline__ uint4 operator()(uint32_t i) const { return __ldcg((const uint4*)(a + i)); }
};

template <int BLOCK, class Sync, class LoadA>
__device__ __forceinline__ void rmsnorm_row_t(const uint32_t tid, Sync sync, LoadA load_a, const uint16_t* a, const uint16_t* r,
                                              const uint16_t* __restrict__ g, const uint16_t* __restrict__ b,
                                              uint16_t* sum_out, uint16_t* y, uint32_t width, float* row, double* part,
                                              float* s_rms) {
    // Rows of up to 4 * BLOCK * 8 values with 16-byte aligned operands: every thread keeps its (up to 32)
    // values in registers between the two passes. Same loads, sums and roundings as the general path
    // below, without the round trip through the shared row buffer.
    if ((width & 7u) == 0 && width <= 4u * BLOCK * 8u &&
        ((((uintptr_t)a) | ((uintptr_t)r) | ((uintptr_t)sum_out) | ((uintptr_t)g) | ((uintptr_t)b) | ((uintptr_t)y)) & 15u) == 0) {
        float v[4][8];
        double acc = 0.0;
        {
            uint4 qa4[4], qr4[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t i = tid * 8 + u * BLOCK * 8;
                qa4[u] = make_uint4(0, 0, 0, 0); qr4[u] = make_uint4(0, 0, 0, 0);
                if (i < width) {
                    qa4[u] = load_a(i);
                    if (r) qr4[u] = __ldcg((const uint4*)(r + i));
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t i = tid * 8 + u * BLOCK * 8;
                if (i >= width) break;
                const uint32_t wa[4] = {qa4[u].x, qa4[u].y, qa4[u].z, qa4[u].w}, wr[4] = {qr4[u].x, qr4[u].y, qr4[u].z, qr4[u].w};
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
                    v[u][2 * k] = v0;
                    v[u][2 * k + 1] = v1;
                    acc += (double)v0 * (double)v0;
                    acc += (double)v1 * (double)v1;
                }
                if (r && sum_out) *(uint4*)(sum_out + i) = make_uint4(ws[0], ws[1], ws[2], ws[3]);
            }
        }
        // gamma and beta are requested before the threads meet: their latency hides behind the reduction
        uint4 qg4[4], qb4[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t i = tid * 8 + u * BLOCK * 8;
            qg4[u] = make_uint4(0, 0, 0, 0); qb4[u] = make_uint4(0, 0, 0, 0);
            if (i < width) {
                qg4[u] = __ldg((const uint4*)(g + i));
                if (b) qb4[u] = __ldg((const uint4*)(b + i));
            }
        }
        acc = warp_sum_d(acc);
        if ((tid & 31) == 0) part[tid >> 5] = acc;
        sync();
        if (tid == 0) {
            double t = 0.0;
            for (int w = 0; w < BLOCK / 32; w++) t += part[w];
            *s_rms = (float)sqrt(t / (double)width + 1e-6);
        }
        sync();
        const float rms = *s_rms;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t i = tid * 8 + u * BLOCK * 8;
            if (i >= width) break;
            const uint32_t wg[4] = {qg4[u].x, qg4[u].y, qg4[u].z, qg4[u].w}, wb[4] = {qb4[u].x, qb4[u].y, qb4[u].z, qb4[u].w};
            uint32_t wo[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float v0 = __fdiv_rn(v[u][2 * k], rms), v1 = __fdiv_rn(v[u][2 * k + 1], rms);
                v0 = __fadd_rn(__fmul_rn(v0, h2f((uint16_t)(wg[k] & 0xffffu))), b ? h2f((uint16_t)(wb[k] & 0xffffu)) : 0.0f);
                v1 = __fadd_rn(__fmul_rn(v1, h2f((uint16_t)(wg[k] >> 16))), b ? h2f((uint16_t)(wb[k] >> 16)) : 0.0f);
                wo[k] = (uint32_t)f2h(v0) | ((uint32_t)f2h(v1) << 16);
            }
            *(uint4*)(y + i) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
        }
        return;
    }
    double acc = 0.0;
    if ((width & 7u) == 0 && ((((uintptr_t)a) | ((uintptr_t)r) | ((uintptr_t)sum_out)) & 15u) == 0) {
        // 8 values per 16-byte load; the loads of four steps are issued together (one round trip to L2,
        // not four), the sums are then formed in the same order as step by step
        for (uint32_t i0 = tid * 8; i0 < width; i0 += 4 * BLOCK * 8) {
            uint4 qa4[4], qr4[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t i = i0 + u * BLOCK * 8;
                qa4[u] = make_uint4(0, 0, 0, 0); qr4[u] = make_uint4(0, 0, 0, 0);
                if (i < width) {
                    qa4[u] = load_a(i);
                    if (r) qr4[u] = __ldcg((const uint4*)(r + i));
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t i = i0 + u * BLOCK * 8;
                if (i >= width) break;
                const uint4 qa = qa4[u], qr = qr4[u];
                uint4 qs;
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
        }
    } else {
        for (uint32_t i = tid; i < width; i += BLOCK) {
            float v = h2f(__ldcg(a + i));
            if (r) {
                uint16_t s = f2h(__fadd_rn(v, h2f(__ldcg(r + i))));
                if (sum_out) sum_out[i] = s;
                v = h2f(s);
            }
            row[i] = v;
            acc += (double)v * (double)v;
        }
    }
    acc = warp_sum_d(acc);
    if ((tid & 31) == 0) part[tid >> 5] = acc;
    sync();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < BLOCK / 32; w++) t += part[w];
        *s_rms = (float)sqrt(t / (double)width + 1e-6);
    }
    sync();
    const float rms = *s_rms;
    if ((width & 7u) == 0 && ((((uintptr_t)g) | ((uintptr_t)b) | ((uintptr_t)y)) & 15u) == 0) {
        // 8 outputs per thread and step: one 16-byte load of gamma (and beta), one 16-byte store
        for (uint32_t i = tid * 8; i < width; i += BLOCK * 8) {
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
    for (uint32_t i = tid; i < width; i += BLOCK) {
        float v = __fdiv_rn(row[i], rms);
        v = __fadd_rn(__fmul_rn(v, h2f(g[i])), b ? h2f(b[i]) : 0.0f);
        y[i] = f2h(v);
    }
}

template <int BLOCK>
__device__ __forceinline__ void rmsnorm_row(const uint16_t* a, const uint16_t* r, const uint16_t* __restrict__ g,
                                            const uint16_t* __restrict__ b, uint16_t* sum_out, uint16_t* y,
                                            uint32_t width, float* row, double* part, float* s_rms) {
    rmsnorm_row_t<BLOCK>(threadIdx.x, [] { __syncthreads(); }, NormLoadGlobal{a}, a, r, g, b, sum_out, y, width, row, part, s_rms);
}

}  // namespace gehtp
