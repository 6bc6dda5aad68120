// Kernels that stand for a chain of runlist ops (used by the plan-time fusion).
// Each keeps the fp16 rounding points of the op-by-op form, so results are
// the ones the chain produces.
#include "common.cuh"
#include "launchers_attn.h"

namespace gehtp {

// SPLIT x3 + rotary embedding on q and k (BINARY mul by the cos face, SLICE
// halves, UNARY neg, CONCAT, BINARY mul by the sin face, ADD — the
// decomposition the reference emitter produces, ops 5-13 of its probe blob) +
// KV_APPEND of the rotated k and of v at the state's position counter.
// qkv rows are [q: nh*hd | k: kvh*hd | v: kvh*hd] per sequence. The rotated q
// goes to q_out; k and v go straight into the ring slot of the position.
__global__ void rope_kv_append_kernel(const uint16_t* __restrict__ qkv, const uint16_t* __restrict__ cos_q,
                                      const uint16_t* __restrict__ sin_q, const uint16_t* __restrict__ cos_k,
                                      const uint16_t* __restrict__ sin_k, uint16_t* __restrict__ q_out,
                                      uint16_t* __restrict__ ring, uint32_t* __restrict__ posmap,
                                      const uint32_t* __restrict__ counter, uint32_t B, uint32_t nh,
                                      uint32_t kvh, uint32_t hd, uint32_t nslots, uint32_t pos_const) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t pos = (pos_const == 0xFFFFFFFAu) ? *counter : pos_const;
    const uint32_t slot = pos % nslots;
    const uint32_t row_w = (nh + 2 * kvh) * hd, h = hd / 2;
    const uint32_t kv_elems = B * kvh * hd;
    uint16_t* kf = ring + (size_t)slot * kv_elems * 2;
    uint16_t* vf = kf + kv_elems;
    const uint32_t nq = B * nh * hd, nk = B * kvh * hd;
    const uint32_t total = nq + 2 * nk;
    for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        if (e < nq) {
            uint32_t b = e / (nh * hd), r = e % (nh * hd), d = r % hd;
            const uint16_t* src = qkv + (size_t)b * row_w + (r - d);
            float x = h2f(src[d]);
            float rot = d < h ? -h2f(src[d + h]) : h2f(src[d - h]);
            float xc = h2f(f2h(__fmul_rn(x, h2f(cos_q[e]))));
            float xs = h2f(f2h(__fmul_rn(rot, h2f(sin_q[e]))));
            q_out[e] = f2h(__fadd_rn(xc, xs));
        } else if (e < nq + nk) {
            uint32_t i = e - nq;
            uint32_t b = i / (kvh * hd), r = i % (kvh * hd), d = r % hd;
            const uint16_t* src = qkv + (size_t)b * row_w + nh * hd + (r - d);
            float x = h2f(src[d]);
            float rot = d < h ? -h2f(src[d + h]) : h2f(src[d - h]);
            float xc = h2f(f2h(__fmul_rn(x, h2f(cos_k[i]))));
            float xs = h2f(f2h(__fmul_rn(rot, h2f(sin_k[i]))));
            kf[i] = f2h(__fadd_rn(xc, xs));
        } else {
            uint32_t i = e - nq - nk;
            uint32_t b = i / (kvh * hd), r = i % (kvh * hd);
            vf[i] = qkv[(size_t)b * row_w + (nh + kvh) * hd + r];
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) posmap[slot] = pos;
}

void k_rope_kv_append(cudaStream_t st, const uint16_t* qkv, const uint16_t* cos_q, const uint16_t* sin_q,
                      const uint16_t* cos_k, const uint16_t* sin_k, uint16_t* q_out, uint16_t* ring,
                      uint32_t* posmap, const uint32_t* counter, uint32_t B, uint32_t nh, uint32_t kvh,
                      uint32_t hd, uint32_t nslots, uint32_t pos_const) {
    uint32_t total = B * (nh + 2 * kvh) * hd;
    uint32_t grid = (total + 255) / 256;
    if (grid > 148 * 8) grid = 148 * 8;
    launch_pdl(rope_kv_append_kernel, dim3(grid), dim3(256), 0, st, qkv, cos_q, sin_q, cos_k, sin_k, q_out, ring, posmap, counter,
               B, nh, kvh, hd, nslots, pos_const);
    g_launches++;
}

// Rotary embedding on its own (the same seven-op chain, without the split and
// the append): x, cos, sin and out are [rows][hd].
__global__ void rope_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ cos_t,
                            const uint16_t* __restrict__ sin_t, uint16_t* __restrict__ out, uint32_t n, uint32_t hd) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t h = hd / 2;
    // two elements per thread (d even): both read the same partner pair
    for (uint32_t e = (blockIdx.x * blockDim.x + threadIdx.x) * 2; e < n; e += gridDim.x * blockDim.x * 2) {
        const uint32_t d = e % hd;
        const uint32_t pe = d < h ? e + h : e - h;
        const uint32_t xv = *(const uint32_t*)(x + e), pv = *(const uint32_t*)(x + pe);
        const uint32_t cv = *(const uint32_t*)(cos_t + e), sv = *(const uint32_t*)(sin_t + e);
        uint16_t r[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const float xf = h2f((uint16_t)(xv >> (16 * k))), pf = h2f((uint16_t)(pv >> (16 * k)));
            const float rot = d < h ? -pf : pf;
            const float xc = h2f(f2h(__fmul_rn(xf, h2f((uint16_t)(cv >> (16 * k))))));
            const float xs = h2f(f2h(__fmul_rn(rot, h2f((uint16_t)(sv >> (16 * k))))));
            r[k] = f2h(__fadd_rn(xc, xs));
        }
        *(uint32_t*)(out + e) = (uint32_t)r[0] | ((uint32_t)r[1] << 16);
    }
}

void k_rope(cudaStream_t st, const uint16_t* x, const uint16_t* cos_t, const uint16_t* sin_t, uint16_t* out,
            uint32_t rows, uint32_t hd) {
    const uint32_t n = rows * hd;
    if (!n) return;
    uint32_t grid = (n / 2 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    launch_pdl(rope_kernel, dim3(grid), dim3(256), 0, st, x, cos_t, sin_t, out, n, hd);
    g_launches++;
}

}  // namespace gehtp
