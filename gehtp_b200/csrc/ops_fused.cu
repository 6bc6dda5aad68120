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

// Prefill form of the head of the attention block: SPLIT q, rotary chain on q, SPLIT k, rotary
// chain on k, SPLIT v (17 ops) in one pass over the projection's [tokens][q | k | v] rows.
// cos/sin tables are [tokens * heads][hd], as the chain's BINARY mul ops take them.
__global__ void qkv_split_rope_kernel(const uint16_t* qkv, const uint16_t* __restrict__ cos_q,
                                      const uint16_t* __restrict__ sin_q, const uint16_t* __restrict__ cos_k,
                                      const uint16_t* __restrict__ sin_k, uint16_t* __restrict__ q_out,
                                      uint16_t* __restrict__ k_out, uint16_t* __restrict__ v_out, uint32_t tokens,
                                      uint32_t nh, uint32_t kvh, uint32_t hd) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t h = hd / 2, wq = nh * hd, wk = kvh * hd, W = wq + 2 * wk;
    const size_t n = (size_t)tokens * W;
    for (size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; e < n; e += (size_t)gridDim.x * blockDim.x * 2) {
        const uint32_t t = (uint32_t)(e / W), c = (uint32_t)(e % W);
        const uint32_t xv = *(const uint32_t*)(qkv + e);
        if (c >= wq + wk) {
            *(uint32_t*)(v_out + (size_t)t * wk + (c - wq - wk)) = xv;
            continue;
        }
        const bool is_q = c < wq;
        const uint32_t cc = is_q ? c : c - wq, d = cc % hd;
        const size_t o = (size_t)t * (is_q ? wq : wk) + cc;
        const uint32_t pv = *(const uint32_t*)(qkv + (d < h ? e + h : e - h));
        const uint32_t cv = *(const uint32_t*)((is_q ? cos_q : cos_k) + o), sv = *(const uint32_t*)((is_q ? sin_q : sin_k) + o);
        uint16_t r[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const float xf = h2f((uint16_t)(xv >> (16 * k))), pf = h2f((uint16_t)(pv >> (16 * k)));
            const float rot = d < h ? -pf : pf;
            const float xc = h2f(f2h(__fmul_rn(xf, h2f((uint16_t)(cv >> (16 * k))))));
            const float xs = h2f(f2h(__fmul_rn(rot, h2f((uint16_t)(sv >> (16 * k))))));
            r[k] = f2h(__fadd_rn(xc, xs));
        }
        *(uint32_t*)((is_q ? q_out : k_out) + o) = (uint32_t)r[0] | ((uint32_t)r[1] << 16);
    }
}

// The same with 16-byte accesses: 8 consecutive values of a row per thread and step (head_dim a multiple of 16, so
// that a group of 8 lies in one half of a head; all operands 16-byte aligned). Same products and roundings.
__global__ void qkv_split_rope_vec8_kernel(const uint16_t* qkv, const uint16_t* __restrict__ cos_q,
                                           const uint16_t* __restrict__ sin_q, const uint16_t* __restrict__ cos_k,
                                           const uint16_t* __restrict__ sin_k, uint16_t* __restrict__ q_out,
                                           uint16_t* __restrict__ k_out, uint16_t* __restrict__ v_out, uint32_t tokens,
                                           uint32_t nh, uint32_t kvh, uint32_t hd) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t h = hd / 2, wq = nh * hd, wk = kvh * hd, W = wq + 2 * wk, W8 = W / 8;
    const uint32_t n8 = tokens * W8;          // < 2^32: the caller checks
    for (uint32_t e8 = blockIdx.x * blockDim.x + threadIdx.x; e8 < n8; e8 += gridDim.x * blockDim.x) {
        const uint32_t t = e8 / W8, c = (e8 % W8) * 8;
        const size_t e = (size_t)t * W + c;
        const uint4 xv = *(const uint4*)(qkv + e);
        if (c >= wq + wk) {
            *(uint4*)(v_out + (size_t)t * wk + (c - wq - wk)) = xv;
            continue;
        }
        const bool is_q = c < wq;
        const uint32_t cc = is_q ? c : c - wq, d = cc % hd;
        const size_t o = (size_t)t * (is_q ? wq : wk) + cc;
        const uint4 pv = *(const uint4*)(qkv + (d < h ? e + h : e - h));
        const uint4 cv = *(const uint4*)((is_q ? cos_q : cos_k) + o), sv = *(const uint4*)((is_q ? sin_q : sin_k) + o);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, pw[4] = {pv.x, pv.y, pv.z, pv.w};
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
        uint32_t r[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {
            uint16_t rr[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float xf = h2f((uint16_t)(xw[w] >> (16 * k))), pf = h2f((uint16_t)(pw[w] >> (16 * k)));
                const float rot = d < h ? -pf : pf;
                const float xc = h2f(f2h(__fmul_rn(xf, h2f((uint16_t)(cw[w] >> (16 * k))))));
                const float xs = h2f(f2h(__fmul_rn(rot, h2f((uint16_t)(sw[w] >> (16 * k))))));
                rr[k] = f2h(__fadd_rn(xc, xs));
            }
            r[w] = (uint32_t)rr[0] | ((uint32_t)rr[1] << 16);
        }
        *(uint4*)((is_q ? q_out : k_out) + o) = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

void k_qkv_split_rope(cudaStream_t st, const uint16_t* qkv, const uint16_t* cos_q, const uint16_t* sin_q,
                      const uint16_t* cos_k, const uint16_t* sin_k, uint16_t* q_out, uint16_t* k_out, uint16_t* v_out,
                      uint32_t tokens, uint32_t nh, uint32_t kvh, uint32_t hd) {
    const size_t n = (size_t)tokens * (nh + 2 * kvh) * hd;
    if (!n) return;
    const uintptr_t all = (uintptr_t)qkv | (uintptr_t)cos_q | (uintptr_t)sin_q | (uintptr_t)cos_k | (uintptr_t)sin_k | (uintptr_t)q_out |
                          (uintptr_t)k_out | (uintptr_t)v_out;
    if (hd % 16 == 0 && !(all & 15u) && n / 8 < 0xFFFFFFFFull) {
        size_t grid = (n / 8 + 255) / 256;
        if (grid > 148 * 8) grid = 148 * 8;
        launch_pdl(qkv_split_rope_vec8_kernel, dim3((unsigned)grid), dim3(256), 0, st, qkv, cos_q, sin_q, cos_k, sin_k, q_out, k_out, v_out,
                   tokens, nh, kvh, hd);
        g_launches++;
        return;
    }
    size_t grid = (n / 2 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    launch_pdl(qkv_split_rope_kernel, dim3((unsigned)grid), dim3(256), 0, st, qkv, cos_q, sin_q, cos_k, sin_k, q_out, k_out, v_out,
               tokens, nh, kvh, hd);
    g_launches++;
}

// Elementwise tail of a SwiGLU whose projections run as GEMMs (more rows than the fused
// GEMV form takes): UNARY sigmoid of the gate, BINARY mul gate * sigmoid, BINARY mul by the
// up projection, each rounded to fp16 as the three ops round.
__global__ void swiglu_tail_kernel(const uint16_t* gate, const uint16_t* up, uint16_t* __restrict__ y, size_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    auto one = [](uint16_t gh, uint16_t uh) {
        const float gt = h2f(gh);
        const float sg = h2f(f2h(1.0f / (1.0f + expf(-gt))));
        const float act = h2f(f2h(__fmul_rn(gt, sg)));
        return f2h(__fmul_rn(act, h2f(uh)));
    };
    const size_t n8 = n / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 gv = *((const uint4*)gate + i), uv = *((const uint4*)up + i);
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            r[k] = (uint32_t)one((uint16_t)gw[k], (uint16_t)uw[k]) | ((uint32_t)one((uint16_t)(gw[k] >> 16), (uint16_t)(uw[k] >> 16)) << 16);
        *((uint4*)y + i) = make_uint4(r[0], r[1], r[2], r[3]);
    }
    if (blockIdx.x == 0)
        for (size_t i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) y[i] = one(gate[i], up[i]);
}

void k_swiglu_tail(cudaStream_t st, const uint16_t* gate, const uint16_t* up, uint16_t* y, size_t n) {
    if (!n) return;
    size_t grid = (n / 8 + 255) / 256;
    if (grid < 1) grid = 1;
    if (grid > 148 * 16) grid = 148 * 16;
    launch_pdl(swiglu_tail_kernel, dim3((unsigned)grid), dim3(256), 0, st, gate, up, y, n);
    g_launches++;
}

}  // namespace gehtp
