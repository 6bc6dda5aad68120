// RMSNorm, row softmax and the KV ring ops, one launch per runlist op.
// Reference routines: exec_rmsnorm2 (oplist_exec.c:1817-1872), exec_softmax
// (:1163-1194) with the host body of hvhx_v2_softmax_f32 (hvx_softmax.c:83-95),
// exec_kv_append / exec_kv_gather (:2154-2231) over the ring of kvcache.c.
#include "common.cuh"
#include "launchers.h"
#include "norm_row.cuh"

namespace gehtp {

// ------------------------------------------------------------- RMSNorm
// One CTA per row (norm_row.cuh).
template <int BLOCK>
__global__ void rmsnorm_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ r,
                               const uint16_t* __restrict__ g, const uint16_t* __restrict__ b,
                               uint16_t* __restrict__ sum_out, uint16_t* __restrict__ y,
                               uint32_t width) {
    extern __shared__ float row[];  // width floats
    __shared__ double part[BLOCK / 32];
    __shared__ float s_rms;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * width;
    rmsnorm_row<BLOCK>(a + base, r ? r + base : nullptr, g, b, sum_out ? sum_out + base : nullptr, y + base, width, row, part, &s_rms);
}

void k_add_rmsnorm(cudaStream_t st, const uint16_t* a, const uint16_t* r, const uint16_t* g,
                   const uint16_t* b, uint16_t* sum_out, uint16_t* y, uint32_t rows, uint32_t width) {
    if (!rows || !width) return;
    if (width <= 512)
        launch_pdl(rmsnorm_kernel<64>, dim3(rows), dim3(64), width * sizeof(float), st, a, r, g, b, sum_out, y, width);
    else
        launch_pdl(rmsnorm_kernel<256>, dim3(rows), dim3(256), width * sizeof(float), st, a, r, g, b, sum_out, y, width);
    g_launches++;
}

void k_rmsnorm(cudaStream_t st, const uint16_t* x, const uint16_t* g, const uint16_t* b,
               uint16_t* y, uint32_t rows, uint32_t width) {
    k_add_rmsnorm(st, x, nullptr, g, b, nullptr, y, rows, width);
}

// ------------------------------------------------------------- softmax
// One CTA per row. wide = 1: the reference's n % 32 == 0 path (fp32 exp,
// double sum, multiply by float(1/sum), one fp16 rounding). wide = 0: its
// scalar path (exp rounded to fp16 first, then divided by the fp32 sum).
template <int BLOCK>
__global__ void softmax_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                               uint32_t n, int wide) {
    __shared__ float redf[BLOCK / 32];
    __shared__ double redd[BLOCK / 32];
    __shared__ float s_mx;
    __shared__ double s_sum;
    const uint16_t* xr = x + (size_t)blockIdx.x * n;
    uint16_t* yr = y + (size_t)blockIdx.x * n;
    float mx = -3.402823466e38f;
    for (uint32_t i = threadIdx.x; i < n; i += BLOCK) mx = fmaxf(mx, h2f(xr[i]));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = redf[0];
        for (int w = 1; w < BLOCK / 32; w++) m = fmaxf(m, redf[w]);
        s_mx = m;
    }
    __syncthreads();
    mx = s_mx;
    double sum = 0.0;
    for (uint32_t i = threadIdx.x; i < n; i += BLOCK) sum += (double)expf(h2f(xr[i]) - mx);
    sum = warp_sum_d(sum);
    if ((threadIdx.x & 31) == 0) redd[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < BLOCK / 32; w++) t += redd[w];
        s_sum = t;
    }
    __syncthreads();
    if (wide) {
        const float inv = (s_sum > 0.0) ? (float)(1.0 / s_sum) : 0.0f;
        for (uint32_t i = threadIdx.x; i < n; i += BLOCK)
            yr[i] = f2h(__fmul_rn(expf(h2f(xr[i]) - mx), inv));
    } else {
        const float fs = (float)s_sum;
        for (uint32_t i = threadIdx.x; i < n; i += BLOCK)
            yr[i] = f2h(__fdiv_rn(h2f(f2h(expf(h2f(xr[i]) - mx))), fs));
    }
}

void k_softmax(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n) {
    if (!rows || !n) return;
    int wide = (n % 32u) == 0u && (size_t)rows * n >= 32u;
    if (n <= 256)
        softmax_kernel<32><<<rows, 32, 0, st>>>(x, y, n, wide);
    else
        softmax_kernel<256><<<rows, 256, 0, st>>>(x, y, n, wide);
    g_launches++;
}

// ------------------------------------------------------------- KV ring
// Ring layout (kvcache.h:19-47): slot s at ring + s*slot_elems, K face first,
// V face after kv_elems elements; posmap[s] = absolute position held, or
// 0xFFFFFFFF. One CTA: the copy is at most a few hundred KB.
__global__ void kv_append_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                                 uint16_t* __restrict__ ring, uint32_t* __restrict__ posmap,
                                 uint32_t* __restrict__ counter, uint32_t kv_elems,
                                 uint32_t nslots, uint32_t pos_const) {
    __shared__ uint32_t s_pos;
    if (threadIdx.x == 0) s_pos = (pos_const == 0xFFFFFFFAu) ? *counter : pos_const;
    __syncthreads();
    const uint32_t pos = s_pos;
    const uint32_t slot = pos % nslots;
    uint16_t* kf = ring + (size_t)slot * kv_elems * 2;
    uint16_t* vf = kf + kv_elems;
    if ((kv_elems & 7u) == 0) {
        const uint4* k4 = (const uint4*)k; const uint4* v4 = (const uint4*)v;
        uint4* kf4 = (uint4*)kf; uint4* vf4 = (uint4*)vf;
        for (uint32_t i = threadIdx.x; i < kv_elems / 8; i += blockDim.x) { kf4[i] = k4[i]; vf4[i] = v4[i]; }
    } else {
        for (uint32_t i = threadIdx.x; i < kv_elems; i += blockDim.x) { kf[i] = k[i]; vf[i] = v[i]; }
    }
    if (threadIdx.x == 0) {
        posmap[slot] = pos;
        if (pos_const == 0xFFFFFFFAu) *counter = pos + 1;
    }
}

void k_kv_append(cudaStream_t st, const uint16_t* k, const uint16_t* v, uint16_t* ring,
                 uint32_t* posmap, uint32_t* counter, uint32_t kv_elems, uint32_t nslots,
                 uint32_t pos_const) {
    kv_append_kernel<<<1, 1024, 0, st>>>(k, v, ring, posmap, counter, kv_elems, nslots, pos_const);
    g_launches++;
}

// Gather with GQA expansion: kT[h][d][p] (row stride pstride) and vo[h][p][d].
// Block = (32 positions, one KV head); the K tile is transposed through shared
// memory so both the ring reads and the kT writes are contiguous. Positions in
// [n_kv, pstride) are written as zeros. A position whose ring slot holds
// another position raises the status word ("kv gather miss").
__global__ void kv_gather_kernel(const uint16_t* __restrict__ ring,
                                 const uint32_t* __restrict__ posmap,
                                 const uint32_t* __restrict__ counter, uint16_t* __restrict__ kT,
                                 uint16_t* __restrict__ vo, uint32_t n_kv_const, uint32_t pstride,
                                 uint32_t n_heads, uint32_t kv_heads, uint32_t hd, uint32_t nslots,
                                 unsigned int* status, unsigned int op_code) {
    extern __shared__ uint16_t tile[];  // [32][hd + 2]
    const uint32_t n_kv = (n_kv_const == 0xFFFFFFFAu) ? *counter : n_kv_const;
    const uint32_t kvh = blockIdx.y;
    const uint32_t p0 = blockIdx.x * 32;
    const uint32_t rep = n_heads / kv_heads;
    const uint32_t kv_elems = kv_heads * hd;
    const uint32_t ld = hd + 2;
    // load K tile; V rows are copied straight out
    for (uint32_t e = threadIdx.x; e < 32 * hd; e += blockDim.x) {
        uint32_t pi = e / hd, d = e % hd, p = p0 + pi;
        uint16_t kval = 0, vval = 0;
        if (p < n_kv) {
            uint32_t slot = p % nslots;
            if (posmap[slot] != p) {
                raise_status(status, op_code);
            } else {
                const uint16_t* kf = ring + (size_t)slot * kv_elems * 2 + kvh * hd;
                kval = kf[d];
                vval = kf[kv_elems + d];
            }
        }
        tile[pi * ld + d] = kval;
        if (vo && p < pstride)
            for (uint32_t r = 0; r < rep; r++)
                vo[((size_t)(kvh * rep + r) * pstride + p) * hd + d] = vval;
    }
    __syncthreads();
    if (kT) {
        for (uint32_t e = threadIdx.x; e < 32 * hd; e += blockDim.x) {
            uint32_t d = e / 32, pi = e % 32, p = p0 + pi;
            if (p >= pstride) continue;
            uint16_t kval = tile[pi * ld + d];
            for (uint32_t r = 0; r < rep; r++)
                kT[((size_t)(kvh * rep + r) * hd + d) * pstride + p] = kval;
        }
    }
}

void k_kv_gather(cudaStream_t st, const uint16_t* ring, const uint32_t* posmap,
                 const uint32_t* counter, uint16_t* kT, uint16_t* vo, uint32_t n_kv_const,
                 uint32_t pstride, uint32_t n_heads, uint32_t kv_heads, uint32_t hd,
                 uint32_t nslots, unsigned int* status, unsigned int op_code) {
    if (!pstride) return;
    dim3 grid((pstride + 31) / 32, kv_heads);
    size_t smem = (size_t)32 * (hd + 2) * sizeof(uint16_t);
    kv_gather_kernel<<<grid, 256, smem, st>>>(ring, posmap, counter, kT, vo, n_kv_const, pstride,
                                             n_heads, kv_heads, hd, nslots, status, op_code);
    g_launches++;
}

}  // namespace gehtp
