// Prefill attention: softmax(Q K^T * scale + mask) V over whole sequences,
// grouped-query heads, flash style (no S x S temp).
//
// It replaces the op chain the runlist carries for this step: TRANSPOSE_GEN of
// q, k and v into head-major faces, batched MATMUL_F16 for the scores
// (oplist_exec.c:1787-1800), the scale multiply/divide and the additive mask
// (exec_binary / exec_add), SOFTMAX (:1163-1194), the batched MATMUL_F16 with V
// and the TRANSPOSE_GEN back to token-major. The fp16 roundings the chain
// applies to a score (after the dot product, after the scale, after the mask)
// are reproduced; the softmax runs in fp32 over unnormalised exponentials,
// which differs from the chain only in rounding.
//
// Layout: q [seq_q][n_heads][hd], k and v [seq_k][kv_heads][hd] (token-major, as
// the projections leave them), out [seq_q][n_heads * hd]. Query head h uses KV
// head h / rep. One CTA = one query head x 64 query rows (16 per warp); K/V
// tiles of 64 positions go through shared memory with cp.async (2 stages,
// 16-byte chunks XOR-swizzled by row), are read with ldmatrix and multiplied
// with mma.sync m16n8k16. Tiles whose mask is -inf everywhere (the upper
// triangle of a causal mask, found on the host from the constant mask slot)
// are skipped: they contribute exact zeros.
#include <cuda_fp16.h>
#include "common.cuh"
#include "launchers_attn.h"

namespace gehtp {

namespace {

constexpr int PF_BQ = 64, PF_BK = 64, PF_WARPS = 4;

__device__ __forceinline__ void pf_cp16(uint32_t smem, const void* gmem, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void pf_ldsm(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void pf_ldsm_t(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&h;
}
__device__ __forceinline__ float pf_round(float x) { return __half2float(__float2half_rn(x)); }
// score as the op chain leaves it: fp16 after the dot, after the scale, after the mask
__device__ __forceinline__ float pf_score(float dot, float scale, int scale_div, float maskv) {
    float s = pf_round(dot);
    s = pf_round(scale_div ? __fdiv_rn(s, scale) : __fmul_rn(s, scale));
    return pf_round(__fadd_rn(s, maskv));
}

struct PrefillArgs {
    const uint16_t *q, *k, *v;
    const uint16_t* mask;        // [heads or 1][seq_q][seq_k] additive fp16, or NULL
    size_t mask_head_stride;     // elements between the masks of two heads (0 = shared)
    const uint8_t* skip;         // [q tiles][k tiles], 1 = tile fully masked, or NULL
    uint16_t* out;
    uint32_t seq_q, seq_k, nh, kvh;
    float scale;
    int scale_div;
};

template <int HD>
__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(PrefillArgs A) {
    constexpr int ROWB = HD * 2, CHUNKS = ROWB / 16, KSTEPS = HD / 16, DBLK = HD / 8;
    constexpr int TILE_B = PF_BK * ROWB;
    extern __shared__ __align__(128) unsigned char pf_smem[];
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(pf_smem);
    const uint32_t sK = sQ + PF_BQ * ROWB, sV = sK + 2 * TILE_B;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t qt = blockIdx.x, head = blockIdx.y, kvhd = head / (A.nh / A.kvh);
    const uint32_t q0 = qt * PF_BQ;
    const uint32_t n_kt = (A.seq_k + PF_BK - 1) / PF_BK;
    const uint8_t* skip = A.skip ? A.skip + (size_t)qt * n_kt : nullptr;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Q tile -> shared (rows past seq_q are zero)
    for (int idx = tid; idx < PF_BQ * CHUNKS; idx += PF_WARPS * 32) {
        const int row = idx / CHUNKS, ch = idx % CHUNKS;
        const uint32_t qr = q0 + row;
        const bool ok = qr < A.seq_q;
        const uint16_t* src = A.q + ((size_t)(ok ? qr : 0) * A.nh + head) * HD + ch * 8;
        pf_cp16(sQ + row * ROWB + ((ch ^ (row & 7)) << 4), src, ok);
    }
    pf_commit();
    auto issue = [&](uint32_t kt, int stage) {
        const uint32_t p0 = kt * PF_BK;
        for (int idx = tid; idx < PF_BK * CHUNKS; idx += PF_WARPS * 32) {
            const int row = idx / CHUNKS, ch = idx % CHUNKS;
            const uint32_t p = p0 + row;
            const bool ok = p < A.seq_k;
            const size_t off = ((size_t)(ok ? p : 0) * A.kvh + kvhd) * HD + ch * 8;
            const uint32_t so = row * ROWB + ((ch ^ (row & 7)) << 4);
            pf_cp16(sK + stage * TILE_B + so, A.k + off, ok);
            pf_cp16(sV + stage * TILE_B + so, A.v + off, ok);
        }
    };
    // first live tile
    uint32_t kt = 0;
    while (kt < n_kt && skip && skip[kt]) kt++;
    if (kt < n_kt) issue(kt, 0);
    pf_commit();

    uint32_t qa[KSTEPS][4];
    float o[DBLK][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    pf_wait<1>();
    __syncthreads();
    {
        // A fragments of this warp's 16 query rows
        const int mat = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (mat & 1) * 8 + r;
#pragma unroll
        for (int j = 0; j < KSTEPS; j++) {
            const int ch = j * 2 + (mat >> 1);
            pf_ldsm(qa[j], sQ + row * ROWB + ((ch ^ (row & 7)) << 4));
        }
    }
    const uint32_t qrow0 = q0 + warp * 16 + g, qrow1 = qrow0 + 8;
    const uint16_t* mbase = A.mask ? A.mask + (size_t)head * A.mask_head_stride : nullptr;
    int stage = 0;
    while (kt < n_kt) {
        uint32_t nxt = kt + 1;
        while (nxt < n_kt && skip && skip[nxt]) nxt++;
        if (nxt < n_kt) issue(nxt, stage ^ 1);
        pf_commit();
        pf_wait<1>();
        __syncthreads();
        const uint32_t k_s = sK + stage * TILE_B, v_s = sV + stage * TILE_B;
        const uint32_t p0 = kt * PF_BK;
        float s[PF_BK / 8][4];
#pragma unroll
        for (int nb = 0; nb < PF_BK / 8; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
        for (int j = 0; j < KSTEPS; j++) {
#pragma unroll
            for (int np = 0; np < PF_BK / 16; np++) {
                uint32_t kb[4];
                const int mat = lane >> 3, r = lane & 7;
                const int row = np * 16 + (mat >> 1) * 8 + r;
                const int ch = j * 2 + (mat & 1);
                pf_ldsm(kb, k_s + row * ROWB + ((ch ^ (row & 7)) << 4));
                pf_mma(s[np * 2], qa[j], kb[0], kb[1]);
                pf_mma(s[np * 2 + 1], qa[j], kb[2], kb[3]);
            }
        }
        // scores -> chain roundings, running max
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < PF_BK / 8; nb++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t p = p0 + nb * 8 + 2 * t + (c & 1);
                const uint32_t qr = (c & 2) ? qrow1 : qrow0;
                float v = -INFINITY;
                if (p < A.seq_k && qr < A.seq_q) {
                    const float mk = mbase ? __half2float(__ushort_as_half(mbase[(size_t)qr * A.seq_k + p])) : 0.0f;
                    v = pf_score(s[nb][c], A.scale, A.scale_div, mk);
                }
                s[nb][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            alpha[h] = (m_new == -INFINITY) ? 1.0f : __expf(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= alpha[h];
        }
#pragma unroll
        for (int nb = 0; nb < PF_BK / 8; nb++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float mr = m_run[c >> 1];
                const float e = (mr == -INFINITY) ? 0.0f : __expf(s[nb][c] - mr);
                s[nb][c] = e;
                l_run[c >> 1] += e;
            }
        if (alpha[0] != 1.0f || alpha[1] != 1.0f) {
#pragma unroll
            for (int i = 0; i < DBLK; i++) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int kk = 0; kk < PF_BK / 16; kk++) {
            uint32_t pa[4];
            pa[0] = pf_pack(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pf_pack(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DBLK / 2; dp++) {
                uint32_t vb[4];
                const int mat = lane >> 3, r = lane & 7;
                const int row = kk * 16 + (mat & 1) * 8 + r;
                const int ch = dp * 2 + (mat >> 1);
                pf_ldsm_t(vb, v_s + row * ROWB + ((ch ^ (row & 7)) << 4));
                pf_mma(o[dp * 2], pa, vb[0], vb[1]);
                pf_mma(o[dp * 2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();   // every warp is done with this stage before it is refilled
        stage ^= 1;
        kt = nxt;
    }
    pf_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
#pragma unroll
    for (int i = 0; i < DBLK; i++) {
        const int d = i * 8 + 2 * t;
        if (qrow0 < A.seq_q)
            *(uint32_t*)(A.out + ((size_t)qrow0 * A.nh + head) * HD + d) = (uint32_t)f2h(o[i][0] * inv0) | ((uint32_t)f2h(o[i][1] * inv0) << 16);
        if (qrow1 < A.seq_q)
            *(uint32_t*)(A.out + ((size_t)qrow1 * A.nh + head) * HD + d) = (uint32_t)f2h(o[i][2] * inv1) | ((uint32_t)f2h(o[i][3] * inv1) << 16);
    }
}

}  // namespace

uint32_t attn_prefill_tile() { return PF_BQ; }

bool k_attn_prefill(cudaStream_t st, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask,
                    size_t mask_head_stride, const uint8_t* skip, float scale, int scale_div, uint32_t seq_q,
                    uint32_t seq_k, uint32_t nh, uint32_t kvh, uint32_t hd, uint16_t* out) {
    if (!seq_q || !seq_k || !kvh || nh % kvh || (hd != 128 && hd != 64)) return false;
    if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v)) & 15u || ((uintptr_t)out & 3u)) return false;
    PrefillArgs a{q, k, v, mask, mask_head_stride, skip, out, seq_q, seq_k, nh, kvh, scale, scale_div};
    const dim3 grid((seq_q + PF_BQ - 1) / PF_BQ, nh);
    const size_t smem = (size_t)(PF_BQ + 4 * PF_BK) * hd * 2;
    if (hd == 128) {
        static int have[64] = {};
        if (!ensure_dyn_smem(attn_prefill_kernel<128>, smem, have)) return false;
        launch_pdl(attn_prefill_kernel<128>, grid, dim3(PF_WARPS * 32), smem, st, a);
    } else {
        static int have[64] = {};
        if (!ensure_dyn_smem(attn_prefill_kernel<64>, smem, have)) return false;
        launch_pdl(attn_prefill_kernel<64>, grid, dim3(PF_WARPS * 32), smem, st, a);
    }
    g_launches++;
    return true;
}

}  // namespace gehtp
