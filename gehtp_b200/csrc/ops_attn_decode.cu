// Decode attention read straight off the KV ring: softmax(q K^T * scale + mask) V
// for one new token per sequence, grouped-query heads, split over the context.
//
// It replaces the op chain the runlist carries for this step — KV_GATHER (K^T
// and V faces, GQA-expanded, oplist_exec.c:2183-2231), batched MATMUL_F16 for
// the scores (:1787-1800), the scale multiply/divide and the additive mask
// (exec_binary / exec_add), SOFTMAX (:1163-1194) and the batched MATMUL_F16
// with V — without materialising any of those faces. The fp16 roundings the
// chain applies to the score (after the dot product, after the scale, after
// the mask) are reproduced; the softmax runs in fp32 over unnormalised
// exponentials (flash style), which differs from the chain only in rounding.
//
// Layout. Ring slot s = [K face: kv_heads x hd][V face: same] (kvcache.h:19-47);
// position p lives in slot p % nslots. Query head h uses KV head h / rep.
// One CTA = one KV head x one slice of the context; its `rep` query heads are
// the rows of a 16-row tensor-core tile, so K and V are read once per group.
// K/V tiles of 64 positions are staged in shared memory with cp.async (3
// stages, 16-byte chunks XOR-swizzled by row), read back with ldmatrix and
// multiplied with mma.sync m16n8k16. Each CTA writes (max, sum, unnormalised
// output) for its slice to a scratch buffer; a second small kernel merges the
// slices in slice order.
#include <cuda_fp16.h>
#include "common.cuh"
#include "launchers_attn.h"

namespace gehtp {

namespace {

constexpr int TILE = 64;      // positions per stage
constexpr int STAGES = 3;
constexpr int NWARP = 4;      // 16 positions of a tile each

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *(uint32_t*)&h;
}
__device__ __forceinline__ float round_h(float x) { return __half2float(__float2half_rn(x)); }

// score as the op chain leaves it: fp16 after the dot, after the scale, after the mask
__device__ __forceinline__ float chain_score(float dot, float scale, int scale_div, float maskv) {
    float s = round_h(dot);
    s = round_h(scale_div ? __fdiv_rn(s, scale) : __fmul_rn(s, scale));
    return round_h(__fadd_rn(s, maskv));
}

template <int HD>
__global__ void __launch_bounds__(NWARP * 32)
attn_decode_split_kernel(AttnDecodeArgs A) {
    constexpr int ROWB = HD * 2;          // bytes per K or V row
    constexpr int CHUNKS = ROWB / 16;     // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    constexpr int DBLK = HD / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t rep = A.rep;
    const uint32_t n_kv = A.counter ? *A.counter + A.n_kv_add : A.n_kv;
    uint32_t per = (n_kv + A.nsplit - 1) / A.nsplit;
    per = (per + TILE - 1) / TILE * TILE;
    const uint32_t p_begin = split * per;
    const uint32_t p_end = (p_begin + per < n_kv) ? p_begin + per : n_kv;
    const uint32_t kv_elems = A.kv_heads * HD;
    const uint16_t* ring_k = A.ring + (size_t)kvh * HD;
    const uint16_t* maskp = A.mask ? A.mask + (size_t)(kvh / A.kvh_per_seq) * A.mask_seq_stride : nullptr;

    // Q fragments: rows = the group's query heads (zero rows beyond rep)
    uint32_t qa[KSTEPS][4];
    {
        const uint16_t* q0 = A.q + ((size_t)kvh * rep + g) * HD;
        const uint16_t* q1 = A.q + ((size_t)kvh * rep + g + 8) * HD;
#pragma unroll
        for (int j = 0; j < KSTEPS; j++) {
            qa[j][0] = (uint32_t)g < rep ? *(const uint32_t*)(q0 + 16 * j + 2 * t) : 0u;
            qa[j][1] = (uint32_t)(g + 8) < rep ? *(const uint32_t*)(q1 + 16 * j + 2 * t) : 0u;
            qa[j][2] = (uint32_t)g < rep ? *(const uint32_t*)(q0 + 16 * j + 2 * t + 8) : 0u;
            qa[j][3] = (uint32_t)(g + 8) < rep ? *(const uint32_t*)(q1 + 16 * j + 2 * t + 8) : 0u;
        }
    }

    float o[DBLK][4];
#pragma unroll
    for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    const int ntiles = p_end > p_begin ? (int)((p_end - p_begin + TILE - 1) / TILE) : 0;
    auto issue = [&](int tile) {
        if (tile < ntiles) {
            unsigned char* sk = smem + (size_t)(tile % STAGES) * (2 * TILE * ROWB);
            unsigned char* sv = sk + TILE * ROWB;
            const uint32_t p0 = p_begin + tile * TILE;
            for (int idx = tid; idx < TILE * CHUNKS; idx += NWARP * 32) {
                int row = idx / CHUNKS, ch = idx % CHUNKS;
                uint32_t p = p0 + row;
                bool ok = p < p_end;
                uint32_t slot = ok ? p % A.nslots : 0;
                const uint16_t* src = ring_k + (size_t)slot * kv_elems * 2 + ch * 8;
                int so = row * ROWB + ((ch ^ (row & 7)) << 4);
                cp_async16(sk + so, src, ok);
                cp_async16(sv + so, src + kv_elems, ok);
            }
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    for (int tile = 0; tile < ntiles; tile++) {
        issue(tile + 2);
        cp_async_wait<2>();
        __syncthreads();
        const unsigned char* sk = smem + (size_t)(tile % STAGES) * (2 * TILE * ROWB);
        const unsigned char* sv = sk + TILE * ROWB;
        const int wrow0 = warp * 16;
        const uint32_t pw0 = p_begin + tile * TILE + wrow0;
        if (pw0 < p_end) {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int j = 0; j < KSTEPS; j++) {
                uint32_t kb[4];
                int mat = lane >> 3, r = lane & 7;
                int row = wrow0 + (mat >> 1) * 8 + r;
                int ch = j * 2 + (mat & 1);
                ldsm_x4(kb, sk + row * ROWB + ((ch ^ (row & 7)) << 4));
                mma_f16(s[0], qa[j], kb[0], kb[1]);
                mma_f16(s[1], qa[j], kb[2], kb[3]);
            }
            // scores -> chain roundings, mask, running max
            float x[2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t p = pw0 + nb * 8 + 2 * t + (c & 1);
                    float v = -INFINITY;
                    if (p < p_end) {
                        float mk = maskp ? __half2float(__ushort_as_half(maskp[p])) : 0.0f;
                        v = chain_score(s[nb][c], A.scale, A.scale_div, mk);
                    }
                    x[nb][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = (m_new == -INFINITY) ? 1.0f : expf(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            uint32_t pa[4];
            {
                float pv[2][4];
#pragma unroll
                for (int nb = 0; nb < 2; nb++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        float mr = m_run[c >> 1];
                        float e = (mr == -INFINITY) ? 0.0f : expf(x[nb][c] - mr);
                        pv[nb][c] = e;
                        l_run[c >> 1] += e;
                    }
                pa[0] = pack_h2(pv[0][0], pv[0][1]);
                pa[1] = pack_h2(pv[0][2], pv[0][3]);
                pa[2] = pack_h2(pv[1][0], pv[1][1]);
                pa[3] = pack_h2(pv[1][2], pv[1][3]);
            }
#pragma unroll
            for (int i = 0; i < DBLK; i++) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
#pragma unroll
            for (int dp = 0; dp < DBLK / 2; dp++) {
                uint32_t vb[4];
                int mat = lane >> 3, r = lane & 7;
                int row = wrow0 + (mat & 1) * 8 + r;
                int ch = dp * 2 + (mat >> 1);
                ldsm_x4_t(vb, sv + row * ROWB + ((ch ^ (row & 7)) << 4));
                mma_f16(o[dp * 2], pa, vb[0], vb[1]);
                mma_f16(o[dp * 2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the four warps (each saw a disjoint quarter of every tile)
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* sm_o = (float*)smem;                       // [NWARP][16][HD]
    float* sm_ml = sm_o + NWARP * 16 * HD;            // [NWARP][16][2]
#pragma unroll
    for (int i = 0; i < DBLK; i++) {
        int d = i * 8 + 2 * t;
        sm_o[(warp * 16 + g) * HD + d] = o[i][0];
        sm_o[(warp * 16 + g) * HD + d + 1] = o[i][1];
        sm_o[(warp * 16 + g + 8) * HD + d] = o[i][2];
        sm_o[(warp * 16 + g + 8) * HD + d + 1] = o[i][3];
    }
    if (t == 0) {
        sm_ml[(warp * 16 + g) * 2] = m_run[0];
        sm_ml[(warp * 16 + g) * 2 + 1] = l_run[0];
        sm_ml[(warp * 16 + g + 8) * 2] = m_run[1];
        sm_ml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    float* po = A.part_o + ((size_t)kvh * A.nsplit + split) * rep * HD;
    float* pml = A.part_ml + ((size_t)kvh * A.nsplit + split) * rep * 2;
    for (uint32_t e = tid; e < rep * HD; e += NWARP * 32) {
        uint32_t r = e / HD, d = e % HD;
        float mt = -INFINITY;
        for (int w = 0; w < NWARP; w++) mt = fmaxf(mt, sm_ml[(w * 16 + r) * 2]);
        float acc = 0.0f, lt = 0.0f;
        for (int w = 0; w < NWARP; w++) {
            float mw = sm_ml[(w * 16 + r) * 2];
            float wgt = (mw == -INFINITY) ? 0.0f : expf(mw - mt);
            acc += sm_o[(w * 16 + r) * HD + d] * wgt;
            lt += sm_ml[(w * 16 + r) * 2 + 1] * wgt;
        }
        po[e] = acc;
        if (d == 0) { pml[r * 2] = mt; pml[r * 2 + 1] = lt; }
    }
}

// out[h][d] = sum_s O_s[d] e^{m_s - m} / sum_s l_s e^{m_s - m}, slices in order.
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         uint16_t* __restrict__ out, uint32_t rep, uint32_t hd, uint32_t nsplit,
                                         uint32_t* bump_counter) {
    const uint32_t h = blockIdx.x;           // query head, = kvh * rep + r
    const uint32_t kvh = h / rep, r = h % rep;
    float mt = -INFINITY;
    for (uint32_t s = 0; s < nsplit; s++) mt = fmaxf(mt, part_ml[(((size_t)kvh * nsplit + s) * rep + r) * 2]);
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f, lt = 0.0f;
        for (uint32_t s = 0; s < nsplit; s++) {
            size_t base = ((size_t)kvh * nsplit + s) * rep + r;
            float ms = part_ml[base * 2];
            float w = (ms == -INFINITY) ? 0.0f : expf(ms - mt);
            acc += part_o[base * hd + d] * w;
            lt += part_ml[base * 2 + 1] * w;
        }
        out[(size_t)h * hd + d] = f2h(lt > 0.0f ? acc / lt : 0.0f);
    }
    // every reader of the counter (the split kernel) has finished: stream order
    if (bump_counter && blockIdx.x == 0 && threadIdx.x == 0) *bump_counter += 1;
}

}  // namespace

uint32_t attn_decode_pick_splits(uint32_t kv_heads_total, uint32_t max_positions) {
    // aim at two CTAs per SM, at least one 64-position tile per slice
    uint32_t want = (2 * 148 + kv_heads_total - 1) / kv_heads_total;
    uint32_t most = (max_positions + TILE - 1) / TILE;
    if (want > most) want = most;
    if (want < 1) want = 1;
    if (want > 64) want = 64;
    return want;
}

size_t attn_decode_scratch_floats(uint32_t kv_heads_total, uint32_t rep, uint32_t hd, uint32_t nsplit) {
    return (size_t)kv_heads_total * nsplit * rep * (hd + 2);
}

bool k_attn_decode(cudaStream_t st, const AttnDecodeArgs& a, uint32_t hd, uint16_t* out, uint32_t kv_heads_total) {
    if (a.rep == 0 || a.rep > 16 || (hd != 128 && hd != 64)) return false;
    dim3 grid(kv_heads_total, a.nsplit);
    size_t smem = (size_t)STAGES * 2 * TILE * hd * 2;
    size_t merge = (size_t)NWARP * 16 * (hd + 2) * sizeof(float);
    if (merge > smem) smem = merge;
    if (hd == 128) {
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(attn_decode_split_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = true; }
        attn_decode_split_kernel<128><<<grid, NWARP * 32, smem, st>>>(a);
    } else {
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(attn_decode_split_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = true; }
        attn_decode_split_kernel<64><<<grid, NWARP * 32, smem, st>>>(a);
    }
    attn_decode_merge_kernel<<<kv_heads_total * a.rep, hd < 128 ? 64 : 128, 0, st>>>(a.part_o, a.part_ml, out, a.rep, hd, a.nsplit, a.bump_counter);
    g_launches += 2;
    return true;
}

}  // namespace gehtp
