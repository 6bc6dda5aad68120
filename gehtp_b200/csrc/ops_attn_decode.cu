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
// multiplied with mma.sync m16n8k16. The context is cut into chunks of 256
// positions; a (KV head, chunk) pair is a work item, items are dealt round-robin
// to 2 CTAs per SM, and a CTA streams the tiles of its items back to back. Each
// item leaves (max, sum, unnormalised output) in a scratch buffer; a second
// small kernel merges the chunks in chunk order.
#include <cstdio>
#include <map>
#include <utility>
#include <vector>
#include <tuple>
#include <cuda.h>
#include <cuda_fp16.h>
#include "common.cuh"
#include "launchers_attn.h"
#include "engine.h"

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
attn_decode_split_kernel(AttnDecodeArgs A, uint32_t kv_heads_total) {
    constexpr int ROWB = HD * 2;          // bytes per K or V row
    constexpr int CHUNKS = ROWB / 16;     // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    constexpr int DBLK = HD / 8;
    constexpr int STAGE_B = 2 * TILE * ROWB;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rep = A.rep;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t n_kv = A.counter ? *A.counter + A.n_kv_add : A.n_kv;
    uint32_t CHUNK_POS = (n_kv + A.nsplit - 1) / A.nsplit;           // even split of the context over nsplit slices
    CHUNK_POS = (CHUNK_POS + TILE - 1) / TILE * TILE;
    const uint32_t n_chunks = (n_kv + CHUNK_POS - 1) / CHUNK_POS;   // <= A.nsplit by construction
    const uint32_t n_items = kv_heads_total * n_chunks;
    const uint32_t kv_elems = A.kv_heads * HD;
    // slices past the last one that holds positions: marked empty (max = -inf, sum = 0) for the merge kernel,
    // which reads all nsplit slices of a head
    for (uint32_t e = blockIdx.x * blockDim.x + tid; e < kv_heads_total * (A.nsplit - n_chunks) * rep; e += gridDim.x * blockDim.x) {
        const uint32_t r = e % rep, sl = n_chunks + (e / rep) % (A.nsplit - n_chunks), kh = e / (rep * (A.nsplit - n_chunks));
        float* pml = A.part_ml + (((size_t)kh * A.nsplit + sl) * rep + r) * 2;
        pml[0] = -INFINITY;
        pml[1] = 0.0f;
    }
    float* sm_o = (float*)(smem + STAGES * STAGE_B);     // [NWARP][rep][HD]
    float* sm_ml = sm_o + NWARP * rep * HD;               // [NWARP][rep][2]

    // A work item = (KV head, chunk of CHUNK_POS positions), heads fastest: CTAs that
    // run side by side read neighbouring heads of the same positions, i.e. one
    // contiguous stretch of the ring, which keeps DRAM pages open. This CTA takes
    // items blockIdx.x, blockIdx.x + gridDim.x, ... and streams their tiles back to
    // back, so the copy pipeline never drains between items.
    struct Cursor { uint32_t item, tile; };
    auto tiles_of = [&](uint32_t item) -> uint32_t {
        uint32_t pb = (item / kv_heads_total) * CHUNK_POS;
        uint32_t pe = pb + CHUNK_POS < n_kv ? pb + CHUNK_POS : n_kv;
        return (pe - pb + TILE - 1) / TILE;
    };
    auto advance = [&](Cursor& c) {
        if (++c.tile >= tiles_of(c.item)) { c.item += gridDim.x; c.tile = 0; }
    };
    auto issue = [&](const Cursor& c, uint32_t stage) {
        if (c.item < n_items) {
            const uint32_t kvh = c.item % kv_heads_total;
            const uint32_t pb = (c.item / kv_heads_total) * CHUNK_POS;
            const uint32_t pe = pb + CHUNK_POS < n_kv ? pb + CHUNK_POS : n_kv;
            const uint32_t p0 = pb + c.tile * TILE;
            unsigned char* sk = smem + (size_t)stage * STAGE_B;
            unsigned char* sv = sk + TILE * ROWB;
            const uint16_t* base = A.ring + (size_t)kvh * HD;
            for (int idx = tid; idx < TILE * CHUNKS; idx += NWARP * 32) {
                int row = idx / CHUNKS, ch = idx % CHUNKS;
                uint32_t p = p0 + row;
                bool ok = p < pe;
                const uint16_t* src = base + (size_t)(ok ? p : 0) * kv_elems * 2 + ch * 8;   // slot = position: no wrap below nslots
                int so = row * ROWB + ((ch ^ (row & 7)) << 4);
                cp_async16(sk + so, src, ok);
                cp_async16(sv + so, src + kv_elems, ok);
            }
        }
        cp_async_commit();
    };

    Cursor ic{blockIdx.x, 0}, cc{blockIdx.x, 0};
    uint32_t si = 0, sc = 0;
    for (int s = 0; s < STAGES - 1; s++) {
        issue(ic, si % STAGES);
        if (ic.item < n_items) advance(ic);
        si++;
    }

    uint32_t qa[KSTEPS][4];
    float o[DBLK][4];
    float m_run[2], l_run[2];
    while (cc.item < n_items) {
        const uint32_t kvh = cc.item % kv_heads_total, chunk = cc.item / kv_heads_total;
        const uint32_t pb = chunk * CHUNK_POS;
        const uint32_t pe = pb + CHUNK_POS < n_kv ? pb + CHUNK_POS : n_kv;
        if (cc.tile == 0) {
            const uint16_t* q0 = A.q + ((size_t)kvh * rep + g) * HD;
            const uint16_t* q1 = A.q + ((size_t)kvh * rep + g + 8) * HD;
#pragma unroll
            for (int j = 0; j < KSTEPS; j++) {
                qa[j][0] = (uint32_t)g < rep ? *(const uint32_t*)(q0 + 16 * j + 2 * t) : 0u;
                qa[j][1] = (uint32_t)(g + 8) < rep ? *(const uint32_t*)(q1 + 16 * j + 2 * t) : 0u;
                qa[j][2] = (uint32_t)g < rep ? *(const uint32_t*)(q0 + 16 * j + 2 * t + 8) : 0u;
                qa[j][3] = (uint32_t)(g + 8) < rep ? *(const uint32_t*)(q1 + 16 * j + 2 * t + 8) : 0u;
            }
#pragma unroll
            for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.0f;
        }
        issue(ic, si % STAGES);
        if (ic.item < n_items) advance(ic);
        si++;
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const unsigned char* sk = smem + (size_t)(sc % STAGES) * STAGE_B;
        const unsigned char* sv = sk + TILE * ROWB;
        const int wrow0 = warp * 16;
        const uint32_t pw0 = pb + cc.tile * TILE + wrow0;
        const uint16_t* maskp = A.mask ? A.mask + (size_t)(kvh / A.kvh_per_seq) * A.mask_seq_stride : nullptr;
        if (pw0 < pe) {
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
            float x[2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t p = pw0 + nb * 8 + 2 * t + (c & 1);
                    float v = -INFINITY;
                    if (p < pe) {
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
                alpha[h] = (m_new == -INFINITY) ? 1.0f : __expf(m_run[h] - m_new);
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
                        float e = (mr == -INFINITY) ? 0.0f : __expf(x[nb][c] - mr);
                        pv[nb][c] = e;
                        l_run[c >> 1] += e;
                    }
                pa[0] = pack_h2(pv[0][0], pv[0][1]);
                pa[1] = pack_h2(pv[0][2], pv[0][3]);
                pa[2] = pack_h2(pv[1][0], pv[1][1]);
                pa[3] = pack_h2(pv[1][2], pv[1][3]);
            }
            if (alpha[0] != 1.0f || alpha[1] != 1.0f) {
#pragma unroll
                for (int i = 0; i < DBLK; i++) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
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
        sc++;
        const bool last = cc.tile + 1 >= tiles_of(cc.item);
        if (last) {
            // merge the four warps (disjoint quarters of every tile) and store the item's partial result
#pragma unroll
            for (int h = 0; h < 2; h++) {
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            }
#pragma unroll
            for (int i = 0; i < DBLK; i++) {
                int d = i * 8 + 2 * t;
                if ((uint32_t)g < rep) { sm_o[(warp * rep + g) * HD + d] = o[i][0]; sm_o[(warp * rep + g) * HD + d + 1] = o[i][1]; }
                if ((uint32_t)(g + 8) < rep) { sm_o[(warp * rep + g + 8) * HD + d] = o[i][2]; sm_o[(warp * rep + g + 8) * HD + d + 1] = o[i][3]; }
            }
            if (t == 0) {
                if ((uint32_t)g < rep) { sm_ml[(warp * rep + g) * 2] = m_run[0]; sm_ml[(warp * rep + g) * 2 + 1] = l_run[0]; }
                if ((uint32_t)(g + 8) < rep) { sm_ml[(warp * rep + g + 8) * 2] = m_run[1]; sm_ml[(warp * rep + g + 8) * 2 + 1] = l_run[1]; }
            }
        }
        __syncthreads();   // stage (sc-1) is free for the next copy; merge buffers are complete
        if (last) {
            float* po = A.part_o + ((size_t)kvh * A.nsplit + chunk) * rep * HD;
            float* pml = A.part_ml + ((size_t)kvh * A.nsplit + chunk) * rep * 2;
            for (uint32_t e = tid; e < rep * HD; e += NWARP * 32) {
                uint32_t r = e / HD, d = e % HD;
                float mt = -INFINITY;
                for (int w = 0; w < NWARP; w++) mt = fmaxf(mt, sm_ml[(w * rep + r) * 2]);
                float acc = 0.0f, lt = 0.0f;
                for (int w = 0; w < NWARP; w++) {
                    float mw = sm_ml[(w * rep + r) * 2];
                    float wgt = (mw == -INFINITY) ? 0.0f : __expf(mw - mt);
                    acc += sm_o[(w * rep + r) * HD + d] * wgt;
                    lt += sm_ml[(w * rep + r) * 2 + 1] * wgt;
                }
                po[e] = acc;
                if (d == 0) { pml[r * 2] = mt; pml[r * 2 + 1] = lt; }
            }
        }
        advance(cc);
    }
    cp_async_wait<0>();
}

// Grouped form: one CTA = NW neighbouring KV heads (one per warp) x one chunk of
// positions. A ring row of NW heads is NW*HD*2 contiguous bytes, so the CTA's
// copies are 1 KB (NW = 4) stretches instead of 256-byte ones, and each warp
// owns a whole (head, chunk) result: no cross-warp merge, the partial goes from
// registers to the scratch buffer.
template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32)
attn_decode_group_kernel(AttnDecodeArgs A, uint32_t kv_heads_total) {
    constexpr int ROWB = HD * 2;
    constexpr int CHUNKS = ROWB / 16;
    constexpr int KSTEPS = HD / 16;
    constexpr int DBLK = HD / 8;
    constexpr int TP = 16;                               // positions per tile
    constexpr int HEAD_B = TP * ROWB;                    // one head's K (or V) rows of a tile
    constexpr int STAGE_B = 2 * NW * HEAD_B;
    constexpr int GSTAGES = 3;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rep = A.rep;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t n_kv = A.counter ? *A.counter + A.n_kv_add : A.n_kv;
    const uint32_t n_groups = kv_heads_total / NW;
    const uint32_t grp = blockIdx.x % n_groups, split = blockIdx.x / n_groups;   // groups fastest: neighbours share ring rows
    uint32_t per = (n_kv + A.nsplit - 1) / A.nsplit;
    per = (per + TP - 1) / TP * TP;
    const uint32_t pb = split * per;
    const uint32_t pe = pb + per < n_kv ? pb + per : n_kv;
    const uint32_t kv_elems = A.kv_heads * HD;
    const uint32_t kvh = grp * NW + warp;
    const int ntiles = pe > pb ? (int)((pe - pb + TP - 1) / TP) : 0;

    auto issue = [&](int tile) {
        if (tile < ntiles) {
            const uint32_t p0 = pb + tile * TP;
            unsigned char* sk = smem + (size_t)(tile % GSTAGES) * STAGE_B;
            unsigned char* sv = sk + NW * HEAD_B;
            const uint16_t* base = A.ring + (size_t)grp * NW * HD;
            for (int idx = tid; idx < TP * NW * CHUNKS; idx += NW * 32) {
                int row = idx / (NW * CHUNKS), c2 = idx % (NW * CHUNKS);
                int head = c2 / CHUNKS, ch = c2 % CHUNKS;
                uint32_t p = p0 + row;
                bool ok = p < pe;
                const uint16_t* src = base + (size_t)(ok ? p : 0) * kv_elems * 2 + c2 * 8;
                int so = head * HEAD_B + row * ROWB + ((ch ^ (row & 7)) << 4);
                cp_async16(sk + so, src, ok);
                cp_async16(sv + so, src + kv_elems, ok);
            }
        }
        cp_async_commit();
    };
    for (int s2 = 0; s2 < GSTAGES - 1; s2++) issue(s2);

    uint32_t qa[KSTEPS][4];
    float o[DBLK][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
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
#pragma unroll
        for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    }
    const uint16_t* maskp = A.mask ? A.mask + (size_t)(kvh / A.kvh_per_seq) * A.mask_seq_stride : nullptr;
    for (int tile = 0; tile < ntiles; tile++) {
        issue(tile + GSTAGES - 1);
        cp_async_wait<GSTAGES - 1>();
        __syncthreads();
        const unsigned char* sk = smem + (size_t)(tile % GSTAGES) * STAGE_B + warp * HEAD_B;
        const unsigned char* sv = sk + NW * HEAD_B;
        const uint32_t pw0 = pb + tile * TP;
        {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int j = 0; j < KSTEPS; j++) {
                uint32_t kb[4];
                int mat = lane >> 3, r = lane & 7;
                int row = (mat >> 1) * 8 + r;
                int ch = j * 2 + (mat & 1);
                ldsm_x4(kb, sk + row * ROWB + ((ch ^ (row & 7)) << 4));
                mma_f16(s[0], qa[j], kb[0], kb[1]);
                mma_f16(s[1], qa[j], kb[2], kb[3]);
            }
            float x[2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t p = pw0 + nb * 8 + 2 * t + (c & 1);
                    float v = -INFINITY;
                    if (p < pe) {
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
                alpha[h] = (m_new == -INFINITY) ? 1.0f : __expf(m_run[h] - m_new);
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
                        float e = (mr == -INFINITY) ? 0.0f : __expf(x[nb][c] - mr);
                        pv[nb][c] = e;
                        l_run[c >> 1] += e;
                    }
                pa[0] = pack_h2(pv[0][0], pv[0][1]);
                pa[1] = pack_h2(pv[0][2], pv[0][3]);
                pa[2] = pack_h2(pv[1][0], pv[1][1]);
                pa[3] = pack_h2(pv[1][2], pv[1][3]);
            }
            if (alpha[0] != 1.0f || alpha[1] != 1.0f) {
#pragma unroll
                for (int i = 0; i < DBLK; i++) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int dp = 0; dp < DBLK / 2; dp++) {
                uint32_t vb[4];
                int mat = lane >> 3, r = lane & 7;
                int row = (mat & 1) * 8 + r;
                int ch = dp * 2 + (mat >> 1);
                ldsm_x4_t(vb, sv + row * ROWB + ((ch ^ (row & 7)) << 4));
                mma_f16(o[dp * 2], pa, vb[0], vb[1]);
                mma_f16(o[dp * 2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();   // every warp is done with this stage
    }
    cp_async_wait<0>();
    // this warp's (head, split) partial, straight from registers (empty slices leave max = -inf, sum = 0)
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* po = A.part_o + ((size_t)kvh * A.nsplit + split) * rep * HD;
    float* pml = A.part_ml + ((size_t)kvh * A.nsplit + split) * rep * 2;
#pragma unroll
    for (int i = 0; i < DBLK; i++) {
        int d = i * 8 + 2 * t;
        if ((uint32_t)g < rep) *(float2*)(po + (size_t)g * HD + d) = make_float2(o[i][0], o[i][1]);
        if ((uint32_t)(g + 8) < rep) *(float2*)(po + (size_t)(g + 8) * HD + d) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
        if ((uint32_t)g < rep) { pml[g * 2] = m_run[0]; pml[g * 2 + 1] = l_run[0]; }
        if ((uint32_t)(g + 8) < rep) { pml[(g + 8) * 2] = m_run[1]; pml[(g + 8) * 2 + 1] = l_run[1]; }
    }
}

// ---------------------------------------------------------------- TMA-fed grouped form
// Same work split as the grouped kernel above (one CTA = 4 neighbouring KV heads
// x one even slice of the context, one head per consumer warp), but the K/V
// tiles are brought in by a fifth warp with tiled bulk copies (TMA): the ring
// is described as a 2-D tensor [slot][K face | V face], a tile of 16 positions
// is 16 boxes of 64 elements x 16 rows with the 128-byte swizzle, which is the
// XOR pattern ldmatrix wants. The consumers issue no copy instructions and meet
// the producer only on mbarriers (no CTA-wide barrier in the loop). Tiles that
// cannot hold the row the preceding kernel appends are requested before the
// dependency wait. Waits are bounded; a timeout raises the engine status word.
constexpr int TMA_TP = 16;                    // positions per tile
constexpr int TMA_BOX_B = TMA_TP * 128;       // one box: 16 rows x 64 fp16
constexpr int TMA_NW = 4;
constexpr int TMA_STAGE_B = 2 * TMA_NW * 2 * TMA_BOX_B;   // K,V x heads x halves = 32 KB
constexpr int TMA_STAGES = 3;
constexpr uint32_t TMA_SPIN = 4u * 1000u * 1000u;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < TMA_SPIN; it++) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void ldsm_x4_s(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t_s(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

__global__ void __launch_bounds__((TMA_NW + 1) * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, AttnDecodeArgs A, uint32_t kv_heads_total) {
    constexpr int HD = 128, DBLK = HD / 8, KSTEPS = HD / 16, NW = TMA_NW, TP = TMA_TP;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + TMA_STAGES * TMA_STAGE_B);     // full[STAGES], empty[STAGES]
    const uint32_t full0 = s_u32(bars), empty0 = s_u32(bars + TMA_STAGES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rep = A.rep;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int s = 0; s < TMA_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full0 + 8 * s), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * s), "r"(NW));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The position counter of this state is advanced by the merge kernel of the
    // previous step, not by the kernel right before this one: it may be read now.
    const uint32_t n_kv = A.counter ? *A.counter + A.n_kv_add : A.n_kv;
    const uint32_t n_groups = kv_heads_total / NW;
    const uint32_t grp = blockIdx.x % n_groups, split = blockIdx.x / n_groups;   // groups fastest: neighbours share ring rows
    uint32_t per = (n_kv + A.nsplit - 1) / A.nsplit;
    per = (per + TP - 1) / TP * TP;
    const uint32_t pb = split * per;
    const uint32_t pe = pb + per < n_kv ? pb + per : n_kv;
    const uint32_t kv_elems = A.kv_heads * HD;
    const int ntiles = pe > pb ? (int)((pe - pb + TP - 1) / TP) : 0;

    if (warp == NW) {
        // ---- producer
        if (lane == 0) {
            bool waited = false;
            int tile = 0;
            for (; tile < ntiles; tile++) {
                const uint32_t p0 = pb + tile * TP;
                // the row appended by the preceding kernel is position n_kv - 1
                if (!waited && p0 + TP >= n_kv) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
                const int s = tile % TMA_STAGES;
                if (!mbar_wait_bounded(empty0 + 8 * s, ((tile / TMA_STAGES) & 1) ^ 1)) { raise_status(A.status, kStatusAttnTimeout); break; }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * s), "r"(TMA_STAGE_B) : "memory");
                const uint32_t dst = s_u32(smem + (size_t)s * TMA_STAGE_B);
#pragma unroll
                for (int b = 0; b < 2 * NW * 2; b++) {      // b = (kv * NW + head) * 2 + half
                    const int kv = b / (NW * 2), head = (b >> 1) % NW, half = b & 1;
                    const int x = (int)(kv * kv_elems + (grp * NW + head) * HD + half * 64);
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst + b * TMA_BOX_B), "l"(&tmap), "r"(full0 + 8 * s), "r"(x), "r"((int)p0) : "memory");
                }
            }
            // requested copies must have landed before the CTA may go away
            for (int j = tile > TMA_STAGES ? tile - TMA_STAGES : 0; j < tile; j++)
                mbar_wait_bounded(full0 + 8 * (j % TMA_STAGES), (j / TMA_STAGES) & 1);
            if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
        }
        return;
    }

    // ---- consumers: warp = KV head of the group
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t kvh = grp * NW + warp;
    uint32_t qa[KSTEPS][4];
    float o[DBLK][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
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
#pragma unroll
        for (int i = 0; i < DBLK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    }
    const uint16_t* maskp = A.mask ? A.mask + (size_t)(kvh / A.kvh_per_seq) * A.mask_seq_stride : nullptr;
    // per-lane ldmatrix offsets inside a box (row stride 128 B, chunk XOR row & 7)
    const int mat = lane >> 3, r8 = lane & 7;
    const int krow = (mat >> 1) * 8 + r8, vrow = (mat & 1) * 8 + r8;
    const uint32_t smem0 = s_u32(smem);
    for (int tile = 0; tile < ntiles; tile++) {
        const int s = tile % TMA_STAGES;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + 8 * s, (tile / TMA_STAGES) & 1))) {
            raise_status(A.status, kStatusAttnTimeout);
            break;
        }
        const uint32_t sk = smem0 + s * TMA_STAGE_B + (warp * 2) * TMA_BOX_B;            // K boxes of this head
        const uint32_t sv = smem0 + s * TMA_STAGE_B + ((NW + warp) * 2) * TMA_BOX_B;     // V boxes
        const uint32_t pw0 = pb + tile * TP;
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int j = 0; j < KSTEPS; j++) {
            uint32_t kb[4];
            const int ch = (j & 3) * 2 + (mat & 1);
            ldsm_x4_s(kb, sk + (j >> 2) * TMA_BOX_B + krow * 128 + ((ch ^ (krow & 7)) << 4));
            mma_f16(sc[0], qa[j], kb[0], kb[1]);
            mma_f16(sc[1], qa[j], kb[2], kb[3]);
        }
        float x[2][4];
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t p = pw0 + nb * 8 + 2 * t + (c & 1);
                float v = -INFINITY;
                if (p < pe) {
                    float mk = maskp ? __half2float(__ushort_as_half(maskp[p])) : 0.0f;
                    v = chain_score(sc[nb][c], A.scale, A.scale_div, mk);
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
            alpha[h] = (m_new == -INFINITY) ? 1.0f : __expf(m_run[h] - m_new);
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
                    float e = (mr == -INFINITY) ? 0.0f : __expf(x[nb][c] - mr);
                    pv[nb][c] = e;
                    l_run[c >> 1] += e;
                }
            pa[0] = pack_h2(pv[0][0], pv[0][1]);
            pa[1] = pack_h2(pv[0][2], pv[0][3]);
            pa[2] = pack_h2(pv[1][0], pv[1][1]);
            pa[3] = pack_h2(pv[1][2], pv[1][3]);
        }
        if (alpha[0] != 1.0f || alpha[1] != 1.0f) {
#pragma unroll
            for (int i = 0; i < DBLK; i++) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int dp = 0; dp < DBLK / 2; dp++) {
            uint32_t vb[4];
            const int ch = (dp & 3) * 2 + (mat >> 1);
            ldsm_x4_t_s(vb, sv + (dp >> 2) * TMA_BOX_B + vrow * 128 + ((ch ^ (vrow & 7)) << 4));
            mma_f16(o[dp * 2], pa, vb[0], vb[1]);
            mma_f16(o[dp * 2 + 1], pa, vb[2], vb[3]);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * s) : "memory");
    }
    // this warp's (head, split) partial, straight from registers (empty slices leave max = -inf, sum = 0)
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* po = A.part_o + ((size_t)kvh * A.nsplit + split) * rep * HD;
    float* pml = A.part_ml + ((size_t)kvh * A.nsplit + split) * rep * 2;
#pragma unroll
    for (int i = 0; i < DBLK; i++) {
        int d = i * 8 + 2 * t;
        if ((uint32_t)g < rep) *(float2*)(po + (size_t)g * HD + d) = make_float2(o[i][0], o[i][1]);
        if ((uint32_t)(g + 8) < rep) *(float2*)(po + (size_t)(g + 8) * HD + d) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
        if ((uint32_t)g < rep) { pml[g * 2] = m_run[0]; pml[g * 2 + 1] = l_run[0]; }
        if ((uint32_t)(g + 8) < rep) { pml[(g + 8) * 2] = m_run[1]; pml[(g + 8) * 2 + 1] = l_run[1]; }
    }
}

// out[h][d] = sum_s O_s[d] e^{m_s - m} / sum_s l_s e^{m_s - m}.
// One CTA of 16 warps per query head. Warp w folds the slices w, w+16, ... (eight at a time, all their loads in
// flight together) into a running (max, sum, vector) of its own; the 16 warp results are then combined in warp
// order. Every slice of the scratch buffers is written by the split-KV kernel (an empty one as max = -inf,
// sum = 0), so nothing here depends on the position counter and the first loads leave right after the wait.
// MERGE_WARPS warps share the slices of one query head (8 slices in flight per warp and pass); their partial
// results meet in shared memory. Few slices want few warps: the closing combination walks all of them.
template <int MERGE_WARPS>
__global__ void __launch_bounds__(MERGE_WARPS * 32)
attn_decode_merge_kernel(const float* part_o, const float* part_ml, uint16_t* out, uint32_t rep, uint32_t hd,
                         uint32_t nsplit, uint32_t* bump_counter) {
    __shared__ float s_acc[MERGE_WARPS][128];
    __shared__ float s_l[MERGE_WARPS];
    __shared__ float s_m[MERGE_WARPS];
    const uint32_t h = blockIdx.x;           // query head, = kvh * rep + r
    const uint32_t kvh = h / rep, r = h % rep;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The kernels behind this one start their weight loads as soon as they are allowed on an SM. They are
    // released only once the split-KV kernel has finished. Released at entry (measured on B200, batch 8,
    // context 8192), they came up beside that kernel's last CTAs, and with their loads in flight the P.V
    // sums of single (KV head, slice) pairs came out off by about one tile of V in some runs (maxima and
    // exp sums unchanged): results differed from run to run by ~1 % in a few heads. With the release
    // placed here, 24 of 24 repeated steps were bit-identical.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t row0 = ((size_t)kvh * nsplit) * rep + r;     // slice s is at row0 + s*rep
    const uint32_t per_lane = hd / 32;       // 4 for head_dim 128, 2 for 64
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float m_run = -INFINITY, l_run = 0.0f;
    for (uint32_t s0 = warp; s0 < nsplit; s0 += MERGE_WARPS * 8) {
        float ms[8], ls[8], ov[8][4];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint32_t s = s0 + MERGE_WARPS * u;
            const bool ok = s < nsplit;
            const size_t base = row0 + (size_t)(ok ? s : s0) * rep;
            ms[u] = ok ? __ldcg(part_ml + base * 2) : -INFINITY;
            ls[u] = ok ? __ldcg(part_ml + base * 2 + 1) : 0.0f;
            const float* po = part_o + base * hd + lane * per_lane;
            if (per_lane == 4) {
                float4 v = __ldcg((const float4*)po);
                ov[u][0] = v.x; ov[u][1] = v.y; ov[u][2] = v.z; ov[u][3] = v.w;
            } else {
                float2 v = __ldcg((const float2*)po);
                ov[u][0] = v.x; ov[u][1] = v.y; ov[u][2] = 0.0f; ov[u][3] = 0.0f;
            }
        }
        float m_new = m_run;
#pragma unroll
        for (int u = 0; u < 8; u++) m_new = fmaxf(m_new, ms[u]);
        if (m_new == -INFINITY) continue;                      // nothing but empty slices so far
        const float keep = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_new);
        l_run *= keep;
#pragma unroll
        for (int k = 0; k < 4; k++) acc[k] *= keep;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (ms[u] == -INFINITY) continue;                   // empty slice: its vector may be stale memory
            const float w = __expf(ms[u] - m_new);
            l_run += ls[u] * w;
#pragma unroll
            for (int k = 0; k < 4; k++) acc[k] += ov[u][k] * w;
        }
        m_run = m_new;
    }
    for (uint32_t k = 0; k < per_lane; k++) s_acc[warp][lane * per_lane + k] = acc[k];
    if (lane == 0) { s_l[warp] = l_run; s_m[warp] = m_run; }
    __syncthreads();
    if (threadIdx.x < hd) {
        const uint32_t d = threadIdx.x;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < MERGE_WARPS; w++) mt = fmaxf(mt, s_m[w]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < MERGE_WARPS; w++) {
            const float f = (s_m[w] == -INFINITY) ? 0.0f : __expf(s_m[w] - mt);
            num += s_acc[w][d] * f;
            den += s_l[w] * f;
        }
        out[(size_t)h * hd + d] = f2h(den > 0.0f ? num / den : 0.0f);
    }
    // all readers of the counter in this launch must be done before it moves: the
    // last block to finish advances it
    if (bump_counter) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            unsigned int done = atomicAdd(bump_counter + 64, 1u) + 1;   // arrival count kept beside the counters
            if (done == gridDim.x) { bump_counter[64] = 0; *bump_counter += 1; }
        }
    }
}

}  // namespace

// Context slices per KV head: as many as give every one of the 2 x 148 CTAs one
// evenly sized work item (a group of 4 neighbouring heads x a slice when the
// head count is a multiple of 4, else one head x a slice), at least 64
// positions per slice, and, when max_floats != 0, few enough for the scratch
// buffers to fit in that many floats. 0 = does not fit even unsliced.
uint32_t attn_decode_nsplit(uint32_t kv_heads_total, uint32_t max_positions, uint32_t rep, uint32_t hd, size_t max_floats) {
    const uint32_t group = (kv_heads_total % 4 == 0 && hd == 128) ? 4 : 1;
    const uint32_t n_groups = kv_heads_total / group;
    uint32_t ns = (2 * 148) / n_groups;
    if (ns < 1) ns = 1;
    uint32_t most = (max_positions + 63) / 64;
    if (ns > most) ns = most;
    if (ns < 1) ns = 1;
    while (max_floats && ns > 1 && attn_decode_scratch_floats(kv_heads_total, rep, hd, ns) > max_floats) ns--;
    if (max_floats && attn_decode_scratch_floats(kv_heads_total, rep, hd, ns) > max_floats) return 0;
    return ns;
}

size_t attn_decode_scratch_floats(uint32_t kv_heads_total, uint32_t rep, uint32_t hd, uint32_t nsplit) {
    return (size_t)kv_heads_total * nsplit * rep * (hd + 2);
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn attn_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Tensor map of a KV ring: [nslots][K face | V face] fp16, boxes of 64 elements x 16 slots, 128-byte swizzle.
const CUtensorMap* ring_tensor_map(const uint16_t* ring, uint32_t nslots, uint32_t kv_elems, bool no_cache) {
    static std::map<std::tuple<const void*, uint32_t, uint32_t>, CUtensorMap> cache;
    static thread_local CUtensorMap tm;
    auto key = std::make_tuple((const void*)ring, nslots, kv_elems);
    if (!no_cache) {
        auto it = cache.find(key);
        if (it != cache.end()) return &it->second;
    }
    EncodeTiledFn enc = attn_encode_fn();
    if (!enc || ((uintptr_t)ring & 15) || (kv_elems % 64) || !nslots) return nullptr;
    cuuint64_t dims[2] = {(cuuint64_t)2 * kv_elems, nslots};
    cuuint64_t strides[1] = {(cuuint64_t)2 * kv_elems * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TMA_TP};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)ring, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    if (no_cache) return &tm;
    if (cache.size() > 4096) cache.clear();
    return &(cache[key] = tm);
}
}  // namespace

namespace {
bool g_attn_prof = false;
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_attn_prof_events;
}  // namespace

void attn_prof_begin() {
    g_attn_prof_events.clear();
    g_attn_prof = true;
}

void attn_prof_end(float* total_ms, uint32_t* launches) {
    g_attn_prof = false;
    float tot = 0.0f;
    uint32_t n = 0;
    for (auto& e : g_attn_prof_events) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, e.first, e.second) == cudaSuccess) { tot += ms; n++; }
        cudaEventDestroy(e.first);
        cudaEventDestroy(e.second);
    }
    cudaGetLastError();
    g_attn_prof_events.clear();
    if (total_ms) *total_ms = tot;
    if (launches) *launches = n;
}

bool k_attn_decode(cudaStream_t st, const AttnDecodeArgs& a, uint32_t hd, uint16_t* out, uint32_t kv_heads_total) {
    if (a.rep == 0 || a.rep > 16 || (hd != 128 && hd != 64)) return false;
    if (!a.nsplit) return false;
    // the opt-in to large dynamic shared memory is per device: one record per device ordinal
    static int have_tma[64] = {}, have_group[64] = {}, have_s128[64] = {}, have_s64[64] = {};
    bool ok = true;
    if (hd == 128 && kv_heads_total % 4 == 0) {
        const CUtensorMap* tm = ring_tensor_map(a.ring, a.nslots, a.kv_heads * hd, a.no_cache != 0);
        const size_t tsmem = 1024 + (size_t)TMA_STAGES * TMA_STAGE_B + 2 * TMA_STAGES * sizeof(uint64_t);
        if (tm && ensure_dyn_smem(attn_decode_tma_kernel, tsmem, have_tma)) {
            cudaEvent_t pe0 = nullptr, pe1 = nullptr;
            if (g_attn_prof) { cudaEventCreate(&pe0); cudaEventCreate(&pe1); cudaEventRecord(pe0, st); }
            ok = launch_pdl(attn_decode_tma_kernel, dim3((kv_heads_total / 4) * a.nsplit), dim3((TMA_NW + 1) * 32), tsmem, st, *tm, a, kv_heads_total) == cudaSuccess;
            if (g_attn_prof) { cudaEventRecord(pe1, st); g_attn_prof_events.emplace_back(pe0, pe1); }
        } else {
            const size_t gsmem = (size_t)3 * 2 * 4 * 16 * hd * 2;
            if (!ensure_dyn_smem(attn_decode_group_kernel<128, 4>, gsmem, have_group)) return false;
            ok = launch_pdl(attn_decode_group_kernel<128, 4>, dim3((kv_heads_total / 4) * a.nsplit), dim3(128), gsmem, st, a, kv_heads_total) == cudaSuccess;
        }
    } else {
        const size_t smem = (size_t)STAGES * 2 * TILE * hd * 2 + (size_t)NWARP * a.rep * (hd + 2) * sizeof(float);
        const uint32_t items = kv_heads_total * a.nsplit;
        const uint32_t grid = items < 2 * 148 ? items : 2 * 148;
        if (hd == 128) {
            if (!ensure_dyn_smem(attn_decode_split_kernel<128>, smem, have_s128)) return false;
            ok = launch_pdl(attn_decode_split_kernel<128>, dim3(grid), dim3(NWARP * 32), smem, st, a, kv_heads_total) == cudaSuccess;
        } else {
            if (!ensure_dyn_smem(attn_decode_split_kernel<64>, smem, have_s64)) return false;
            ok = launch_pdl(attn_decode_split_kernel<64>, dim3(grid), dim3(NWARP * 32), smem, st, a, kv_heads_total) == cudaSuccess;
        }
    }
    if (!ok) { cudaGetLastError(); return false; }
    {
        static const int forced = [] { const char* e = std::getenv("GEHTP_CUDA_MERGE_WARPS"); return e ? std::atoi(e) : 0; }();
        const int mw = forced ? forced : (a.nsplit <= 32 ? 4 : a.nsplit <= 64 ? 8 : 16);
        const dim3 grid(kv_heads_total * a.rep);
        const float *po = (const float*)a.part_o, *pml = (const float*)a.part_ml;
        cudaError_t ce;
        if (mw <= 4) ce = launch_pdl(attn_decode_merge_kernel<4>, grid, dim3(128), 0, st, po, pml, out, a.rep, hd, a.nsplit, a.bump_counter);
        else if (mw <= 8) ce = launch_pdl(attn_decode_merge_kernel<8>, grid, dim3(256), 0, st, po, pml, out, a.rep, hd, a.nsplit, a.bump_counter);
        else ce = launch_pdl(attn_decode_merge_kernel<16>, grid, dim3(512), 0, st, po, pml, out, a.rep, hd, a.nsplit, a.bump_counter);
        ok = ce == cudaSuccess;
    }
    if (!ok) { cudaGetLastError(); return false; }
    g_launches += 2;
    return true;
}

}  // namespace gehtp

namespace gehtp {
// ---------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a
// serving loop whose memory was carved up front by a pool allocator, inside a
// real-time thread where an allocation could block on the driver's lock, or in
// a process whose device-memory budget is fixed by its operator. The split-KV
// attention kernel needs a scratch buffer for the per-chunk partial results;
// here that scratch is a fixed array that lives in the library's device image,
// so the call needs nothing beyond the caller's own input and output buffers.
//
// The array is GEHTP_NOALLOC_SCRATCH_BYTES large on every GPU that loads the
// library, for the life of the process. Every call uses the same array: two
// calls that overlap on the GPU (different streams, or different host threads)
// race on it and must be serialised by the caller. Nothing in it has to start
// at zero: each call writes every partial it later reads.
constexpr size_t kNoAllocFloats = GEHTP_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];
// Status word of the calls below: the kernel's bounded waits report here (kStatusAttnTimeout),
// read and cleared by gehtp_attn_decode_noalloc_status.
static __device__ unsigned int g_noalloc_status;

}  // namespace gehtp

extern "C" int gehtp_attn_decode_noalloc(const uint16_t* q_dev, const uint16_t* ring_dev, const uint16_t* mask_dev,
                                         uint16_t* out_dev, uint32_t n_heads, uint32_t kv_heads, uint32_t head_dim,
                                         uint32_t n_kv, uint32_t nslots, float scale, void* stream) {
    using namespace gehtp;
    auto fail = [](const char* m) { g.last_error = m; return -1; };
    if (!q_dev || !ring_dev || !out_dev) return fail("attn noalloc: null pointer");
    if (!n_heads || !kv_heads || n_heads % kv_heads || !nslots || !n_kv || n_kv > nslots) return fail("attn noalloc: bad shape");
    const uint32_t rep = n_heads / kv_heads;
    if (rep > 16 || (head_dim != 128 && head_dim != 64)) return fail("attn noalloc: head layout not handled by the fused kernel");
    const uint32_t nsplit = attn_decode_nsplit(kv_heads, n_kv, rep, head_dim, kNoAllocFloats);
    const size_t need = attn_decode_scratch_floats(kv_heads, rep, head_dim, nsplit ? nsplit : 1);
    if (!nsplit) {
        char m[160];
        std::snprintf(m, sizeof m, "attn noalloc: needs %zu bytes of scratch, the built-in array holds %zu", need * sizeof(float),
                      (size_t)GEHTP_NOALLOC_SCRATCH_BYTES);
        return fail(m);
    }
    // The array's name is only a host-side handle; the kernel needs its device
    // address, looked up once per device with that device current.
    static float* scratch_of_device[64] = {};
    static unsigned int* status_of_device[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail("attn noalloc: no current CUDA device");
    if (!scratch_of_device[dev]) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) { cudaGetLastError(); return fail("attn noalloc: cudaGetSymbolAddress failed"); }
        unsigned int* sp = nullptr;
        e = cudaGetSymbolAddress((void**)&sp, g_noalloc_status);
        if (e != cudaSuccess || !sp) { cudaGetLastError(); return fail("attn noalloc: cudaGetSymbolAddress failed"); }
        scratch_of_device[dev] = p;
        status_of_device[dev] = sp;
    }
    AttnDecodeArgs a{};
    a.q = q_dev; a.ring = ring_dev; a.counter = nullptr; a.n_kv = n_kv; a.n_kv_add = 0; a.bump_counter = nullptr;
    a.mask = mask_dev; a.mask_seq_stride = 0; a.kvh_per_seq = kv_heads;
    a.scale = scale; a.scale_div = 0; a.rep = rep; a.kv_heads = kv_heads; a.nslots = nslots; a.nsplit = nsplit;
    a.part_o = scratch_of_device[dev];
    a.part_ml = a.part_o + (size_t)kv_heads * nsplit * rep * head_dim;
    a.no_cache = 1;
    a.status = status_of_device[dev];
    if (!k_attn_decode((cudaStream_t)stream, a, head_dim, out_dev, kv_heads)) return fail("attn noalloc: launch refused");
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    return 0;
}

// 0 when no bounded wait of the allocation-free calls on the current device has run out since the last
// query, else the code it left (and the word is cleared). Copies one word from the device without
// allocating; call it after the stream the calls were queued on has been synchronised.
extern "C" int gehtp_attn_decode_noalloc_status(void) {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, gehtp::g_noalloc_status, sizeof v) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (v) {
        const unsigned int zero = 0;
        cudaMemcpyToSymbol(gehtp::g_noalloc_status, &zero, sizeof zero);
        gehtp::g.last_error = "attn noalloc: a K/V tile copy never arrived (bounded wait ran out); the output is incomplete";
    }
    return (int)(v & 0x7fffffffu);
}
