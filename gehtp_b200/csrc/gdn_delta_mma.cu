// Chunked gated delta rule on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
//
// Same mathematics as delta_chunk_kernel of ops_gdn.cu (reference: delta_chunk_f16 / solve_tri_f16,
// kernels/src/hvx/gdn_kern.c:54-167; formulas in kernels/include/gdn_sm.h:5-12): L and T = (I + L)^-1
// are fp16 matrices, y is rounded once. Entries of T outside the 16 x 16 diagonal blocks see one fp16
// rounding where the reference's substitution rounds along the way (differences of an fp16 step in T).
// What changes is who does the contractions. Per head and chunk of c <= 64 tokens there are seven
// small dependent matrix products (64 x 64 x D, 64 x D x D, 64 x D x 64, D x D x 64); as scalar
// fp32 loops they took 170 us per chunk on a B200 (2048 tokens: 32 chunks in sequence, 5.4 ms).
// Here every product is a handful of m16n8k16 tiles per warp, operands staged in shared memory
// as fp16:
//   * k, q (and k transposed) are fp16 by definition: exact operands;
//   * fp32 quantities that enter a product (the state S, b, u, the decayed q.k matrix) are split
//     into hi = f16(x) and lo = f16(x - hi) and multiplied as hi + lo (two or three MMAs), which
//     carries about 22 bits of mantissa: fp32-class, the state does not degrade over the chunks;
//   * T = (I + L)^-1: the reference's row-by-row forward substitution inside 16 x 16 diagonal blocks (column j
//     depends on column j only: one lane owns a column, its entries in registers, no block-wide barrier), block
//     forward substitution on the tensor cores below the diagonal.
// The products are far too small for tcgen05 tiles (M = 64 or 32 rows, each result feeds the next
// product through registers and a rounding); the chain is latency bound, and mma.sync keeps every
// intermediate in registers on its way to the next operand.
//
// Grid (H, D / 16): the value dimension m is split into slices of 16 rows, one CTA each (b, u, y and the rows
// of S are independent across m); L, T and the q.k matrix are recomputed by each of them.
#include "common.cuh"
#include "launchers.h"
#include "w4_stream.cuh"

namespace gehtp {

namespace {

constexpr int C = 64;          // chunk rows (shorter chunks are padded with zero rows)
constexpr int CP = C + 8;      // row stride (halves) of [..][C] operands: rows fall on different banks


// acc += A[16 x K] . Bt[8 x K]^T ; A, Bt row-major fp16 in shared memory with K contiguous
__device__ __forceinline__ void mma_rows(float (&acc)[4], const uint16_t* A, int lda, const uint16_t* Bt, int ldb, int K, int g, int t) {
    const uint16_t* a_lo = A + g * lda + 2 * t;
    const uint16_t* a_hi = A + (g + 8) * lda + 2 * t;
    const uint16_t* b = Bt + g * ldb + 2 * t;
#pragma unroll 4
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[4];
        a[0] = *(const uint32_t*)(a_lo + k0);
        a[1] = *(const uint32_t*)(a_hi + k0);
        a[2] = *(const uint32_t*)(a_lo + k0 + 8);
        a[3] = *(const uint32_t*)(a_hi + k0 + 8);
        mma16816(acc, a, *(const uint32_t*)(b + k0), *(const uint32_t*)(b + k0 + 8));
    }
}

__device__ __forceinline__ void split_store(uint16_t* hi, uint16_t* lo, float x) {
    const uint16_t h = f2h(x);
    *hi = h;
    *lo = f2h(x - h2f(h));
}

template <int D, int NQ>
__global__ void __launch_bounds__(256)
delta_chunk_mma_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v, const uint16_t* __restrict__ q,
                       const uint16_t* __restrict__ beta, const uint16_t* __restrict__ gl, uint16_t* __restrict__ y,
                       float* __restrict__ Sg, int c, int ntok, int q_raw) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int DM = D / NQ, DP = D + 8;
    static_assert(DM % 16 == 0, "a CTA owns whole 16-row tiles of the state");
    extern __shared__ __align__(16) unsigned char smem[];
    uint16_t* Kh = (uint16_t*)smem;                 // [C][DP]   k
    uint16_t* Qh = Kh + C * DP;                     // [C][DP]   q (unscaled)
    uint16_t* Kt = Qh + C * DP;                     // [D][CP]   k transposed
    uint16_t* Shi = Kt + D * CP;                    // [DM][DP]  rows m0.. of the state, hi and lo
    uint16_t* Slo = Shi + DM * DP;
    uint16_t* bThi = Slo + DM * DP;                 // [DM][CP]  b transposed
    uint16_t* bTlo = bThi + DM * CP;
    uint16_t* uThi = bTlo + DM * CP;                // [DM][CP]  u transposed
    uint16_t* uTlo = uThi + DM * CP;
    uint16_t* wuhi = uTlo + DM * CP;                // [DM][CP]  decay-weighted u transposed
    uint16_t* wulo = wuhi + DM * CP;
    uint16_t* Lh = wulo + DM * CP;                  // [C][CP]   L
    uint16_t* Th = Lh + C * CP;                     // [C][CP]   T
    uint16_t* QKlo = Th + C * CP;                   // [C][CP]   the decayed q.k matrix (lo)
    uint16_t* QKhi = QKlo + C * CP;                 // [C][CP]   the decayed q.k matrix (hi)
    uint16_t* Tt = QKhi + C * CP;                   // [C][CP]   T transposed (operand of the block forward substitution)
    uint16_t* xs = Tt + C * CP;                     // [3][2][16][24] per-warp scratch of that substitution
    float* G = (float*)(xs + 3 * 768);              // [C] running sum of the log decays
    float* bj = G + C;                              // [C] beta
    float* eG = bj + C;                             // [C] exp(G)
    float* wd = eG + C;                             // [C] exp(G_last - G_i)

    const int h = blockIdx.x, m0 = blockIdx.y * DM, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint16_t* kh = k + (size_t)h * ntok * D;
    const uint16_t* vh = v + (size_t)h * ntok * D;
    const uint16_t* qh = q + (size_t)h * ntok * D;
    const uint16_t* bh = beta + (size_t)h * ntok;
    const uint16_t* gh = gl + (size_t)h * ntok;
    uint16_t* yh = y + (size_t)h * ntok * D;
    float* Sglob = Sg + (size_t)h * D * D;
    const float scale = q_raw ? 1.0f : 1.0f / sqrtf((float)D);

    // ---- stage 0: operands into shared memory
    {
        // every global load of the thread is requested before the first one is used (one round trip, not one per step);
        // a warp takes 32 consecutive rows of one 8-column group: the 16-bit stores of the transposed copy then fall on
        // consecutive addresses (taken along a row they hit one bank 16 times over)
        constexpr int KQ_STEPS = C * (D / 8) / 256, S_STEPS = DM * (D / 4) / 256;
        static_assert(C * (D / 8) % 256 == 0 && DM * (D / 4) % 256 == 0, "whole steps of the 256 threads");
        uint4 kv[KQ_STEPS], qv[KQ_STEPS];
        float4 sv[S_STEPS];
#pragma unroll
        for (int u = 0; u < KQ_STEPS; u++) {
            const int e = tid + u * 256, r = e % C, n8 = (e / C) * 8;
            kv[u] = make_uint4(0, 0, 0, 0); qv[u] = make_uint4(0, 0, 0, 0);
            if (r < c) { kv[u] = *(const uint4*)(kh + (size_t)r * D + n8); qv[u] = *(const uint4*)(qh + (size_t)r * D + n8); }
        }
#pragma unroll
        for (int u = 0; u < S_STEPS; u++) {
            const int e = tid + u * 256, r = e / (D / 4), n4 = (e % (D / 4)) * 4;
            sv[u] = *(const float4*)(Sglob + (size_t)(m0 + r) * D + n4);
        }
        // (between the requests and their use: the scan of warp 0 runs while the loads are under way)
        if (warp == 0) {
            // running sum of g over the chunk, in token order (a warp scan would add in another order): every lane
            // adds the 64 values up itself, from registers, and keeps the two sums that are its own
            for (int i = lane; i < C; i += 32) wd[i] = i < c ? h2f(gh[i]) : 0.0f;      // wd as scratch for the raw values
            __syncwarp();
            float acc = 0.0f, mine0 = 0.0f, mine1 = 0.0f, last = 0.0f;
#pragma unroll
            for (int i = 0; i < C; i++) {
                acc += wd[i];
                if (i == lane) mine0 = acc;
                if (i == lane + 32) mine1 = acc;
                if (i == c - 1) last = acc;
            }
            __syncwarp();
            G[lane] = mine0; G[lane + 32] = mine1;
            eG[lane] = expf(mine0); eG[lane + 32] = expf(mine1);
            wd[lane] = expf(last - mine0); wd[lane + 32] = expf(last - mine1);
            for (int i = lane; i < C; i += 32) bj[i] = i < c ? h2f(bh[i]) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < KQ_STEPS; u++) {
            const int e = tid + u * 256, r = e % C, n8 = (e / C) * 8;
            *(uint4*)(Kh + r * DP + n8) = kv[u];
            *(uint4*)(Qh + r * DP + n8) = qv[u];
            const uint16_t* ke = (const uint16_t*)&kv[u];
#pragma unroll
            for (int i = 0; i < 8; i++) Kt[(n8 + i) * CP + r] = ke[i];
        }
#pragma unroll
        for (int u = 0; u < S_STEPS; u++) {
            const int e = tid + u * 256, r = e / (D / 4), n4 = (e % (D / 4)) * 4;
            split_store(Shi + r * DP + n4, Slo + r * DP + n4, sv[u].x);
            split_store(Shi + r * DP + n4 + 1, Slo + r * DP + n4 + 1, sv[u].y);
            split_store(Shi + r * DP + n4 + 2, Slo + r * DP + n4 + 2, sv[u].z);
            split_store(Shi + r * DP + n4 + 3, Slo + r * DP + n4 + 3, sv[u].w);
        }
    }
    __syncthreads();

    // ---- stage 1 (with 3 and 5 below): L[j][i] = f16(exp(G_j - G_i) (k_j . k_i) beta_j) for i < j, else 0
    // Only the 20 tiles of 16 x 8 that touch the lower triangle carry values (row block mi has 2 mi + 2 of them);
    // they are numbered 0..19 and dealt out to the warps in turn, the other 12 are zero and filled apart.
    auto lower_tile = [](int idx, int& mi, int& ni) { mi = idx < 2 ? 0 : idx < 6 ? 1 : idx < 12 ? 2 : 3; ni = idx - (mi * mi + mi); };
    constexpr int LOWER = 20;
    static_assert(C == 64, "the tile numbering above is that of a 64-row chunk");
    for (int idx = warp; idx < LOWER; idx += 8) {
        int mi, ni;
        lower_tile(idx, mi, ni);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(acc, Kh + mi * 16 * DP, DP, Kh + ni * 8 * DP, DP, D, g, t);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = mi * 16 + g + (e >> 1) * 8, i = ni * 8 + 2 * t + (e & 1);
            Lh[j * CP + i] = i < j ? f2h(expf(G[j] - G[i]) * acc[e] * bj[j]) : (uint16_t)0;
        }
    }
    for (int e = tid; e < C * C; e += 256) {          // the tiles above: L = 0, QK = 0
        const int r = e / C, i = e % C;
        if (i >= ((r >> 4) + 1) * 16) { Lh[r * CP + i] = 0; QKhi[r * CP + i] = 0; QKlo[r * CP + i] = 0; }
    }
    // stages 3 and 5 need the operands only, not L or T: same phase, one barrier for the three
    // ---- stage 3: b[j][m] = beta_j (v[j][m] - e^{G_j} (S0 k_j)[m]), stored transposed as hi + lo
    for (int tile = warp; tile < (C / 16) * (DM / 8); tile += 8) {
        const int mi = tile / (DM / 8), ni = tile % (DM / 8);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(acc, Kh + mi * 16 * DP, DP, Shi + ni * 8 * DP, DP, D, g, t);
        mma_rows(acc, Kh + mi * 16 * DP, DP, Slo + ni * 8 * DP, DP, D, g, t);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = mi * 16 + g + (e >> 1) * 8, m = ni * 8 + 2 * t + (e & 1);
            const float vv = j < c ? h2f(vh[(size_t)j * D + m0 + m]) : 0.0f;
            split_store(bThi + m * CP + j, bTlo + m * CP + j, bj[j] * (vv - eG[j] * acc[e]));
        }
    }
    // ---- stage 5: QK[t][i] = exp(G_t - G_i) (q_t . k_i) for i <= t, as hi + lo
    for (int idx = 7 - warp; idx < LOWER; idx += 8) {     // dealt out from the other end: a warp with 3 tiles of L gets 2 here
        int mi, ni;
        lower_tile(idx, mi, ni);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(acc, Qh + mi * 16 * DP, DP, Kh + ni * 8 * DP, DP, D, g, t);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int tt = mi * 16 + g + (e >> 1) * 8, i = ni * 8 + 2 * t + (e & 1);
            split_store(QKhi + tt * CP + i, QKlo + tt * CP + i, i <= tt ? acc[e] * scale * expf(G[tt] - G[i]) : 0.0f);
        }
    }
    __syncthreads();

    // ---- stage 2: T = (I + L)^-1 in fp16. Within a 16 x 16 diagonal block it is the forward substitution of the
    // reference, row by row with every entry rounded to fp16 before the next row uses it; column j depends on column j
    // only, so one lane owns a column and runs down the 16 rows (all four diagonal blocks at once, no block-wide
    // barrier). The blocks below the diagonal follow from (I + L) T = I block row by block row:
    //     T_ik = -T_ii (sum_{k <= m < i} L_im T_mk)
    // two small products per block on the tensor cores (the inner sum as hi + lo), rounded to fp16 once.
    {
        // One lane per column (64 lanes, two warps): the sum over i < r runs in i order, as the reference's
        // solve_tri_f16 forms it, with the column's earlier entries in registers; the entries of L of a row are the
        // same for all 16 columns of a block (broadcast reads that depend on nothing before them).
        if (tid < C) {
            const int j = tid, r0 = j & ~15, jl = j & 15;
            float tc[16];
#pragma unroll
            for (int rr = 0; rr < 16; rr++) {
                float s = 0.0f;
#pragma unroll
                for (int il = 0; il < rr; il++) {
                    const float l = h2f(Lh[(r0 + rr) * CP + r0 + il]);
                    if (il >= jl) s -= l * tc[il];
                }
                const uint16_t tv = jl <= rr ? f2h((rr == jl ? 1.0f : 0.0f) + s) : (uint16_t)0;
                Th[(r0 + rr) * CP + j] = tv;
                Tt[j * CP + r0 + rr] = tv;
                tc[rr] = h2f(tv);
            }
        }
        for (int e = tid; e < C * C; e += 256) {     // blocks above the block diagonal
            const int r = e / C, jj = e % C;
            if ((jj >> 4) > (r >> 4)) Th[r * CP + jj] = 0;
        }
    }
    __syncthreads();
    for (int bi = 1; bi < C / 16; bi++) {
        if (warp < bi) {
            const int bk = warp;
            uint16_t* xhi = xs + warp * 768;        // X transposed [16][24], hi and lo
            uint16_t* xlo = xhi + 384;
            for (int nt = 0; nt < 2; nt++) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                mma_rows(acc, Lh + bi * 16 * CP + bk * 16, CP, Tt + (bk * 16 + nt * 8) * CP + bk * 16, CP, 16 * (bi - bk), g, t);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int row = g + (e >> 1) * 8, n = nt * 8 + 2 * t + (e & 1);
                    split_store(xhi + n * 24 + row, xlo + n * 24 + row, acc[e]);
                }
            }
            __syncwarp();
            for (int nt = 0; nt < 2; nt++) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                mma_rows(acc, Th + bi * 16 * CP + bi * 16, CP, xhi + nt * 8 * 24, 24, 16, g, t);
                mma_rows(acc, Th + bi * 16 * CP + bi * 16, CP, xlo + nt * 8 * 24, 24, 16, g, t);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int row = bi * 16 + g + (e >> 1) * 8, col = bk * 16 + nt * 8 + 2 * t + (e & 1);
                    const uint16_t tv = f2h(-acc[e]);
                    Th[row * CP + col] = tv;
                    Tt[col * CP + row] = tv;
                }
            }
        }
        __syncthreads();
    }

    // ---- stage 4: u = T b ; also u_i weighted with the decay to the end of the chunk (for the state update)
    for (int tile = warp; tile < (C / 16) * (DM / 8); tile += 8) {
        const int mi = tile / (DM / 8), ni = tile % (DM / 8);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(acc, Th + mi * 16 * CP, CP, bThi + ni * 8 * CP, CP, C, g, t);
        mma_rows(acc, Th + mi * 16 * CP, CP, bTlo + ni * 8 * CP, CP, C, g, t);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = mi * 16 + g + (e >> 1) * 8, m = ni * 8 + 2 * t + (e & 1);
            split_store(uThi + m * CP + j, uTlo + m * CP + j, acc[e]);
            split_store(wuhi + m * CP + j, wulo + m * CP + j, j < c ? wd[j] * acc[e] : 0.0f);
        }
    }
    __syncthreads();

    // ---- stage 6: y_t = e^{G_t} (S0 q_t) + sum_{i<=t} QK[t][i] u_i
    for (int tile = warp; tile < (C / 16) * (DM / 8); tile += 8) {
        const int mi = tile / (DM / 8), ni = tile % (DM / 8);
        float a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(a1, Qh + mi * 16 * DP, DP, Shi + ni * 8 * DP, DP, D, g, t);
        mma_rows(a1, Qh + mi * 16 * DP, DP, Slo + ni * 8 * DP, DP, D, g, t);
        mma_rows(a2, QKhi + mi * 16 * CP, CP, uThi + ni * 8 * CP, CP, C, g, t);
        mma_rows(a2, QKhi + mi * 16 * CP, CP, uTlo + ni * 8 * CP, CP, C, g, t);
        mma_rows(a2, QKlo + mi * 16 * CP, CP, uThi + ni * 8 * CP, CP, C, g, t);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int tt = mi * 16 + g + (e >> 1) * 8, m = ni * 8 + 2 * t + (e & 1);
            if (tt < c) yh[(size_t)tt * D + m0 + m] = f2h(eG[tt] * scale * a1[e] + a2[e]);
        }
    }

    // ---- stage 7: S'[m][n] = e^{G_last} S0[m][n] + sum_i (decay_i u_i[m]) k_i[n]   (reads wu and k transposed: no barrier needed)
    const float eC = eG[c - 1];
    for (int tile = warp; tile < (DM / 16) * (D / 8); tile += 8) {
        const int mi = tile / (D / 8), ni = tile % (D / 8);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows(acc, wuhi + mi * 16 * CP, CP, Kt + ni * 8 * CP, CP, C, g, t);
        mma_rows(acc, wulo + mi * 16 * CP, CP, Kt + ni * 8 * CP, CP, C, g, t);
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
            const int m = m0 + mi * 16 + g + (e >> 1) * 8, n = ni * 8 + 2 * t;
            float2* sp = (float2*)(Sglob + (size_t)m * D + n);
            const float2 s0 = *sp;
            *sp = make_float2(s0.x * eC + acc[e], s0.y * eC + acc[e + 1]);
        }
    }
}

template <int D, int NQ>
bool launch(cudaStream_t st, const uint16_t* k, const uint16_t* v, const uint16_t* q, const uint16_t* beta, const uint16_t* g,
            uint16_t* y, float* S, uint32_t c, uint32_t ntok, uint32_t H, uint32_t q_raw) {
    static int have[64];
    constexpr int DM = D / NQ, DP = D + 8;
    const size_t smem = (size_t)(2 * C * DP + D * CP + 2 * DM * DP + 6 * DM * CP + 5 * C * CP + 3 * 768) * 2 + 4 * C * sizeof(float);
    if (!ensure_dyn_smem(delta_chunk_mma_kernel<D, NQ>, smem, have)) return false;
    launch_pdl(delta_chunk_mma_kernel<D, NQ>, dim3(dim3(H, NQ)), dim3(256), smem, st, k, v, q, beta, g, y, S, (int)c, (int)ntok, (int)q_raw);
    g_launches++;
    return true;
}

}  // namespace

// false: shape not taken (head dim other than 64 or 128, operands not 16-byte aligned); nothing launched
bool k_delta_chunk_mma(cudaStream_t st, const uint16_t* k, const uint16_t* v, const uint16_t* q, const uint16_t* beta,
                       const uint16_t* g, uint16_t* y, float* S, uint32_t c, uint32_t ntok, uint32_t H, uint32_t D, uint32_t q_raw) {
    if (!c || c > 64 || c > ntok || !H) return false;
    if ((((uintptr_t)k) | ((uintptr_t)q) | ((uintptr_t)S)) & 15u) return false;
    // the value dimension in slices of 16 rows per CTA: 8 CTAs per head at 128, 4 at 64
    if (D == 128) return launch<128, 8>(st, k, v, q, beta, g, y, S, c, ntok, H, q_raw);
    if (D == 64) return launch<64, 4>(st, k, v, q, beta, g, y, S, c, ntok, H, q_raw);
    return false;
}

}  // namespace gehtp
