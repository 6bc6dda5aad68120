// Gated-delta-net ops: depthwise causal conv1d (whole sequence and one-token
// step) and the chunked gated delta rule. Reference: exec_conv1d_ssm
// (kernels/src/runtime/oplist_exec.c:1349-1376), conv1d_step_f16 and
// delta_chunk_f16 / solve_tri_f16 (kernels/src/hvx/gdn_kern.c:14-38, 54-167;
// formulas in kernels/include/gdn_sm.h:5-12).
// Compiled with --fmad=false: the reference multiplies, rounds, then adds, and
// each sum below runs in the reference's order so that results differ from it
// only through expf.
#include "common.cuh"
#include "launchers.h"

namespace gehtp {

// y[t,c] = sum_j w[j,c] * x[t-(k-1)+j, c]; input rows beyond seq-k+1 and
// before 0 count as zero; no activation.
__global__ void conv1d_ssm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                                  uint16_t* __restrict__ y, uint32_t seq, uint32_t C, uint32_t k) {
    const int32_t in_rows = (seq >= k) ? (int32_t)(seq - k + 1) : 0;
    const size_t total = (size_t)seq * C;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        uint32_t t = (uint32_t)(e / C), c = (uint32_t)(e % C);
        float acc = 0.0f;
        for (uint32_t j = 0; j < k; j++) {
            int32_t src = (int32_t)t - (int32_t)(k - 1) + (int32_t)j;
            if (src < 0 || src >= in_rows) continue;
            acc += h2f(x[(size_t)src * C + c]) * h2f(w[(size_t)j * C + c]);
        }
        y[e] = f2h(acc);
    }
}

// The same for C % 8 == 0 and k = 2..4 with 16-byte accesses: a thread owns 8 neighbouring channels and TT
// consecutive tokens; the k - 1 rows before them slide through registers, so every input row is loaded
// once per TT outputs (HBM traffic ~ (1 + (k-1)/TT) reads + 1 write per element). Sums run over j
// ascending and skip rows outside [0, seq-k+1), exactly as above.
constexpr int CONV_TT = 8;
template <int K>
__global__ void __launch_bounds__(256)
conv1d_ssm_vec_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w, uint4* __restrict__ y, uint32_t seq,
                      uint32_t C8) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int32_t in_rows = (seq >= (uint32_t)K) ? (int32_t)(seq - K + 1) : 0;
    const uint32_t c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 >= C8) return;
    const uint32_t t0 = blockIdx.y * CONV_TT;
    float wf[K][8];            // [tap][channel]
#pragma unroll
    for (int j = 0; j < K; j++) {
        const uint4 q = __ldg(w + (size_t)j * C8 + c8);
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { wf[j][2 * i] = h2f((uint16_t)(ww[i] & 0xffffu)); wf[j][2 * i + 1] = h2f((uint16_t)(ww[i] >> 16)); }
    }
    // rows t0-(K-1) .. t0+TT-1 of this channel group
    constexpr int R = CONV_TT + K - 1;
    float xf[R][8];
    bool ok[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int32_t src = (int32_t)t0 - (K - 1) + r;
        ok[r] = src >= 0 && src < in_rows;
        uint4 q = make_uint4(0, 0, 0, 0);
        if (ok[r]) q = __ldcs(x + (size_t)src * C8 + c8);
        const uint32_t xx[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { xf[r][2 * i] = h2f((uint16_t)(xx[i] & 0xffffu)); xf[r][2 * i + 1] = h2f((uint16_t)(xx[i] >> 16)); }
    }
#pragma unroll
    for (int tt = 0; tt < CONV_TT; tt++) {
        const uint32_t t = t0 + tt;
        if (t < seq) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < K; j++) {
                if (ok[tt + j]) {                       // input row t - (K-1) + j
#pragma unroll
                    for (int ch = 0; ch < 8; ch++) acc[ch] += xf[tt + j][ch] * wf[j][ch];
                }
            }
            uint4 o;
            o.x = (uint32_t)f2h(acc[0]) | ((uint32_t)f2h(acc[1]) << 16);
            o.y = (uint32_t)f2h(acc[2]) | ((uint32_t)f2h(acc[3]) << 16);
            o.z = (uint32_t)f2h(acc[4]) | ((uint32_t)f2h(acc[5]) << 16);
            o.w = (uint32_t)f2h(acc[6]) | ((uint32_t)f2h(acc[7]) << 16);
            y[(size_t)t * C8 + c8] = o;
        }
    }
}

void k_conv1d_ssm(cudaStream_t st, const uint16_t* x, const uint16_t* w, uint16_t* y, uint32_t seq,
                  uint32_t C, uint32_t k) {
    size_t total = (size_t)seq * C;
    if (!total) return;
    if (C % 8 == 0 && k >= 2 && k <= 4 && !((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)y)) & 15)) {
        const uint32_t C8 = C / 8;
        const uint32_t bx = C8 >= 128 ? 128 : 64;
        const dim3 grid((C8 + bx - 1) / bx, (seq + CONV_TT - 1) / CONV_TT);
        if (k == 4) launch_pdl(conv1d_ssm_vec_kernel<4>, dim3(grid), dim3(bx), 0, st, (const uint4*)x, (const uint4*)w, (uint4*)y, seq, C8);
        else if (k == 3) launch_pdl(conv1d_ssm_vec_kernel<3>, dim3(grid), dim3(bx), 0, st, (const uint4*)x, (const uint4*)w, (uint4*)y, seq, C8);
        else launch_pdl(conv1d_ssm_vec_kernel<2>, dim3(grid), dim3(bx), 0, st, (const uint4*)x, (const uint4*)w, (uint4*)y, seq, C8);
        g_launches++;
        return;
    }
    size_t g = (total + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    conv1d_ssm_kernel<<<(unsigned)g, 256, 0, st>>>(x, w, y, seq, C, k);
    g_launches++;
}

// One token: s = sum_{i<dc-1} w[i,c]*win[i,c] + w[dc-1,c]*x[c]; y = silu(s);
// then the fp32 window shifts by one and takes x.
__global__ void conv1d_step_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                                   uint16_t* __restrict__ y, float* __restrict__ win, uint32_t C,
                                   uint32_t dc) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float xf = h2f(x[c]);
    float s = 0.0f;
    for (uint32_t i = 0; i + 1 < dc; i++) s += h2f(w[(size_t)i * C + c]) * win[(size_t)i * C + c];
    s += h2f(w[(size_t)(dc - 1) * C + c]) * xf;
    y[c] = f2h(s / (1.0f + expf(-s)));
    for (uint32_t i = 0; i + 2 < dc; i++) win[(size_t)i * C + c] = win[(size_t)(i + 1) * C + c];
    win[(size_t)(dc - 2) * C + c] = xf;
}

void k_conv1d_step(cudaStream_t st, const uint16_t* x, const uint16_t* w, uint16_t* y, float* win,
                   uint32_t C, uint32_t dc) {
    conv1d_step_kernel<<<(C + 127) / 128, 128, 0, st>>>(x, w, y, win, C, dc);
    g_launches++;
}

// Chunked gated delta rule, one CTA per head, c <= 64 tokens, state S[D][D]
// fp32 updated in place. Shared memory: kf, qf, bm (v then b), u [c][D] fp32;
// S [D][D] fp32 when D <= 128; L and T [c][c] fp16, later reused as QK fp32.
template <bool S_SMEM>
__global__ void __launch_bounds__(256)
delta_chunk_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                   const uint16_t* __restrict__ q, const uint16_t* __restrict__ beta,
                   const uint16_t* __restrict__ g, uint16_t* __restrict__ y, float* __restrict__ Sg,
                   int c, int ntok, int D, int q_raw) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int h = blockIdx.x, tid = threadIdx.x, NT = blockDim.x;
    // The value dimension m is split over gridDim.y CTAs per head: b, u, y and the rows of S are
    // independent across m (every element is computed exactly as an unsplit CTA would), while the
    // small c x c matrices L, T and QK are recomputed by each of them.
    const int Dm = D / (int)gridDim.y, m0 = (int)blockIdx.y * Dm;
    // Rows of kf, qf and S are padded by one float: several loops walk them with the
    // row index on the lanes, which without the pad lands every lane in the same bank.
    const int DP = D + 1;
    float* kf = (float*)smem;
    float* qf = kf + (size_t)c * DP;
    float* bm = qf + (size_t)c * DP;
    float* u = bm + (size_t)c * D;
    float* G = u + (size_t)c * D;      // [64]
    float* bj = G + 64;                // [64]
    uint16_t* Lh = (uint16_t*)(bj + 64);  // [c][c]
    uint16_t* T = Lh + 64 * 64;           // [c][c]
    float* QK = (float*)Lh;               // [c][c] fp32, after T is dead
    float* S = S_SMEM ? (float*)(T + 64 * 64) : Sg + (size_t)h * D * D;
    float* Sglob = Sg + (size_t)h * D * D;

    const uint16_t* kh = k + (size_t)h * ntok * D;
    const uint16_t* vh = v + (size_t)h * ntok * D;
    const uint16_t* qh = q + (size_t)h * ntok * D;
    const uint16_t* bh = beta + (size_t)h * ntok;
    const uint16_t* gh = g + (size_t)h * ntok;
    uint16_t* yh = y + (size_t)h * ntok * D;
    const float scale = q_raw ? 1.0f : 1.0f / sqrtf((float)D);

    if (tid == 0) {
        float acc = 0.0f;
        for (int t = 0; t < c; t++) { acc += h2f(gh[t]); G[t] = acc; }
    }
    for (int t = tid; t < c; t += NT) bj[t] = h2f(bh[t]);
    const int SP = S_SMEM ? DP : D;   // row stride of S (the global copy is not padded)
    const int ms0 = S_SMEM ? m0 : 0;  // first row held by S (the shared copy holds this CTA's rows only)
    for (int e = tid; e < c * D; e += NT) {
        const int r = e / D, n = e % D;
        kf[r * DP + n] = h2f(kh[e]);
        bm[e] = h2f(vh[e]);
        qf[r * DP + n] = h2f(qh[e]) * scale;
    }
    if (S_SMEM)
        for (int e = tid; e < Dm * D; e += NT) S[(e / D) * SP + e % D] = Sglob[(size_t)m0 * D + e];
    __syncthreads();

    // L[j][i] = exp(G_j - G_i) * (k_j . k_i) * beta_j for i < j, else 0 (fp16)
    for (int e = tid; e < c * c; e += NT) {
        int j = e / c, i = e % c;
        uint16_t r = 0;
        if (i < j) {
            float s = 0.0f;
            for (int n = 0; n < D; n++) s += kf[j * DP + n] * kf[i * DP + n];
            r = f2h(expf(G[j] - G[i]) * s * bj[j]);
        }
        Lh[j * c + i] = r;
    }
    __syncthreads();
    // T = (I + L)^-1 by rows; each row needs the rows above it
    // Four lanes share a column j and split the sum over i (the rows are a dependency chain of c
    // steps, so the step itself has to be short); the four partial sums are added pairwise.
    for (int r = 0; r < c; r++) {
        for (int base = 0; base < c * 4; base += NT) {        // every thread runs the body: the shuffles need whole warps
            const int jj = base + tid, j = jj >> 2, part = jj & 3;
            float s = 0.0f;
            if (j < r && j < c)
                for (int i = j + part; i < r; i += 4) s -= h2f(Lh[r * c + i]) * h2f(T[i * c + j]);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (part == 0 && j < c) T[r * c + j] = j <= r ? f2h((r == j ? 1.0f : 0.0f) + s) : (uint16_t)0;
        }
        __syncthreads();
    }
    // b_j = beta_j (v_j - e^{G_j} S0 k_j), in place over v
    for (int e = tid; e < c * Dm; e += NT) {
        int j = e / Dm, m = m0 + e % Dm;
        float sk = 0.0f;
        for (int n = 0; n < D; n++) sk += S[(m - ms0) * SP + n] * kf[j * DP + n];
        bm[j * D + m] = bj[j] * (bm[j * D + m] - expf(G[j]) * sk);
    }
    __syncthreads();
    // u = T b
    for (int e = tid; e < c * Dm; e += NT) {
        int j = e / Dm, m = m0 + e % Dm;
        float acc = 0.0f;
        for (int i = 0; i <= j; i++) {
            float tij = h2f(T[j * c + i]);
            if (tij == 0.0f) continue;
            acc += tij * bm[i * D + m];
        }
        u[j * D + m] = acc;
    }
    __syncthreads();
    // QK[t][i] = exp(G_t - G_i) (q_t . k_i), i <= t (T and L are dead now)
    for (int e = tid; e < c * c; e += NT) {
        int t = e / c, i = e % c;
        float qk = 0.0f;
        if (i <= t) {
            for (int n = 0; n < D; n++) qk += qf[t * DP + n] * kf[i * DP + n];
            qk *= expf(G[t] - G[i]);
        }
        QK[e] = qk;
    }
    __syncthreads();
    // y_t = e^{G_t} (S0 q_t) + sum_{i<=t} QK[t][i] u_i
    for (int e = tid; e < c * Dm; e += NT) {
        int t = e / Dm, m = m0 + e % Dm;
        float s = 0.0f;
        for (int n = 0; n < D; n++) s += S[(m - ms0) * SP + n] * qf[t * DP + n];
        float acc = expf(G[t]) * s;
        for (int i = 0; i <= t; i++) {
            float qk = QK[t * c + i];
            if (qk == 0.0f) continue;
            acc += qk * u[i * D + m];
        }
        yh[t * D + m] = f2h(acc);
    }
    __syncthreads();
    // S' = e^{G_c} S0 + sum_i e^{G_c - G_i} u_i k_i^T
    const float eC = expf(G[c - 1]);
    for (int i = tid; i < c; i += NT) bj[i] = expf(G[c - 1] - G[i]);   // beta is dead by now: its row holds the decay of token i
    __syncthreads();
    for (int e = tid; e < Dm * D; e += NT) {
        int m = m0 + e / D, n = e % D;
        float sv = S[(m - ms0) * SP + n] * eC;
        for (int i = 0; i < c; i++) {
            float wu = bj[i] * u[i * D + m];
            if (wu == 0.0f) continue;
            sv += wu * kf[i * DP + n];
        }
        Sglob[(size_t)m * D + n] = sv;
    }
}

void k_delta_chunk(cudaStream_t st, const uint16_t* k, const uint16_t* v, const uint16_t* q,
                   const uint16_t* beta, const uint16_t* g, uint16_t* y, float* S, uint32_t c,
                   uint32_t ntok, uint32_t H, uint32_t D, uint32_t q_raw) {
    // 4 CTAs per head when D allows: each owns D/4 value columns and D/4 rows of S
    const uint32_t MS = (D % 4 == 0 && D >= 64) ? 4 : 1;
    size_t base = (size_t)2 * c * D * 4 + (size_t)2 * c * (D + 1) * 4 + 128 * 4 + 2 * 64 * 64 * 2;
    size_t s_bytes = (size_t)(D / MS) * (D + 1) * 4;
    bool s_smem = base + s_bytes <= 227 * 1024;
    size_t smem = base + (s_smem ? s_bytes : 0);
    const dim3 grid(H, MS);
    if (s_smem) {
        cudaFuncSetAttribute(delta_chunk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        delta_chunk_kernel<true><<<grid, 256, smem, st>>>(k, v, q, beta, g, y, S, (int)c, (int)ntok, (int)D, (int)q_raw);
    } else {
        cudaFuncSetAttribute(delta_chunk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        delta_chunk_kernel<false><<<grid, 256, smem, st>>>(k, v, q, beta, g, y, S, (int)c, (int)ntok, (int)D, (int)q_raw);
    }
    g_launches++;
}

}  // namespace gehtp
