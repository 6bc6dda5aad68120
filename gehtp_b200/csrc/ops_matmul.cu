// fp16 x fp16 -> fp16 matmul of the runlist (opcodes 24 and 35).
// Reference: exec_matmul_f16 (kernels/src/runtime/oplist_exec.c:1709-1813) and
// its GEMV variant (:1483-1590): Y[M,N] = A.W with fp32 accumulation in
// ascending k and one fp16 rounding; flags choose A stored [K,M], W stored
// [N,K], and a leading batch dim; the SPLIT form writes columns
// [n0, n0+N) of a row of N_full.
//
// This kernel keeps the reference's summation order: every output element is
// accumulated by one thread, k ascending, in fp32. A product of two fp16 values
// is exact in fp32, so fma and multiply-then-add agree and the result is
// bit-identical to the reference's scalar loop for any shape.
#include "common.cuh"
#include "launchers.h"

namespace gehtp {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
matmul_f16_exact_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ w,
                        uint16_t* __restrict__ y, uint32_t M, uint32_t K, uint32_t N, uint32_t n0,
                        uint32_t N_full, int t0, int t1) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    const uint32_t bb = blockIdx.z;
    a += (size_t)bb * M * K;
    w += (size_t)bb * K * N_full;
    y += (size_t)bb * M * N_full;
    const uint32_t m0 = blockIdx.y * TM, c0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
        for (int e = threadIdx.x; e < TM * TK; e += 256) {
            int m, k;
            if (t0) { m = e % TM; k = e / TM; } else { k = e % TK; m = e / TK; }
            uint32_t gm = m0 + m, gk = k0 + k;
            float v = 0.0f;
            if (gm < M && gk < K) v = h2f(a[t0 ? (size_t)gk * M + gm : (size_t)gm * K + gk]);
            As[k][m] = v;
        }
        for (int e = threadIdx.x; e < TN * TK; e += 256) {
            int n, k;
            if (t1) { k = e % TK; n = e / TK; } else { n = e % TN; k = e / TN; }
            uint32_t gn = c0 + n, gk = k0 + k;
            float v = 0.0f;
            if (gn < N && gk < K)
                v = h2f(w[t1 ? (size_t)(n0 + gn) * K + gk : (size_t)gk * N_full + (n0 + gn)]);
            Ws[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; k++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t gn = c0 + tx * 4 + j;
            if (gn < N) y[(size_t)gm * N_full + n0 + gn] = f2h(acc[i][j]);
        }
    }
}

// Skinny form (M <= 4): one warp per output column group, k split across
// lanes is NOT used, to keep the ascending-k order; instead each thread owns
// one column and walks k. Coalesced for W stored [K,N]; for W stored [N,K]
// each thread streams its own row.
__global__ void __launch_bounds__(128)
matvec_f16_exact_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ w,
                        uint16_t* __restrict__ y, uint32_t M, uint32_t K, uint32_t N, uint32_t n0,
                        uint32_t N_full, int t0, int t1) {
    extern __shared__ float av[];  // [M][K]
    const uint32_t bb = blockIdx.z;
    a += (size_t)bb * M * K;
    w += (size_t)bb * K * N_full;
    y += (size_t)bb * M * N_full;
    for (uint32_t e = threadIdx.x; e < M * K; e += blockDim.x) {
        uint32_t m = e / K, k = e % K;
        av[e] = h2f(a[t0 ? (size_t)k * M + m : (size_t)m * K + k]);
    }
    __syncthreads();
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (t1) {
        const uint16_t* wr = w + (size_t)(n0 + n) * K;
        for (uint32_t k = 0; k < K; k++) {
            float wv = h2f(wr[k]);
            for (uint32_t m = 0; m < M; m++) acc[m] = fmaf(av[m * K + k], wv, acc[m]);
        }
    } else {
        const uint16_t* wc = w + n0 + n;
        for (uint32_t k = 0; k < K; k++) {
            float wv = h2f(wc[(size_t)k * N_full]);
            for (uint32_t m = 0; m < M; m++) acc[m] = fmaf(av[m * K + k], wv, acc[m]);
        }
    }
    for (uint32_t m = 0; m < M; m++) y[(size_t)m * N_full + n0 + n] = f2h(acc[m]);
}

void k_matmul_f16(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M,
                  uint32_t K, uint32_t N, uint32_t n0, uint32_t N_full, int t0, int t1,
                  uint32_t Bn) {
    if (!M || !N || !Bn) return;
    if (Bn > 1) t0 = 0;  // the batched form ignores the A-transposed bit (oplist_exec.c:1787-1800)
    if (M <= 4 && !t1 && (size_t)M * K * sizeof(float) <= 40 * 1024) {
        dim3 grid((N + 127) / 128, 1, Bn);
        matvec_f16_exact_kernel<<<grid, 128, (size_t)M * K * sizeof(float), st>>>(
            a, w, y, M, K, N, n0, N_full, t0, t1);
    } else {
        dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, Bn);
        matmul_f16_exact_kernel<<<grid, 256, 0, st>>>(a, w, y, M, K, N, n0, N_full, t0, t1);
    }
    g_launches++;
}

}  // namespace gehtp
