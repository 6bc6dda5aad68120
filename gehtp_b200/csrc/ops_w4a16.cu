// W4A16 group-64 matmul, streaming form for small M (decode), plus the one-time
// repack of a weight slot into the device layout both W4A16 kernels read.
//
// Slot form (the runlist ABI): nibbles[K][N/2] with the low nibble holding the
// even column, then fp16 scales[K/64][N]; w = fp16((q - 8) * scale).
//
// Device layout ("strip-major"): the matrix is cut into units of 64 k (one
// scale group) x 16 n. A unit is 512 contiguous bytes = one 16-byte vector per
// lane of a warp, units ordered [k group][n strip]. Lane (g = lane/4,
// t = lane%4) holds, for columns n0+g and n0+g+8, the 16 weights at
// k = kg*64 + t*16 + 0..15. Its four 32-bit words j = 0..3 cover k offsets
// 4j..4j+3; inside a word the nibbles sit so that two mask-and-or steps yield
// the four fp16 pairs of an mma.m16n8k16 A fragment:
//     nibble 0,4 : (g,   4j+0), (g,   4j+1)      nibble 1,5 : (g+8, 4j+0), (g+8, 4j+1)
//     nibble 2,6 : (g,   4j+2), (g,   4j+3)      nibble 3,7 : (g+8, 4j+2), (g+8, 4j+3)
// The k order inside a group is therefore permuted for the tensor-core
// contraction; the activations are read with the same permutation (each lane
// reads the 16 contiguous fp16 at k = kg*64 + t*16), so no shared memory and no
// shuffle is needed to build the B fragment.
//
// Skinny kernel: one CTA per 16-column strip and per tile of 8 (or 16) rows of
// A; warp w streams the k groups [w*kgw, (w+1)*kgw) of that strip with all its
// 16-byte loads issued up front, accumulates in fp32 through mma.sync, and the
// warps' partial sums are added in warp order through shared memory, so the
// result does not depend on scheduling.
#include <cuda_fp16.h>
#include "common.cuh"
#include "launchers_w4.h"

namespace gehtp {

// ------------------------------------------------------------------ repack
__device__ __forceinline__ uint32_t nib_at(const uint8_t* __restrict__ nib, uint32_t N, uint32_t k,
                                           uint32_t n) {
    uint8_t b = nib[(size_t)k * (N / 2) + (n >> 1)];
    return (n & 1u) ? (b >> 4) : (b & 15u);
}

__global__ void w4_repack_kernel(const uint8_t* __restrict__ nib, uint32_t* __restrict__ packed,
                                 uint32_t K, uint32_t N) {
    const uint32_t NB = N / 16;
    const size_t words = (size_t)K * N / 8;
    for (size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; wi < words;
         wi += (size_t)gridDim.x * blockDim.x) {
        uint32_t j = (uint32_t)(wi & 3), lane = (uint32_t)((wi >> 2) & 31);
        size_t unit = wi >> 7;
        uint32_t nb = (uint32_t)(unit % NB), kg = (uint32_t)(unit / NB);
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t nlo = nb * 16 + g, nhi = nlo + 8, kb = kg * 64 + t * 16 + 4 * j;
        uint32_t w = nib_at(nib, N, kb, nlo) | nib_at(nib, N, kb, nhi) << 4 |
                     nib_at(nib, N, kb + 2, nlo) << 8 | nib_at(nib, N, kb + 2, nhi) << 12 |
                     nib_at(nib, N, kb + 1, nlo) << 16 | nib_at(nib, N, kb + 1, nhi) << 20 |
                     nib_at(nib, N, kb + 3, nlo) << 24 | nib_at(nib, N, kb + 3, nhi) << 28;
        packed[wi] = w;
    }
}

void k_w4_repack(cudaStream_t st, const uint8_t* nib, uint32_t* packed, uint32_t K, uint32_t N) {
    size_t words = (size_t)K * N / 8;
    size_t g = (words + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    w4_repack_kernel<<<(unsigned)g, 256, 0, st>>>(nib, packed, K, N);
    g_launches++;
}

// Inverse of the repack, as integers q - 8: out[k][n].
__global__ void w4_unpack_kernel(const uint32_t* __restrict__ packed, int8_t* __restrict__ out,
                                 uint32_t K, uint32_t N) {
    const uint32_t NB = N / 16;
    const size_t words = (size_t)K * N / 8;
    for (size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; wi < words;
         wi += (size_t)gridDim.x * blockDim.x) {
        uint32_t j = (uint32_t)(wi & 3), lane = (uint32_t)((wi >> 2) & 31);
        size_t unit = wi >> 7;
        uint32_t nb = (uint32_t)(unit % NB), kg = (uint32_t)(unit / NB);
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t nlo = nb * 16 + g, nhi = nlo + 8, kb = kg * 64 + t * 16 + 4 * j;
        uint32_t w = packed[wi];
        const uint32_t koff[8] = {0, 0, 2, 2, 1, 1, 3, 3};
        for (int i = 0; i < 8; i++) {
            uint32_t n = (i & 1) ? nhi : nlo;
            out[(size_t)(kb + koff[i]) * N + n] = (int8_t)((int)((w >> (4 * i)) & 15u) - 8);
        }
    }
}

void k_w4_unpack_i8(cudaStream_t st, const uint32_t* packed, int8_t* out, uint32_t K, uint32_t N) {
    size_t words = (size_t)K * N / 8;
    size_t g = (words + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    w4_unpack_kernel<<<(unsigned)g, 256, 0, st>>>(packed, out, K, N);
    g_launches++;
}

// ------------------------------------------------------------------ skinny matmul
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One packed word -> four fp16 pairs (q - 8) * scale. `slo` / `shi` hold the
// scale of column g / g+8 in both halves.
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 slo, __half2 shi,
                                             uint32_t (&a)[4]) {
    const uint32_t MAGIC = 0x64006400u;          // 1024.0 in both halves
    const __half2 c1032 = __half2half2(__ushort_as_half(0x6408));   // 1032
    const __half2 c16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
    const __half2 cm72 = __half2half2(__ushort_as_half(0xd480));    // -72
    uint32_t w8 = w >> 8;
    uint32_t p0 = (w & 0x000f000fu) | MAGIC;    // 1024 + q
    uint32_t p1 = (w & 0x00f000f0u) | MAGIC;    // 1024 + 16 q
    uint32_t p2 = (w8 & 0x000f000fu) | MAGIC;
    uint32_t p3 = (w8 & 0x00f000f0u) | MAGIC;
    __half2 h0 = __hsub2(*(__half2*)&p0, c1032);
    __half2 h1 = __hfma2(*(__half2*)&p1, c16th, cm72);
    __half2 h2 = __hsub2(*(__half2*)&p2, c1032);
    __half2 h3 = __hfma2(*(__half2*)&p3, c16th, cm72);
    h0 = __hmul2(h0, slo);
    h1 = __hmul2(h1, shi);
    h2 = __hmul2(h2, slo);
    h3 = __hmul2(h3, shi);
    a[0] = *(uint32_t*)&h0;
    a[1] = *(uint32_t*)&h1;
    a[2] = *(uint32_t*)&h2;
    a[3] = *(uint32_t*)&h3;
}

// SwiGLU on two accumulators with the op chain's roundings: gate -> fp16,
// sigmoid -> fp16, gate*sigmoid -> fp16, up -> fp16, product -> fp16
// (UNARY subtype 8 and two BINARY mul ops of the reference executor).
__device__ __forceinline__ uint16_t swiglu_chain(float gate_acc, float up_acc) {
    float gt = h2f(f2h(gate_acc));
    float sg = h2f(f2h(1.0f / (1.0f + expf(-gt))));
    float act = h2f(f2h(__fmul_rn(gt, sg)));
    float up = h2f(f2h(up_acc));
    return f2h(__fmul_rn(act, up));
}

template <int MT, int UNROLL, bool DUAL, bool FULL>
__global__ void __launch_bounds__(640)
w4a16_skinny_kernel(const uint16_t* __restrict__ a, const uint4* __restrict__ wp,
                    const uint16_t* __restrict__ sc, const uint4* __restrict__ wp2,
                    const uint16_t* __restrict__ sc2, uint16_t* __restrict__ y, uint32_t M,
                    uint32_t K, uint32_t N, uint32_t kgw, W4Epilogue ep) {
    extern __shared__ float red[];  // [nwarps][NACC][32]
    constexpr int NACC = MT * 4 * (DUAL ? 2 : 1);
    // Programmatic dependent launch: let the next kernel start early, and order
    // this one after its predecessor only once the first batch of weight loads
    // (constants, independent of the predecessor) is in flight.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    bool waited = false;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t nb = blockIdx.x, NB = N / 16, KG = K / 64;
    const uint32_t m0 = blockIdx.y * (8 * MT);
    const uint32_t n_lo = nb * 16 + g;
    uint32_t kg0 = warp * kgw, kg1 = kg0 + kgw;
    if (kg1 > KG) kg1 = KG;

    float acc[MT][4], acc2[DUAL ? MT : 1][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) { acc[i][c] = 0.0f; if (DUAL) acc2[i][c] = 0.0f; }

    const uint4* wbase = wp + (size_t)nb * 32 + lane;
    const uint4* wbase2 = DUAL ? wp2 + (size_t)nb * 32 + lane : nullptr;
    const uint4* arow[MT];   // this lane's activation row at the warp's first group, or NULL past M
#pragma unroll
    for (int i = 0; i < MT; i++) {
        const uint32_t m = m0 + i * 8 + g;
        arow[i] = m < M ? (const uint4*)(a + (size_t)m * K + (size_t)kg0 * 64 + t * 16) : nullptr;
    }
    for (uint32_t kg = kg0; kg < (FULL ? kg0 + 1 : kg1); kg += UNROLL) {
        uint4 wq[UNROLL], wq2[DUAL ? UNROLL : 1];
        uint16_t s0[UNROLL], s1[UNROLL], t0[DUAL ? UNROLL : 1], t1[DUAL ? UNROLL : 1];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (FULL || kg + u < kg1) {
                wq[u] = __ldcs(wbase + (size_t)(kg + u) * NB * 32);  // streamed once: evict first
                s0[u] = __ldg(sc + (size_t)(kg + u) * N + n_lo);
                s1[u] = __ldg(sc + (size_t)(kg + u) * N + n_lo + 8);
                if (DUAL) {
                    wq2[u] = __ldcs(wbase2 + (size_t)(kg + u) * NB * 32);
                    t0[u] = __ldg(sc2 + (size_t)(kg + u) * N + n_lo);
                    t1[u] = __ldg(sc2 + (size_t)(kg + u) * N + n_lo + 8);
                }
            } else {
                wq[u] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
                s0[u] = 0; s1[u] = 0;
                if (DUAL) { wq2[u] = wq[u]; t0[u] = 0; t1[u] = 0; }
            }
        }
        if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (!FULL && kg + u >= kg1) break;
            uint32_t af[4][4], af2[DUAL ? 4 : 1][4];
            {
                const __half2 slo = __half2half2(__ushort_as_half(s0[u]));
                const __half2 shi = __half2half2(__ushort_as_half(s1[u]));
                dequant_word(wq[u].x, slo, shi, af[0]);
                dequant_word(wq[u].y, slo, shi, af[1]);
                dequant_word(wq[u].z, slo, shi, af[2]);
                dequant_word(wq[u].w, slo, shi, af[3]);
            }
            if (DUAL) {
                const __half2 slo = __half2half2(__ushort_as_half(t0[u]));
                const __half2 shi = __half2half2(__ushort_as_half(t1[u]));
                dequant_word(wq2[u].x, slo, shi, af2[0]);
                dequant_word(wq2[u].y, slo, shi, af2[1]);
                dequant_word(wq2[u].z, slo, shi, af2[2]);
                dequant_word(wq2[u].w, slo, shi, af2[3]);
            }
#pragma unroll
            for (int i = 0; i < MT; i++) {
                uint4 b0 = make_uint4(0, 0, 0, 0), b1 = b0;
                if (arow[i]) {
                    const uint4* ap = arow[i] + (size_t)(kg - kg0 + u) * 8;   // 64 fp16 per group
                    b0 = __ldg(ap);
                    b1 = __ldg(ap + 1);
                }
                mma16816(acc[i], af[0], b0.x, b0.y);
                mma16816(acc[i], af[1], b0.z, b0.w);
                mma16816(acc[i], af[2], b1.x, b1.y);
                mma16816(acc[i], af[3], b1.z, b1.w);
                if (DUAL) {
                    mma16816(acc2[i], af2[0], b0.x, b0.y);
                    mma16816(acc2[i], af2[1], b0.z, b0.w);
                    mma16816(acc2[i], af2[2], b1.x, b1.y);
                    mma16816(acc2[i], af2[3], b1.z, b1.w);
                }
            }
        }
    }

    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            red[(warp * NACC + i * 4 + c) * 32 + lane] = acc[i][c];
            if (DUAL) red[(warp * NACC + MT * 4 + i * 4 + c) * 32 + lane] = acc2[i][c];
        }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < MT * 4 * 32; idx += blockDim.x) {
        float s = 0.0f, s2 = 0.0f;
        for (uint32_t w = 0; w < nwarps; w++) {
            s += red[w * NACC * 32 + idx];
            if (DUAL) s2 += red[w * NACC * 32 + MT * 4 * 32 + idx];
        }
        const uint32_t ln = idx & 31, c = (idx >> 5) & 3, i = idx >> 7;
        const uint32_t gg = ln >> 2, tt = ln & 3;
        const uint32_t n = nb * 16 + gg + ((c & 2) ? 8 : 0);
        const uint32_t m = m0 + i * 8 + tt * 2 + (c & 1);
        if (m < M) {
            if (DUAL) y[(size_t)m * N + n] = swiglu_chain(s, s2);
            else w4_store(ep, y, m, n, N, s);
        }
    }
}

static uint32_t skinny_kgw(uint32_t KG) {
    uint32_t kgw = 8;
    while ((KG + kgw - 1) / kgw > 20) kgw += 8;
    return kgw;
}

void k_w4a16_skinny(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                    uint16_t* y, uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep) {
    if (!M || !N || !K) return;
    const uint32_t KG = K / 64, kgw = skinny_kgw(KG), nwarps = (KG + kgw - 1) / kgw;
    if (M <= 8) {
        dim3 grid(N / 16, 1);
        size_t smem = (size_t)nwarps * 4 * 32 * sizeof(float);
        if (kgw == 8 && KG % 8 == 0) launch_pdl(w4a16_skinny_kernel<1, 8, false, true>, grid, dim3(nwarps * 32), smem, st, a, (const uint4*)packed, sc, (const uint4*)nullptr, (const uint16_t*)nullptr, y, M, K, N, kgw, ep);
        else launch_pdl(w4a16_skinny_kernel<1, 8, false, false>, grid, dim3(nwarps * 32), smem, st, a, (const uint4*)packed, sc, (const uint4*)nullptr, (const uint16_t*)nullptr, y, M, K, N, kgw, ep);
    } else {
        dim3 grid(N / 16, (M + 15) / 16);
        size_t smem = (size_t)nwarps * 8 * 32 * sizeof(float);
        launch_pdl(w4a16_skinny_kernel<2, 4, false, false>, grid, dim3(nwarps * 32), smem, st, a, (const uint4*)packed, sc, (const uint4*)nullptr, (const uint16_t*)nullptr, y, M, K, N, kgw, ep);
    }
    g_launches++;
}

// y = swiglu(a.Wg, a.Wu): two weight matrices of the same shape in one pass.
void k_w4a16_skinny_swiglu(cudaStream_t st, const uint16_t* a, const uint32_t* pg, const uint16_t* sg,
                           const uint32_t* pu, const uint16_t* su, uint16_t* y, uint32_t M, uint32_t K,
                           uint32_t N) {
    if (!M || !N || !K) return;
    const uint32_t KG = K / 64, kgw = skinny_kgw(KG), nwarps = (KG + kgw - 1) / kgw;
    W4Epilogue ep;
    if (M <= 8) {
        dim3 grid(N / 16, 1);
        size_t smem = (size_t)nwarps * 8 * 32 * sizeof(float);
        launch_pdl(w4a16_skinny_kernel<1, 4, true, false>, grid, dim3(nwarps * 32), smem, st, a, (const uint4*)pg, sg, (const uint4*)pu, su, y, M, K, N, kgw, ep);
    } else {
        dim3 grid(N / 16, (M + 15) / 16);
        size_t smem = (size_t)nwarps * 16 * 32 * sizeof(float);
        launch_pdl(w4a16_skinny_kernel<2, 2, true, false>, grid, dim3(nwarps * 32), smem, st, a, (const uint4*)pg, sg, (const uint4*)pu, su, y, M, K, N, kgw, ep);
    }
    g_launches++;
}

}  // namespace gehtp
