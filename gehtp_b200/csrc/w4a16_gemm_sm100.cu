// W4A16 group-64 GEMM for prefill (M >= 128) on the 5th-generation tensor cores:
// Y[M,N] = A[M,K] . W, W = fp16((q-8)*scale), fp32 accumulation in TMEM.
//
// One CTA computes a 128 x 128 tile of Y; K is walked in steps of 64 (one
// scale group, one 128-byte swizzled row per operand row).
//   warp 0    : one lane issues the TMA loads of the A tile (128 rows x 64 k,
//               SWIZZLE_128B) into a 4-stage ring; the warp also owns the TMEM
//               allocation.
//   warps 1-4 : dequant producers. The int4 tile of a stage (8 strip units of
//               512 B in the strip-major layout) is prefetched PRE stages ahead
//               with cp.async into per-lane slots, turned into fp16 with the
//               magic-number trick, multiplied by the group scale and stored as
//               16-byte chunks into the stage's B tile in the 128B-swizzled
//               K-major form tcgen05.mma reads. The same warps run the epilogue
//               (tcgen05.ld -> fp16 -> global).
//   warp 5    : one lane issues tcgen05.mma (4 x k16 per stage, M128 N128) and
//               tcgen05.commit, which frees the stage when the MMAs have read it.
// All mbarrier waits are bounded; on a timeout the CTA raises a status word,
// stops issuing, and still frees its TMEM.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launchers_w4.h"

namespace gehtp {

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 4;          // A/B operand ring
constexpr int PRE = 8;             // int4 prefetch depth (stages of K)
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr uint32_t SPIN_LIMIT = 2u * 1000u * 1000u;   // try_wait polls before a role gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded wait; false = gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}

// instruction descriptor, kind::f16: A,B fp16 K-major, D fp32, M128 N128
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}

// 8 nibbles of one packed word -> 4 fp16 pairs (q-8)*scale: lo pairs belong to column g, hi pairs to g+8
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 slo, __half2 shi, uint32_t (&o)[4]) {
    const uint32_t MAGIC = 0x64006400u;
    const __half2 c1032 = __half2half2(__ushort_as_half(0x6408));
    const __half2 c16th = __half2half2(__ushort_as_half(0x2c00));
    const __half2 cm72 = __half2half2(__ushort_as_half(0xd480));
    uint32_t w8 = w >> 8;
    uint32_t p0 = (w & 0x000f000fu) | MAGIC, p1 = (w & 0x00f000f0u) | MAGIC;
    uint32_t p2 = (w8 & 0x000f000fu) | MAGIC, p3 = (w8 & 0x00f000f0u) | MAGIC;
    __half2 h0 = __hmul2(__hsub2(*(__half2*)&p0, c1032), slo);           // col g,   k+0,k+1
    __half2 h1 = __hmul2(__hfma2(*(__half2*)&p1, c16th, cm72), shi);     // col g+8, k+0,k+1
    __half2 h2 = __hmul2(__hsub2(*(__half2*)&p2, c1032), slo);           // col g,   k+2,k+3
    __half2 h3 = __hmul2(__hfma2(*(__half2*)&p3, c16th, cm72), shi);     // col g+8, k+2,k+3
    o[0] = *(uint32_t*)&h0; o[1] = *(uint32_t*)&h1; o[2] = *(uint32_t*)&h2; o[3] = *(uint32_t*)&h3;
}

struct __align__(8) Barriers {
    uint64_t full_a[STAGES], full_b[STAGES], empty[STAGES], accum;
    uint32_t tmem_base, abort_flag;
};

__device__ unsigned int g_w4gemm_timeouts = 0;   // CTAs that gave up on a barrier

__global__ void __launch_bounds__(192, 1)
w4a16_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint4* __restrict__ wp,
                        const uint16_t* __restrict__ sc, uint16_t* __restrict__ y, uint32_t M, uint32_t K,
                        uint32_t N, W4Epilogue ep) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t KG = K / BK, NB = N / 16;
    unsigned char* sA = smem;
    unsigned char* sB = sA + STAGES * A_BYTES;
    uint4* sRaw = (uint4*)(sB + STAGES * B_BYTES);                  // [PRE][128 threads][2]
    uint16_t* sScale = (uint16_t*)((unsigned char*)sRaw + PRE * 128 * 2 * 16);   // [KG][128]
    Barriers* bars = (Barriers*)(((uintptr_t)(sScale + (size_t)KG * BN) + 15) & ~(uintptr_t)15);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&bars->full_a[s], 1); mbar_init(&bars->full_b[s], 4); mbar_init(&bars->empty[s], 1); }
        mbar_init(&bars->accum, 1);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // group scales of this column tile, all k groups
    for (uint32_t e = threadIdx.x; e < KG * (BN / 8); e += blockDim.x) {
        uint32_t kg = e / (BN / 8), c = e % (BN / 8);
        ((uint4*)sScale)[e] = __ldg((const uint4*)(sc + (size_t)kg * N + n0) + c);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t kb = 0; kb < KG && !*abort_flag; kb++) {
                uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1;
                if (!mbar_wait(&bars->empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                mbar_expect_tx(&bars->full_a[s], A_BYTES);
                tma_load_2d(sA + s * A_BYTES, &tmap_a, (int)(kb * BK), (int)m0, &bars->full_a[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            for (uint32_t kb = 0; kb < KG && !*abort_flag; kb++) {
                uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1;
                if (!mbar_wait(&bars->full_a[s], ph) || !mbar_wait(&bars->full_b[s], ph)) { *abort_flag = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t a0 = smem_u32(sA + s * A_BYTES), b0 = smem_u32(sB + s * B_BYTES);
#pragma unroll
                for (uint32_t k4 = 0; k4 < BK / 16; k4++)
                    umma_f16(tmem, umma_desc(a0 + k4 * 32), umma_desc(b0 + k4 * 32), (kb | k4) ? 1u : 0u);
                umma_commit(&bars->empty[s]);
            }
            umma_commit(&bars->accum);
        }
    } else {
        // ---- dequant producers (128 threads), then epilogue
        const uint32_t dw = warp - 1, dt = dw * 32 + lane, g = lane >> 2, t = lane & 3;
        const uint4* src0 = wp + ((size_t)(n0 / 16) + dw * 2) * 32 + lane;     // unit dw*2, k group 0
        auto prefetch = [&](uint32_t kb) {
            if (kb < KG) {
                const uint4* s0 = src0 + (size_t)kb * NB * 32;
                uint4* dst = sRaw + ((size_t)(kb % PRE) * 128 + dt) * 2;
                cp_async16(dst, s0);
                cp_async16(dst + 1, s0 + 32);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (uint32_t kb = 0; kb < PRE; kb++) prefetch(kb);
        for (uint32_t kb = 0; kb < KG; kb++) {
            uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1;
            asm volatile("cp.async.wait_group %0;" ::"n"(PRE - 1) : "memory");
            uint4 raw[2];
            raw[0] = sRaw[((size_t)(kb % PRE) * 128 + dt) * 2];
            raw[1] = sRaw[((size_t)(kb % PRE) * 128 + dt) * 2 + 1];
            prefetch(kb + PRE);
            // warp-uniform decisions: every lane polls, the warp leaves together
            if (__any_sync(0xffffffffu, *abort_flag != 0)) break;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->empty[s], ph ^ 1))) { *abort_flag = 1; break; }
            unsigned char* bt = sB + s * B_BYTES;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const uint32_t col = (dw * 2 + u) * 16 + g;
                const __half2 slo = __half2half2(__ushort_as_half(sScale[kb * BN + col]));
                const __half2 shi = __half2half2(__ushort_as_half(sScale[kb * BN + col + 8]));
                uint32_t o[4][4];
                dequant_word(raw[u].x, slo, shi, o[0]);
                dequant_word(raw[u].y, slo, shi, o[1]);
                dequant_word(raw[u].z, slo, shi, o[2]);
                dequant_word(raw[u].w, slo, shi, o[3]);
                const uint32_t r0 = col, r1 = col + 8;
                // row r, 16-byte chunk c (8 k) lives at r*128 + ((c ^ (r & 7)) << 4)
                *(uint4*)(bt + r0 * 128 + (((2 * t) ^ (r0 & 7)) << 4)) = make_uint4(o[0][0], o[0][2], o[1][0], o[1][2]);
                *(uint4*)(bt + r0 * 128 + (((2 * t + 1) ^ (r0 & 7)) << 4)) = make_uint4(o[2][0], o[2][2], o[3][0], o[3][2]);
                *(uint4*)(bt + r1 * 128 + (((2 * t) ^ (r1 & 7)) << 4)) = make_uint4(o[0][1], o[0][3], o[1][1], o[1][3]);
                *(uint4*)(bt + r1 * 128 + (((2 * t + 1) ^ (r1 & 7)) << 4)) = make_uint4(o[2][1], o[2][3], o[3][1], o[3][3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->full_b[s]);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");

        // ---- epilogue: TMEM lane = output row; a warp may touch lanes (warp % 4) * 32 .. +31
        bool ok = !__any_sync(0xffffffffu, *abort_flag != 0);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->accum, 0));
        if (!ok) *abort_flag = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const uint32_t lane_base = (warp & 3) * 32;
            const uint32_t m = m0 + lane_base + lane;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                const uint32_t taddr = tmem + (lane_base << 16) + c * 32;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m < M) {
#pragma unroll
                    for (int i = 0; i < 32; i++) w4_store(ep, y, m, n0 + c * 32 + i, N, __uint_as_float(v[i]));
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
        if (lane == 0 && *abort_flag) atomicAdd(&g_w4gemm_timeouts, 1u);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

}  // namespace

unsigned int w4a16_gemm_timeouts() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_w4gemm_timeouts, sizeof v);
    return v;
}

bool k_w4a16_gemm_sm100(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                        uint16_t* y, uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep) {
    if (!M || K % BK || N % BN || ((uintptr_t)a & 15)) return false;
    const uint32_t KG = K / BK;
    size_t smem = 1024 + (size_t)STAGES * (A_BYTES + B_BYTES) + (size_t)PRE * 128 * 2 * 16 + (size_t)KG * BN * 2 + 16 + sizeof(Barriers);
    if (smem > 227 * 1024) return false;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    CUtensorMap tmap;
    cuuint64_t dims[2] = {K, M};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {BK, BM};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    static size_t attr = 0;
    if (attr < smem) {
        if (cudaFuncSetAttribute(w4a16_gemm_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        attr = smem;
    }
    dim3 grid(N / BN, (M + BM - 1) / BM);
    w4a16_gemm_sm100_kernel<<<grid, 192, smem, st>>>(tmap, (const uint4*)packed, sc, y, M, K, N, ep);
    g_launches++;
    return true;
}

}  // namespace gehtp
