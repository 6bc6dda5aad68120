// fp16 x fp16 -> fp16 matmul (opcodes 24 and 35) on the tensor cores, for weights stored [N, K]
// (flags bit 1, the layout the reference's emitter gives every FullyConnected weight,
// compiler/tools/wtop_ops/op_matmul.cpp:50):
//
//   M >= 128 : TMA-fed tcgen05 GEMM. Both operands are K-major, so a tile of A (128 rows x 64 k) and a
//              tile of W (BN rows x 64 k) land in shared memory by cp.async.bulk.tensor with the 128-byte
//              swizzle that tcgen05.mma reads; accumulators live in TMEM, double-buffered so that the
//              epilogue of a tile overlaps the main loop of the next. The reference takes its matrix
//              unit for the same shapes (exec_matmul_f16_hmx, kernels/src/runtime/oplist_exec.c:1600-1706).
//   M <  32  : streaming GEMV, one warp per output column, 16-byte loads along K, fp32 accumulation,
//              shuffle reduction (exec_matmul_f16_gemv, :1483-1590).
//
// Sums are formed in another order than the reference's ascending-k scalar loop, so results agree with
// it within the fp16 gate, not bit for bit; the engine keeps matmul_f16_exact_kernel (ops_matmul.cu) for
// the one-kernel-per-op plan, for other layouts and for batched operands.
//
//   warp 0 : one lane issues the TMA loads of both operand tiles into a STAGES-deep ring
//   warp 1 : one lane issues tcgen05.mma (4 x k16 per stage and row half) and tcgen05.commit
//   warp 3 : owns the TMEM allocation
//   warps 4-7 : epilogue (tcgen05.ld -> fp16 -> 64-byte row segments)
// All mbarrier waits are bounded; on a timeout the CTA raises the engine's status word, every role
// stops, in-flight copies are waited for (bounded) and the TMEM is freed.
#include <cstdlib>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launchers.h"
#include "sm100_umma.cuh"
#include "w4_stream.cuh"

namespace gehtp {

using namespace sm100;

namespace {

constexpr int BK = 64, HALF_A_BYTES = 128 * BK * 2, NTHREADS = 256, EPI_WARPS = 4, MAX_STAGES = 6;

template <int MH, int BN>
struct FCfg {
    static constexpr int A_BYTES = MH * HALF_A_BYTES, B_BYTES = BN * BK * 2;
    static constexpr int STAGES = (A_BYTES + B_BYTES) <= 32768 ? 6 : ((A_BYTES + B_BYTES) <= 49152 ? 4 : 3);
    static constexpr int NBUF = (MH * BN == 512) ? 1 : 2;
    static constexpr uint32_t ACC_COLS = MH * BN, TMEM_COLS = NBUF * ACC_COLS;
};

struct __align__(8) FBarriers {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base, abort_flag;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) { return (uint32_t)f2h(a) | ((uint32_t)f2h(b) << 16); }

// y rows are ldy elements apart (the SPLIT form writes N columns of a row of N_full).
template <int MH, int BN>
__global__ void __launch_bounds__(NTHREADS, 1)
f16_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                      uint16_t* __restrict__ y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy, unsigned int* status,
                      uint32_t S, float* __restrict__ part) {
    using C = FCfg<MH, BN>;
    constexpr int STAGES = C::STAGES, NBUF = C::NBUF, A_BYTES = C::A_BYTES, B_BYTES = C::B_BYTES;
    constexpr uint32_t ACC_COLS = C::ACC_COLS, TMEM_COLS = C::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = sA + STAGES * A_BYTES;
    FBarriers* bars = (FBarriers*)(sB + STAGES * B_BYTES);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t KG = K / BK;
    const uint32_t m_tiles = (M + 128 * MH - 1) / (128 * MH), tiles = m_tiles * (N / BN);
    // Split K (S > 1): a work item is (tile, run of K/64/S k blocks), item = run * tiles + tile; a run leaves its fp32
    // partial sums in part[run][row][N] and f16_splitk_reduce_kernel adds the runs in order.
    const uint32_t items = tiles * S, KGS = KG / S;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
        for (int s = 0; s < NBUF; s++) { mbar_init(&bars->tmem_full[s], 1); mbar_init(&bars->tmem_empty[s], EPI_WARPS); }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // A (and a weight that is a temp) come from the predecessor
            uint32_t it = 0;
            for (uint32_t item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const uint32_t tile = item % tiles, kb0 = (item / tiles) * KGS;
                const uint32_t m0 = (tile % m_tiles) * (128 * MH), n0 = (tile / m_tiles) * BN;
                for (uint32_t kb = kb0; kb < kb0 + KGS; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&bars->empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                    mbar_expect_tx(&bars->full[s], A_BYTES + B_BYTES);
#pragma unroll
                    for (int h = 0; h < MH; h++)
                        tma_load_2d(sA + s * A_BYTES + h * HALF_A_BYTES, &tmap_a, (int)(kb * BK), (int)(m0 + h * 128), &bars->full[s]);
                    tma_load_2d(sB + s * B_BYTES, &tmap_w, (int)(kb * BK), (int)n0, &bars->full[s]);
                }
            }
            if (*abort_flag)   // copies already requested must land before the CTA may go away
                for (uint32_t j = it > (uint32_t)STAGES ? it - STAGES : 0; j < it; j++) mbar_wait(&bars->full[j % STAGES], (j / STAGES) & 1);
        }
    } else if (warp == 1) {
        // MMA issue. The whole warp walks the loop, so that the loop counters, the descriptors and the barrier
        // addresses are warp-uniform values; lane 0 alone executes the tcgen05 instructions.
        uint32_t it = 0, t = 0;
        const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB);
        bool live = true;
        for (uint32_t item = blockIdx.x; item < items && live; item += gridDim.x, t++) {
            const uint32_t buf = t % NBUF;
            if (!__all_sync(0xffffffffu, mbar_wait_or_abort(&bars->tmem_empty[buf], ((t / NBUF) & 1) ^ 1, abort_flag))) { *abort_flag = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + buf * ACC_COLS;
            for (uint32_t kb = 0; kb < KGS; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait_or_abort(&bars->full[s], ph, abort_flag))) { *abort_flag = 1; live = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da0 = umma_desc(a_base + s * A_BYTES), db0 = umma_desc(b_base + s * B_BYTES);
                if (lane == 0) {
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; k4++) {
#pragma unroll
                        for (int h = 0; h < MH; h++)
                            umma_f16(acc + h * BN, da0 + (uint64_t)(h * (HALF_A_BYTES >> 4) + k4 * 2), db0 + (uint64_t)(k4 * 2), idesc_f16(BN),
                                     (kb | k4) ? 1u : 0u);
                    }
                    umma_commit(&bars->empty[s]);
                }
                __syncwarp();
            }
            if (!live) break;
            if (lane == 0) umma_commit(&bars->tmem_full[buf]);
            __syncwarp();
        }
    } else if (warp >= 4) {
        // epilogue: TMEM lane = output row; a warp may touch lanes (warp % 4) * 32 .. +31
        const uint32_t lane_base = (warp & 3) * 32;
        uint32_t t = 0;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // y may be memory the predecessor still reads
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, t++) {
            const uint32_t buf = t % NBUF;
            const uint32_t tile = item % tiles, run = item / tiles;
            const uint32_t m0 = (tile % m_tiles) * (128 * MH), n0 = (tile / m_tiles) * BN;
            bool ok = !__any_sync(0xffffffffu, *abort_flag != 0);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[buf], (t / NBUF) & 1));
            if (!ok) { *abort_flag = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int h = 0; h < MH; h++) {
                const uint32_t m = m0 + h * 128 + lane_base + lane;
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; c++) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + (lane_base << 16) + buf * ACC_COLS + h * BN + c * 32;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (m < M && S > 1) {
                        uint4* dst = (uint4*)(part + ((size_t)run * M + m) * N + n0 + c * 32);
#pragma unroll
                        for (int q = 0; q < 8; q++) dst[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else if (m < M) {
                        uint4* dst = (uint4*)(y + (size_t)m * ldy + n0 + c * 32);     // 16-byte aligned: y is, ldy is a multiple of 8
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            dst[q] = make_uint4(pack2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                                                pack2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                                                pack2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                                                pack2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 3) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
        if (lane == 0 && *abort_flag) raise_status(status, kStatusGemmTimeout);
    }
}

bool make_map(CUtensorMap* tm, const uint16_t* base, uint32_t rows, uint32_t K, uint32_t box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// y[m][n] (rows ldy apart) = sum over the runs of part[run][m][n], in run order
__global__ void __launch_bounds__(256)
f16_splitk_reduce_kernel(const float* __restrict__ part, uint16_t* __restrict__ y, uint32_t M, uint32_t N, uint32_t ldy, uint32_t S) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t quads = (size_t)M * N / 4, plane = quads;
    const uint32_t nq = N / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < S; r++) {
            const float4 p = __ldcg((const float4*)part + r * plane + i);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        const size_t m = i / nq, n = (i % nq) * 4;
        *(uint2*)(y + m * ldy + n) = make_uint2(pack2(acc.x, acc.y), pack2(acc.z, acc.w));
    }
}

struct SplitScratch { float* part = nullptr; size_t bytes = 0; };

// fp32 partial sums of the split-K form, per device, made on first use and grown when needed (never inside a capture)
SplitScratch* split_scratch(cudaStream_t st, size_t need) {
    static SplitScratch per_dev[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SplitScratch& sc = per_dev[dev];
    if (sc.bytes >= need) return &sc;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return nullptr; }
    cudaDeviceSynchronize();          // a launch in flight may still use the old buffer
    if (sc.part) cudaFree(sc.part);
    sc.part = nullptr; sc.bytes = 0;
    if (cudaMalloc(&sc.part, need) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    sc.bytes = need;
    return &sc;
}

template <int MH, int BN>
bool launch(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy,
            unsigned int* status, int sms) {
    using C = FCfg<MH, BN>;
    CUtensorMap ta, tw;
    if (!make_map(&ta, a, M, K, 128) || !make_map(&tw, w, N, K, BN)) return false;
    const size_t smem = 1024 + (size_t)C::STAGES * (C::A_BYTES + C::B_BYTES) + sizeof(FBarriers) + 16;
    static int have[64] = {};
    if (!ensure_dyn_smem(f16_gemm_sm100_kernel<MH, BN>, smem, have)) return false;
    const uint32_t tiles = ((M + 128 * MH - 1) / (128 * MH)) * (N / BN), KG = K / BK;
    // Split K while the tiles alone leave SMs idle (same rule as the W4A16 GEMM): the divisor of K/64 that makes
    // (items per CTA) x (k blocks per item + set-up) smallest, a run at least one trip round the ring, partial sums <= 64 MB.
    uint32_t S = 1;
    if (tiles < (uint32_t)sms) {
        float best = (float)(KG + 4);
        for (uint32_t c = 2; c <= 32 && c <= KG; c++) {
            if (KG % c || KG / c < (uint32_t)C::STAGES || (size_t)c * M * N * sizeof(float) > ((size_t)64 << 20)) continue;
            const uint32_t rounds = (tiles * c + sms - 1) / sms;
            const float cost = (float)rounds * (float)(KG / c + 4) + 0.75f * (float)c + 6.0f;
            if (cost < best) { best = cost; S = c; }
        }
    }
    float* part = nullptr;
    if (S > 1) {
        SplitScratch* ss = split_scratch(st, (size_t)S * M * N * sizeof(float));
        if (ss) part = ss->part; else S = 1;
    }
    const uint32_t items = tiles * S;
    const uint32_t grid = items < (uint32_t)sms ? items : (uint32_t)sms;
    if (launch_pdl(f16_gemm_sm100_kernel<MH, BN>, dim3(grid), dim3(NTHREADS), smem, st, ta, tw, y, M, K, N, ldy, status, S, part) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    if (S > 1) {
        const size_t quads = (size_t)M * N / 4;
        uint32_t rg = (uint32_t)((quads + 255) / 256);
        if (rg > (uint32_t)sms * 8) rg = (uint32_t)sms * 8;
        if (launch_pdl(f16_splitk_reduce_kernel, dim3(rg), dim3(256), 0, st, (const float*)part, y, M, N, ldy, S) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        g_launches++;
    }
    return true;
}

// ---- streaming GEMV for M < 32. A tile of MR rows of A sits in shared memory; every warp walks
// columns (n = warp, warp + stride, ...), its lanes striding K in 16-byte steps with the loads of up to
// four steps in flight, fp32 accumulation, shuffle reduction.
template <int MR>
__global__ void __launch_bounds__(256)
f16_gemv_nk_kernel(const uint16_t* a, const uint16_t* __restrict__ w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy) {
    extern __shared__ __align__(16) unsigned char smem_a[];      // [MR][K] fp16
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const uint32_t m0 = blockIdx.y * MR, K8 = K / 8;
    uint4* sa = (uint4*)smem_a;
    for (uint32_t i = threadIdx.x; i < MR * K8; i += blockDim.x) {
        const uint32_t r = i / K8, m = min(m0 + r, M - 1);       // rows past M repeat row M-1; never stored
        sa[i] = __ldcg((const uint4*)(a + (size_t)m * K) + (i % K8));
    }
    __syncthreads();
    for (uint32_t n = blockIdx.x * nw + warp; n < N; n += gridDim.x * nw) {
        const uint4* wr = (const uint4*)(w + (size_t)n * K);
        float acc[MR];
#pragma unroll
        for (int r = 0; r < MR; r++) acc[r] = 0.0f;
        for (uint32_t i0 = lane; i0 < K8; i0 += 128) {
            uint4 wq[4];
#pragma unroll
            for (int u = 0; u < 4; u++) wq[u] = i0 + 32 * u < K8 ? __ldcs(wr + i0 + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t i = i0 + 32 * u;
                if (i >= K8) break;
                const __half2* wh = (const __half2*)&wq[u];
#pragma unroll
                for (int r = 0; r < MR; r++) {
                    const uint4 aq = sa[r * K8 + i];
                    const __half2* ah = (const __half2*)&aq;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 wf = __half22float2(wh[j]), af = __half22float2(ah[j]);
                        acc[r] = fmaf(af.x, wf.x, acc[r]);
                        acc[r] = fmaf(af.y, wf.y, acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MR; r++) {
            const float sum = warp_sum(acc[r]);
            if (lane == 0 && m0 + r < M) y[(size_t)(m0 + r) * ldy + n] = f2h(sum);
        }
    }
}

// ---- the same on the tensor cores (mma.sync m16n8k16) for up to 8 rows per CTA row tile: a warp owns 8 output
// columns and walks K in chunks of 32. Lane (g, t) loads 16 bytes of weight row n0 + g (8 consecutive k values)
// and the 16 bytes at the same k of activation row g from shared memory; the first and the second half of those
// 8 values feed two MMAs. Which of the 16 k slots of an MMA a value takes does not matter as long as A and B
// agree, so no shuffling into the fragment order is needed: one 16-byte load per operand and chunk, 2 MMAs,
// where the scalar form above spends some 140 instructions on the same 8 weights at 8 rows.
// The first batch of weights (constants) is requested before the dependency wait.
template <int UNR>
__global__ void __launch_bounds__(256)
f16_gemv_mma_kernel(const uint16_t* a, const uint16_t* __restrict__ w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy) {
    extern __shared__ __align__(16) unsigned char smem_a[];      // [8][K * 2 + 64] bytes: rows 64 bytes apart in the banks
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t m0 = blockIdx.y * 8, n0 = (blockIdx.x * 8 + warp) * 8, KC = K / 32, RS = K * 2 + 64;
    const bool active = n0 < N;
    const uint4* wr = (const uint4*)(w + (size_t)min(n0 + g, N - 1) * K) + t;      // chunk kc lies 4 * kc further
    uint4 wq[UNR];
#pragma unroll
    for (int u = 0; u < UNR; u++) wq[u] = (active && (uint32_t)u < KC) ? __ldcs(wr + 4 * u) : make_uint4(0, 0, 0, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = threadIdx.x; i < 8 * (K / 8); i += blockDim.x) {
        const uint32_t r = i / (K / 8), c = i % (K / 8), m = min(m0 + r, M - 1);       // rows past M repeat row M-1; never stored
        *(uint4*)(smem_a + r * RS + c * 16) = __ldcg((const uint4*)(a + (size_t)m * K) + c);
    }
    __syncthreads();
    if (!active) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned char* arow = smem_a + g * RS + t * 16;
    for (uint32_t kc0 = 0; kc0 < KC; kc0 += UNR) {
        uint4 nx[UNR];
#pragma unroll
        for (int u = 0; u < UNR; u++) nx[u] = kc0 + UNR + u < KC ? __ldcs(wr + 4 * (kc0 + UNR + u)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            if (kc0 + u >= KC) break;
            const uint4 av = *(const uint4*)(arow + (kc0 + u) * 64);
            const uint32_t a1[4] = {av.x, 0u, av.y, 0u}, a2[4] = {av.z, 0u, av.w, 0u};    // rows g + 8 of the tile: none
            mma16816(acc, a1, wq[u].x, wq[u].y);
            mma16816(acc, a2, wq[u].z, wq[u].w);
        }
#pragma unroll
        for (int u = 0; u < UNR; u++) wq[u] = nx[u];
    }
    const uint32_t m = m0 + g, n = n0 + 2 * t;
    if (m < M) {
        if (n < N) y[(size_t)m * ldy + n] = f2h(acc[0]);
        if (n + 1 < N) y[(size_t)m * ldy + n + 1] = f2h(acc[1]);
    }
}

bool launch_gemv_mma(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy) {
    const size_t smem = (size_t)8 * (K * 2 + 64);
    static int have[64] = {};
    if (K % 32 || smem > 200 * 1024 || (smem > 48 * 1024 && !ensure_dyn_smem(f16_gemv_mma_kernel<8>, smem, have))) return false;
    if (launch_pdl(f16_gemv_mma_kernel<8>, dim3((N + 63) / 64, (M + 7) / 8), dim3(256), smem, st, a, w, y, M, K, N, ldy) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    return true;
}

template <int MR>
bool launch_gemv(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, uint32_t ldy) {
    const size_t smem = (size_t)MR * K * 2;
    static int have[64] = {};
    if (smem > 200 * 1024 || (smem > 48 * 1024 && !ensure_dyn_smem(f16_gemv_nk_kernel<MR>, smem, have))) return false;
    uint32_t gx = (N + 7) / 8;
    if (gx > 148 * 4) gx = 148 * 4;
    if (launch_pdl(f16_gemv_nk_kernel<MR>, dim3(gx, (M + MR - 1) / MR), dim3(256), smem, st, a, w, y, M, K, N, ldy) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    return true;
}

}  // namespace

// Y[M, N] (rows ldy apart) = A[M, K] . W^T, W stored [N, K]. false: shape or alignment outside what the
// tensor-core forms take (the caller then runs the exact kernel); nothing launched.
bool k_matmul_f16_nk(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K, uint32_t N,
                     uint32_t ldy, unsigned int* status) {
    if (!M || !K || !N || (K & 7u) || ((((uintptr_t)a) | ((uintptr_t)w)) & 15u)) return false;
    if (M < 32) {
        static const int mma_on = [] { const char* e = std::getenv("GEHTP_CUDA_F16_GEMV_MMA"); return e ? std::atoi(e) : 1; }();
        if (mma_on && launch_gemv_mma(st, a, w, y, M, K, N, ldy)) return true;
        return M <= 4 ? launch_gemv<4>(st, a, w, y, M, K, N, ldy) : launch_gemv<8>(st, a, w, y, M, K, N, ldy);
    }
    if (M < 128 || K % BK || N % 128 || (ldy & 7u) || ((uintptr_t)y & 15u)) return false;
    static int sms_of[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int& sms = sms_of[dev & 63];
    if (!sms) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const uint32_t t256 = ((M + 255) / 256) * (N / 256), t128 = ((M + 255) / 256) * (N / 128);
    if (N % 256 == 0 && M > 128 && t256 >= (uint32_t)sms) return launch<2, 256>(st, a, w, y, M, K, N, ldy, status, sms);
    if (M > 128 && t128 >= (uint32_t)sms) return launch<2, 128>(st, a, w, y, M, K, N, ldy, status, sms);
    return launch<1, 128>(st, a, w, y, M, K, N, ldy, status, sms);
}

}  // namespace gehtp
