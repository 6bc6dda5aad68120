// W4A16 group-64 GEMM from 64 rows up (prefill, wide decode batches) on the 5th-generation tensor cores:
// Y[M,N] = A[M,K] . W, W = fp16((q-8)*scale), fp32 accumulation in TMEM.
//
// Persistent kernel, one CTA per SM. A CTA walks output tiles of (128*MH) x BN (MH = 1 or 2 row halves sharing
// one dequantised B tile, BN = 128 or 256 columns); K is walked in steps of 64 (one scale group, one 128-byte
// swizzled row per operand row).
//   warp 0     : one lane issues the TMA loads of the A tile (MH boxes of 128 rows x 64 k, SWIZZLE_128B) into a
//                STAGES-deep ring. A is [M][K], or [K / d][M][d] read through a three-dimensional map (the
//                output of a per-head kernel, without a transposed copy).
//   warp 1     : walks the k loop as a whole warp (uniform counters and descriptors); one lane issues
//                tcgen05.mma (4 x k16 x MH per stage, M128 x BN) and tcgen05.commit, which frees the stage
//                when the MMAs have read it. The accumulators are double-buffered in TMEM (except 256 x 256)
//                so that the epilogue of a tile overlaps the main loop of the next one.
//   warp 2     : one lane streams the int4 tile of each k block (BN / 16 strip units, contiguous in the
//                strip-major layout) and its BN group scales with bulk copies into an RSTAGES-deep ring.
//   warp 3     : owns the TMEM allocation.
//   warps 4-7  : epilogue (tcgen05.ld -> fp16 -> row segments).
//   warps 8-23 : dequant, one group of four warps per operand stage (the 3-stage configurations have no stage
//                for warps 20-23: idle, or epilogue helpers in the gate | up form). A warp turns its strip units
//                into fp16 with the magic-number trick, multiplies by the group scale and stores 16-byte chunks
//                into the stage's B tile in the 128B-swizzled K-major form tcgen05.mma reads.
// Gate | up form (DUAL): the B tile holds 128 columns of two matrices, the epilogue writes their SwiGLU product.
// Few-tile shapes (prefill projections with N = 1024, decode at 64 rows): K is cut into S runs, one work item per
// (tile, run); a run writes its fp32 partial sums and w4a16_splitk_reduce_kernel adds the runs in order (same bits
// on every call) and applies the epilogue - or, where a residual ADD and an RMSNORM2 follow the matmul,
// w4a16_splitk_add_rmsnorm_kernel adds the runs, the residual, and normalises. 512 x 3072 x 1024: 22.9 -> 12.4 us.
// All mbarrier waits are bounded; on a timeout the CTA raises a flag, every role
// stops, in-flight copies are waited for (bounded), and the TMEM is freed.
#include <cstdlib>
#include <initializer_list>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launchers_w4.h"
#include "sm100_umma.cuh"
#include "w4_stream.cuh"
#include "norm_row.cuh"

namespace gehtp {

using namespace sm100;

namespace {

constexpr int BK = 64;
constexpr int MAX_STAGES = 4;      // A/B operand ring (depth per configuration below)
constexpr int RSTAGES_MAX = 4;     // int4 + scale ring
constexpr int HALF_A_BYTES = 128 * BK * 2;
constexpr int NTHREADS = 768;
constexpr int DQ_PER_STAGE = 4, EPI_WARPS = 4;   // 16 dequant warps, 4 of them per k block

// Tile configuration: MH row halves of 128 x BN columns per tile.
//   <1,128>: 128x128, 4 stages, two accumulator buffers   (small M, or N not a multiple of 256)
//   <2,128>: 256x128, 4 stages, two accumulator buffers
//   <2,256>: 256x256, 3 stages, one accumulator buffer (all 512 TMEM columns): per FLOP it reads
//            45 % fewer operand bytes from L2 and a third fewer from shared memory than 256x128;
//            the epilogue is not overlapped (a few % of a K >= 2048 main loop).
//   <1,256>: 128x256, 3 stages, two accumulator buffers: the gate | up form (DUAL) at few rows.
// DUAL (BN = 256 only): the B tile of a k block holds 128 columns of a first weight matrix (gate) and the same 128
// columns of a second one (up); one N = 256 instruction feeds both accumulators and the epilogue writes
// fp16(fp16(gate * fp16(sigmoid(gate))) * up), 128 output columns per tile: the two projections of a gated FFN and
// the three elementwise ops behind them in one launch, neither projection's output going through memory.
template <int MH, int BN>
struct Cfg {
    static constexpr int STAGES = BN == 256 ? 3 : 4;
    static constexpr int NBUF = (MH * BN == 512) ? 1 : 2;
    // One dequant group (4 warps) per operand stage, and one int4/scale slot per group: group q only
    // ever waits on stage q and slot q, so it sees every phase of those barriers in turn. (A parity
    // wait is only sound when the waiter has seen the phase before the one it waits for.)
    static constexpr int GROUPS = STAGES;
    static constexpr int RSTAGES = STAGES;
    static constexpr int A_BYTES = MH * HALF_A_BYTES, B_BYTES = BN * BK * 2;
    static constexpr int RAW_BYTES = BN * BK / 2, RAW_SLOT = RAW_BYTES + BN * 2;   // nibbles + BN fp16 scales
    static constexpr uint32_t ACC_COLS = MH * BN;             // TMEM columns of one accumulator buffer
    static constexpr uint32_t TMEM_COLS = NBUF * ACC_COLS;    // 256 or 512: a power of two
    // instruction descriptor, kind::f16: A,B fp16 K-major, D fp32, M128 x N = BN
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
};

// 8 nibbles of one packed word -> 4 fp16 pairs (q-8)*scale: lo pairs belong to column g, hi pairs to g+8
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 slo, __half2 shi, uint32_t (&o)[4]) {
    const uint32_t MAGIC = 0x64006400u;
    const __half2 c1032 = __half2half2(__ushort_as_half(0x6408));
    const __half2 c16th = __half2half2(__ushort_as_half(0x2c00));
    const __half2 cm72 = __half2half2(__ushort_as_half(0xd480));
    const uint32_t w8 = w >> 8;
    const uint32_t p0 = and_or(w, 0x000f000fu, MAGIC), p1 = and_or(w, 0x00f000f0u, MAGIC);
    const uint32_t p2 = and_or(w8, 0x000f000fu, MAGIC), p3 = and_or(w8, 0x00f000f0u, MAGIC);
    __half2 h0 = __hmul2(__hsub2(*(const __half2*)&p0, c1032), slo);           // col g,   k+0,k+1
    __half2 h1 = __hmul2(__hfma2(*(const __half2*)&p1, c16th, cm72), shi);     // col g+8, k+0,k+1
    __half2 h2 = __hmul2(__hsub2(*(const __half2*)&p2, c1032), slo);           // col g,   k+2,k+3
    __half2 h3 = __hmul2(__hfma2(*(const __half2*)&p3, c16th, cm72), shi);     // col g+8, k+2,k+3
    o[0] = *(uint32_t*)&h0; o[1] = *(uint32_t*)&h1; o[2] = *(uint32_t*)&h2; o[3] = *(uint32_t*)&h3;
}

struct __align__(8) Barriers {
    // full: one phase per k block, completed by the TMA bytes of the A tile (one expect_tx arrival) and the
    // arrivals of the four dequant warps that wrote the B tile - the MMA lane polls a single barrier per k block
    uint64_t full[MAX_STAGES], empty[MAX_STAGES];
    uint64_t raw_full[RSTAGES_MAX], raw_empty[RSTAGES_MAX];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base, abort_flag;
};

// fp32 pair -> packed fp16 pair with the executor's NaN rule (NaN -> signed infinity)
__device__ __forceinline__ uint32_t pack_out(float a, float b) {
    return (uint32_t)f2h(a) | ((uint32_t)f2h(b) << 16);
}
__device__ __forceinline__ uint32_t pack_out_res(float a, float b, uint32_t res) {
    const float ra = h2f((uint16_t)(res & 0xffffu)), rb = h2f((uint16_t)(res >> 16));
    return (uint32_t)f2h(__fadd_rn(h2f(f2h(a)), ra)) | ((uint32_t)f2h(__fadd_rn(h2f(f2h(b)), rb)) << 16);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

template <int MH, int BN, bool DUAL = false>
__global__ void __launch_bounds__(NTHREADS, 1)
w4a16_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint4* __restrict__ wp,
                        const uint16_t* __restrict__ sc, const uint4* __restrict__ wp2, const uint16_t* __restrict__ sc2,
                        uint16_t* __restrict__ y, uint32_t M, uint32_t K,
                        uint32_t N, W4Epilogue ep, uint32_t S, float* __restrict__ part, uint32_t a_d) {
    using C = Cfg<MH, BN>;
    static_assert(!DUAL || BN == 256, "the gate | up form pairs two 128-column halves");
    static_assert(!DUAL || C::GROUPS == 3, "warps 20-23 help the epilogue of the gate | up form: they must own no operand stage");
    constexpr uint32_t BN_OUT = DUAL ? BN / 2 : BN;      // output (and weight) columns of one tile
    constexpr int STAGES = C::STAGES, RSTAGES = C::RSTAGES, NBUF = C::NBUF;
    constexpr int A_BYTES = C::A_BYTES, B_BYTES = C::B_BYTES, RAW_BYTES = C::RAW_BYTES, RAW_SLOT = C::RAW_SLOT;
    constexpr uint32_t ACC_COLS = C::ACC_COLS, TMEM_COLS = C::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t KG = K / BK, NB = N / 16;
    unsigned char* sA = smem;
    unsigned char* sB = sA + STAGES * A_BYTES;
    unsigned char* sRaw = sB + STAGES * B_BYTES;                    // [RSTAGES][RAW_SLOT]
    Barriers* bars = (Barriers*)(sRaw + RSTAGES * RAW_SLOT);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    // Programmatic dependent launch: the set-up below, the weight copies and the dequantisation
    // of the first k blocks (constants, independent of the predecessor) run while the predecessor
    // drains; only the A loads and the epilogue's global accesses order themselves after it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (M + 128 * MH - 1) / (128 * MH), n_tiles = N / BN_OUT;
    const uint32_t tiles = m_tiles * n_tiles;
    // Split K: S > 1 cuts the k blocks of every tile into S runs, one work item each (item = run * tiles + tile);
    // a run leaves its fp32 partial sums in `part` ([run][row][N]) and a small kernel behind this one adds the
    // runs in order and writes y. Few-tile shapes so fill the SMs instead of walking a long K in a few CTAs.
    const uint32_t items = tiles * S, KGS = KG / S;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&bars->full[s], 1 + DQ_PER_STAGE);
            mbar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < RSTAGES; s++) { mbar_init(&bars->raw_full[s], 1); mbar_init(&bars->raw_empty[s], DQ_PER_STAGE); }
        for (int s = 0; s < NBUF; s++) { mbar_init(&bars->tmem_full[s], 1); mbar_init(&bars->tmem_empty[s], DUAL ? 2 * EPI_WARPS : EPI_WARPS); }
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
        // ---- A tiles by TMA
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // A is the predecessor's output
            uint32_t it = 0;
            for (uint32_t item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const uint32_t tile = item % tiles, kb0 = (item / tiles) * KGS;
                const uint32_t m0 = (tile % m_tiles) * (128 * MH);
                for (uint32_t kb = kb0; kb < kb0 + KGS; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&bars->empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                    mbar_expect_tx(&bars->full[s], A_BYTES);
#pragma unroll
                    for (int h = 0; h < MH; h++)
                        if (a_d)     // A stored [head][row][a_d]: column kb * 64 of A is column (kb * 64) % a_d of head (kb * 64) / a_d
                            tma_load_3d(sA + s * A_BYTES + h * HALF_A_BYTES, &tmap_a, (int)((kb * BK) % a_d), (int)(m0 + h * 128), (int)((kb * BK) / a_d),
                                        &bars->full[s]);
                        else
                            tma_load_2d(sA + s * A_BYTES + h * HALF_A_BYTES, &tmap_a, (int)(kb * BK), (int)(m0 + h * 128), &bars->full[s]);
                }
            }
            if (*abort_flag)   // copies already requested must land before the CTA may go away
                for (uint32_t j = it > (uint32_t)STAGES ? it - STAGES : 0; j < it; j++) mbar_wait(&bars->full[j % STAGES], (j / STAGES) & 1);
        }
    } else if (warp == 1) {
        // ---- MMA issue. The whole warp walks the loop, so that the loop counters, the descriptors and the barrier
        // addresses are warp-uniform values; lane 0 alone executes the tcgen05 instructions.
        uint32_t t = 0, s = 0, ph = 0;          // operand stage and phase parity of the k block in hand
        // descriptors of stage 0's first K16 slice; a stage lies A_BYTES / B_BYTES further, a K16 slice 32 bytes
        // (the start-address field counts 16-byte units), the second row half HALF_A_BYTES
        const uint64_t da_base = umma_desc(smem_u32(sA)), db_base = umma_desc(smem_u32(sB));
        bool live = true;
        for (uint32_t item = blockIdx.x; item < items && live; item += gridDim.x, t++) {
            const uint32_t buf = t % NBUF;
            if (!__all_sync(0xffffffffu, mbar_wait_or_abort(&bars->tmem_empty[buf], ((t / NBUF) & 1) ^ 1, abort_flag))) { *abort_flag = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + buf * ACC_COLS;
            for (uint32_t kb = 0; kb < KGS; kb++) {
                if (!__all_sync(0xffffffffu, mbar_wait_or_abort(&bars->full[s], ph, abort_flag))) { *abort_flag = 1; live = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da0 = da_base + (uint64_t)(s * (A_BYTES >> 4)), db0 = db_base + (uint64_t)(s * (B_BYTES >> 4));
                if (lane == 0) {
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; k4++) {
#pragma unroll
                        for (int h = 0; h < MH; h++)
                            umma_f16(acc + h * BN, da0 + (uint64_t)(h * (HALF_A_BYTES >> 4) + k4 * 2), db0 + (uint64_t)(k4 * 2), C::IDESC,
                                     (kb | k4) ? 1u : 0u);
                    }
                    umma_commit(&bars->empty[s]);
                }
                __syncwarp();
                if (++s == (uint32_t)STAGES) { s = 0; ph ^= 1u; }
            }
            if (!live) break;
            if (lane == 0) umma_commit(&bars->tmem_full[buf]);
            __syncwarp();
        }
    } else if (warp == 2) {
        // ---- int4 tiles and scales by bulk copy
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
                const uint32_t tile = item % tiles, kb0 = (item / tiles) * KGS;
                const uint32_t n0 = (tile / m_tiles) * BN_OUT;
                const uint4* wsrc = wp + (size_t)(n0 / 16) * 32;
                const uint16_t* ssrc = sc + n0;
                const uint4* wsrc2 = DUAL ? wp2 + (size_t)(n0 / 16) * 32 : nullptr;
                const uint16_t* ssrc2 = DUAL ? sc2 + n0 : nullptr;
                for (uint32_t kb = kb0; kb < kb0 + KGS; kb++, it++) {
                    const uint32_t r = it % RSTAGES, ph = (it / RSTAGES) & 1;
                    if (*abort_flag || !mbar_wait(&bars->raw_empty[r], ph ^ 1)) { *abort_flag = 1; break; }
                    unsigned char* dst = sRaw + r * RAW_SLOT;
                    mbar_expect_tx(&bars->raw_full[r], RAW_SLOT);
                    if (DUAL) {      // strip units 0-7 and scales 0-127 from the first matrix, the rest from the second
                        bulk_load(dst, wsrc + (size_t)kb * NB * 32, RAW_BYTES / 2, &bars->raw_full[r]);
                        bulk_load(dst + RAW_BYTES / 2, wsrc2 + (size_t)kb * NB * 32, RAW_BYTES / 2, &bars->raw_full[r]);
                        bulk_load(dst + RAW_BYTES, ssrc + (size_t)kb * N, BN_OUT * 2, &bars->raw_full[r]);
                        bulk_load(dst + RAW_BYTES + BN_OUT * 2, ssrc2 + (size_t)kb * N, BN_OUT * 2, &bars->raw_full[r]);
                    } else {
                        bulk_load(dst, wsrc + (size_t)kb * NB * 32, RAW_BYTES, &bars->raw_full[r]);
                        bulk_load(dst + RAW_BYTES, ssrc + (size_t)kb * N, BN * 2, &bars->raw_full[r]);
                    }
                }
            }
            if (*abort_flag)
                for (uint32_t j = it > (uint32_t)RSTAGES ? it - RSTAGES : 0; j < it; j++) mbar_wait(&bars->raw_full[j % RSTAGES], (j / RSTAGES) & 1);
        }
    } else if ((warp >= 4 && warp < 8) || (DUAL && warp >= 20)) {
        // ---- epilogue: TMEM lane = output row; a warp may touch lanes (warp % 4) * 32 .. +31. The gate | up form
        // (three operand stages: dequant warps 20-23 have no stage) gives those four warps every second column chunk.
        const uint32_t lane_base = (warp & 3) * 32;
        const uint32_t chunk0 = (DUAL && warp >= 20) ? 1 : 0;
        uint32_t t = 0;
        // y (and the residual) may be memory the predecessor still reads or writes
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // 32 accumulator values of row m from column n on their way to y
        auto emit = [&](uint32_t m, uint32_t n, const uint32_t (&v)[32]) {
            const size_t o = (size_t)m * N + n;       // 64-byte aligned: N and n are multiples of 32
            uint4* dst = (uint4*)(y + o);
            if (ep.mode == 1) {
                const uint4* res = (const uint4*)(ep.res + o);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 r = res[q];
                    dst[q] = make_uint4(pack_out_res(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1]), r.x),
                                        pack_out_res(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]), r.y),
                                        pack_out_res(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]), r.z),
                                        pack_out_res(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]), r.w));
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; q++)
                    dst[q] = make_uint4(pack_out(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                                        pack_out(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                                        pack_out(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                                        pack_out(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
            }
        };
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, t++) {
            const uint32_t buf = t % NBUF;
            const uint32_t tile = item % tiles, run = item / tiles;
            const uint32_t m0 = (tile % m_tiles) * (128 * MH), n0 = (tile / m_tiles) * BN_OUT;
            bool ok = !__any_sync(0xffffffffu, *abort_flag != 0);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->tmem_full[buf], (t / NBUF) & 1));
            if (!ok) { *abort_flag = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int h = 0; h < MH; h++) {
                const uint32_t m = m0 + h * 128 + lane_base + lane;
                if (DUAL) {
                    // gate in accumulator columns 0-127, up in 128-255: 16 columns of each at a time
#pragma unroll 1
                    for (uint32_t c = chunk0; c < BN_OUT / 16; c += 2) {
                        uint32_t vg[16], vu[16];
                        const uint32_t taddr = tmem + (lane_base << 16) + buf * ACC_COLS + h * BN + c * 16;
                        tmem_ld16(taddr, vg);
                        tmem_ld16(taddr + BN_OUT, vu);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (m < M) {
                            // the 8 pairs without a branch between them (their latencies overlap); a NaN in any of them
                            // sends all 8 through the form that redoes the conversions one by one
                            uint32_t o[8];
                            bool nan = false;
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                o[q] = swiglu_pair_fast(__uint_as_float(vg[2 * q]), __uint_as_float(vg[2 * q + 1]), __uint_as_float(vu[2 * q]),
                                                        __uint_as_float(vu[2 * q + 1]), nan);
                            if (nan) {
#pragma unroll
                                for (int q = 0; q < 8; q++)
                                    o[q] = swiglu_chain2(__uint_as_float(vg[2 * q]), __uint_as_float(vg[2 * q + 1]), __uint_as_float(vu[2 * q]),
                                                         __uint_as_float(vu[2 * q + 1]));
                            }
                            uint4* dst = (uint4*)(y + (size_t)m * N + n0 + c * 16);     // 32-byte aligned: N and n0 are multiples of 128
                            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                    continue;
                }
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
                    if (S == 1) {
                        if (m < M) emit(m, n0 + c * 32, v);
                    } else if (m < M) {
                        // this run's partial sums: [run][row][N] fp32
                        uint4* dst = (uint4*)(part + ((size_t)run * M + m) * N + n0 + c * 32);
#pragma unroll
                        for (int q = 0; q < 8; q++) dst[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[buf]);
        }
    } else if (warp >= 8) {
        // ---- dequant: one group of 4 warps per operand stage; group q takes the k blocks with
        // it % STAGES == q, and warp j of a group turns strip units UPW*j .. UPW*j+UPW-1 (BN/4
        // columns) of that block into fp16, two units at a time. A warp so has STAGES k-block
        // periods for its share, and pays one proxy fence for all of it.
        constexpr int UPW = BN / 64;       // strip units per warp and k block: 2 or 4
        constexpr int GROUPS = C::GROUPS;
        const uint32_t dw = warp - 8, q = dw >> 2, j = dw & 3, g = lane >> 2, t = lane & 3;
        const uint32_t my_items = blockIdx.x < items ? (items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t total = my_items * KGS;
        const uint32_t sB_u32 = smem_u32(sB), sRaw_u32 = smem_u32(sRaw);
        // byte offsets of this lane's four 16-byte chunks inside unit 0 of a B stage; a unit is 16 rows = 2048 bytes:
        // row r, 16-byte chunk c (8 k) lives at r*128 + ((c ^ (r & 7)) << 4), and r & 7 does not depend on the unit
        uint32_t off[4];
        {
            const uint32_t r0 = g, r1 = g + 8;
            off[0] = r0 * 128 + (((2 * t) ^ (r0 & 7)) << 4);
            off[1] = r0 * 128 + (((2 * t + 1) ^ (r0 & 7)) << 4);
            off[2] = r1 * 128 + (((2 * t) ^ (r1 & 7)) << 4);
            off[3] = r1 * 128 + (((2 * t + 1) ^ (r1 & 7)) << 4);
        }
        for (uint32_t it = q; q < (uint32_t)GROUPS && it < total; it += GROUPS) {
            const uint32_t s = q, ph = (it / STAGES) & 1;      // it % STAGES == q
            const uint32_t r = q, rph = ph;
            // warp-uniform decisions: every lane polls, the warp leaves together
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->raw_full[r], rph))) { *abort_flag = 1; break; }
            const uint32_t raw = sRaw_u32 + r * RAW_SLOT;
            uint4 w[UPW];
            uint16_t sl[UPW], sh[UPW];
#pragma unroll
            for (int u = 0; u < UPW; u++) {
                const uint32_t unit = UPW * j + u;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(w[u].x), "=r"(w[u].y), "=r"(w[u].z), "=r"(w[u].w) : "r"(raw + (unit * 32 + lane) * 16));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sl[u]) : "r"(raw + RAW_BYTES + (unit * 16 + g) * 2));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sh[u]) : "r"(raw + RAW_BYTES + (unit * 16 + g + 8) * 2));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->raw_empty[r]);      // the slot has been consumed into registers
            bool stage_free = false;
            const uint32_t bt = sB_u32 + s * B_BYTES;
#pragma unroll
            for (int up = 0; up < UPW; up += 2) {
                uint32_t o[2][4][4];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const __half2 slo = __half2half2(__ushort_as_half(sl[up + u])), shi = __half2half2(__ushort_as_half(sh[up + u]));
                    dequant_word(w[up + u].x, slo, shi, o[u][0]);
                    dequant_word(w[up + u].y, slo, shi, o[u][1]);
                    dequant_word(w[up + u].z, slo, shi, o[u][2]);
                    dequant_word(w[up + u].w, slo, shi, o[u][3]);
                }
                if (!stage_free) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&bars->empty[s], ph ^ 1))) { *abort_flag = 1; break; }
                    stage_free = true;
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const uint32_t ub = bt + (UPW * j + up + u) * 2048;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ub + off[0]), "r"(o[u][0][0]), "r"(o[u][0][2]), "r"(o[u][1][0]), "r"(o[u][1][2]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ub + off[1]), "r"(o[u][2][0]), "r"(o[u][2][2]), "r"(o[u][3][0]), "r"(o[u][3][2]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ub + off[2]), "r"(o[u][0][1]), "r"(o[u][0][3]), "r"(o[u][1][1]), "r"(o[u][1][3]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ub + off[3]), "r"(o[u][2][1]), "r"(o[u][2][3]), "r"(o[u][3][1]), "r"(o[u][3][3]) : "memory");
                }
            }
            if (!stage_free) break;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->full[s]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 3) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
        if (lane == 0 && *abort_flag) raise_status(ep.status, kStatusGemmTimeout);
    }
}

// y[m][n] = sum over the runs of part[run][m][n], in run order, with the epilogue of the GEMM
__global__ void __launch_bounds__(256)
w4a16_splitk_reduce_kernel(const float* __restrict__ part, uint16_t* __restrict__ y, uint32_t M, uint32_t N, uint32_t S, W4Epilogue ep) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t quads = (size_t)M * N / 4, plane = (size_t)M * N / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < S; r++) {
            const float4 p = __ldcg((const float4*)part + r * plane + i);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        uint2 o;
        if (ep.mode == 1) {
            const uint2 res = *((const uint2*)ep.res + i);
            o = make_uint2(pack_out_res(acc.x, acc.y, res.x), pack_out_res(acc.z, acc.w, res.y));
        } else {
            o = make_uint2(pack_out(acc.x, acc.y), pack_out(acc.z, acc.w));
        }
        *((uint2*)y + i) = o;
    }
}

// The same reduction for a GEMM that is followed by a residual add and an RMSNorm (W4Epilogue mode 3): one CTA per
// output row adds the runs (in run order, as above), stores y = f16(sum), then f16(y + res) and its norm - the
// add + norm kernel with the row taken from the partial sums instead of from y.
struct NormLoadRuns {
    const float* part;      // this row's partial sums of run 0
    size_t plane;           // floats between two runs
    uint32_t S;
    uint16_t* y;            // this row of the GEMM's own output
    __device__ __forceinline__ uint4 operator()(uint32_t i) const {
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < S; r++) {
            const float4 p = __ldcg((const float4*)(part + r * plane + i)), q = __ldcg((const float4*)(part + r * plane + i + 4));
            lo.x += p.x; lo.y += p.y; lo.z += p.z; lo.w += p.w;
            hi.x += q.x; hi.y += q.y; hi.z += q.z; hi.w += q.w;
        }
        const uint4 o = make_uint4(pack_out(lo.x, lo.y), pack_out(lo.z, lo.w), pack_out(hi.x, hi.y), pack_out(hi.z, hi.w));
        *(uint4*)(y + i) = o;
        return o;
    }
};

__global__ void __launch_bounds__(256)
w4a16_splitk_add_rmsnorm_kernel(const float* __restrict__ part, uint16_t* __restrict__ y, uint32_t M, uint32_t N, uint32_t S, W4Epilogue ep) {
    extern __shared__ float row[];      // N floats (rows wider than the register form takes)
    __shared__ double red[256 / 32];
    __shared__ float s_rms;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * N;
    const NormLoadRuns load{part + base, (size_t)M * N, S, y + base};
    rmsnorm_row_t<256>(threadIdx.x, [] { __syncthreads(); }, load, (const uint16_t*)nullptr, ep.res + base, ep.gamma, ep.beta, ep.sum_out + base,
                       ep.norm_out + base, N, row, red, &s_rms);
}

// Scratch of the split-K form (fp32 partial sums), per device, made on first use and grown when needed.
struct SplitScratch { float* part = nullptr; size_t bytes = 0; };

SplitScratch* split_scratch(cudaStream_t st, size_t need) {
    static SplitScratch per_dev[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SplitScratch& sc = per_dev[dev];
    if (sc.bytes >= need) return &sc;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return nullptr; }   // no allocation inside a capture
    cudaDeviceSynchronize();          // a launch in flight may still use the old buffer
    if (sc.part) cudaFree(sc.part);
    sc.part = nullptr; sc.bytes = 0;
    if (cudaMalloc(&sc.part, need) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    sc.bytes = need;
    return &sc;
}

template <int MH, int BN, bool DUAL = false>
bool launch(cudaStream_t st, const CUtensorMap& tmap, const uint32_t* packed, const uint16_t* sc, uint16_t* y,
            uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep, int sms, const uint32_t* packed2 = nullptr,
            const uint16_t* sc2 = nullptr, uint32_t a_d = 0) {
    using C = Cfg<MH, BN>;
    const size_t smem = 1024 + (size_t)C::STAGES * (C::A_BYTES + C::B_BYTES) + (size_t)C::RSTAGES * C::RAW_SLOT + sizeof(Barriers) + 16;
    static int have[64] = {};
    if (!ensure_dyn_smem(w4a16_gemm_sm100_kernel<MH, BN, DUAL>, smem, have)) return false;
    const uint32_t tiles = ((M + 128 * MH - 1) / (128 * MH)) * (N / (DUAL ? BN / 2 : BN)), KG = K / BK;
    // Split K when the tiles alone leave SMs idle. A CTA walks a k block in about 0.42 us whatever the shape, so
    // the launch lasts (items per CTA) x (k blocks per item + set-up); S is the divisor of K/64 that makes that
    // smallest, a run keeping at least one trip round the operand ring, the partial sums at most 64 MB.
    static const int split_on = [] { const char* e = std::getenv("GEHTP_CUDA_SPLITK"); return e ? std::atoi(e) : 1; }();
    uint32_t S = 1;
    if (split_on && !DUAL && tiles < (uint32_t)sms) {      // the gate | up form keeps its product in the epilogue: no runs
        float best = (float)(KG + 4);
        for (uint32_t c = 2; c <= 32 && c <= KG; c++) {
            if (KG % c || KG / c < (uint32_t)C::STAGES || (size_t)c * M * N * sizeof(float) > ((size_t)64 << 20)) continue;
            const uint32_t rounds = (tiles * c + sms - 1) / sms;
            const float cost = (float)rounds * (float)(KG / c + 4) + 0.75f * (float)c + 6.0f;   // + the reduction: one launch, c reads
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
    if (launch_pdl(w4a16_gemm_sm100_kernel<MH, BN, DUAL>, dim3(grid), dim3(NTHREADS), smem, st, tmap, (const uint4*)packed, sc,
                   (const uint4*)packed2, sc2, y, M, K, N, ep, S, part, a_d) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    if (S > 1 && ep.mode == 3) {
        if (launch_pdl(w4a16_splitk_add_rmsnorm_kernel, dim3(M), dim3(256), (size_t)N * sizeof(float), st, (const float*)part, y, M, N, S, ep) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        g_launches++;
    } else if (S > 1) {
        const size_t quads = (size_t)M * N / 4;
        uint32_t rg = (uint32_t)((quads + 255) / 256);
        if (rg > (uint32_t)sms * 8) rg = (uint32_t)sms * 8;
        if (launch_pdl(w4a16_splitk_reduce_kernel, dim3(rg), dim3(256), 0, st, (const float*)part, y, M, N, S, ep) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        g_launches++;
    }
    if (S == 1 && ep.mode == 3) k_add_rmsnorm(st, y, ep.res, ep.gamma, ep.beta, ep.sum_out, ep.norm_out, M, N);
    return true;
}

// a_d != 0: A is stored [K / a_d][M][a_d] (heads outermost, as a per-head kernel leaves its output); the map is
// three-dimensional and a k block of 64 columns is a box of one head.
bool make_a_map(CUtensorMap* tmap, const uint16_t* a, uint32_t M, uint32_t K, uint32_t a_d = 0) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    if (a_d) {
        cuuint64_t dims[3] = {a_d, M, K / a_d};
        cuuint64_t strides[2] = {(cuuint64_t)a_d * 2, (cuuint64_t)M * a_d * 2};
        cuuint32_t box[3] = {BK, 128, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        return enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void*)a, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    cuuint64_t dims[2] = {K, M};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {BK, 128};
    cuuint32_t estr[2] = {1, 1};
    return enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
    static int sms_of[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int& sms = sms_of[dev & 63];
    if (!sms) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

}  // namespace

bool k_w4a16_gemm_sm100(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                        uint16_t* y, uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep, int tile, uint32_t a_d) {
    if (!M || K % BK || N % 128) return false;
    if (a_d && (a_d % BK || K % a_d)) return false;
    if (((uintptr_t)a & 15) || ((uintptr_t)packed & 15) || ((uintptr_t)sc & 15) || ((uintptr_t)y & 15)) return false;
    if (ep.mode == 1 && ((uintptr_t)ep.res & 15)) return false;
    if (ep.mode == 3 && (!ep.res || !ep.gamma || !ep.sum_out || !ep.norm_out || N * sizeof(float) > 48u * 1024u ||
                         (((uintptr_t)ep.res | (uintptr_t)ep.gamma | (uintptr_t)ep.beta | (uintptr_t)ep.sum_out | (uintptr_t)ep.norm_out) & 15)))
        return false;
    const int sms = sm_count();
    CUtensorMap tmap;
    if (!make_a_map(&tmap, a, M, K, a_d)) return false;
    // Largest tile that still gives every SM a tile.
    const uint32_t t256 = ((M + 255) / 256) * (N / 256);
    const uint32_t t128 = ((M + 255) / 256) * (N / 128);
    const int force = tile;   // 0: by shape, 1: 128x128, 2: 256x128, 3: 256x256
    if (force == 3 ? N % 256 == 0 : (force == 0 && N % 256 == 0 && M > 128 && t256 >= (uint32_t)sms))
        return launch<2, 256>(st, tmap, packed, sc, y, M, K, N, ep, sms, nullptr, nullptr, a_d);
    if (force == 2 || (force == 0 && M > 128 && t128 >= (uint32_t)sms)) return launch<2, 128>(st, tmap, packed, sc, y, M, K, N, ep, sms, nullptr, nullptr, a_d);
    return launch<1, 128>(st, tmap, packed, sc, y, M, K, N, ep, sms, nullptr, nullptr, a_d);
}

bool w4a16_gemm_sm100_swiglu_takes(uint32_t M, uint32_t K, uint32_t N) {
    static const int on = [] { const char* e = std::getenv("GEHTP_CUDA_GEMM_SWIGLU"); return e ? std::atoi(e) : 1; }();
    return on && M && K && K % BK == 0 && N && N % 128 == 0;
}

bool k_w4a16_gemm_sm100_swiglu(cudaStream_t st, const uint16_t* a, const uint32_t* pg, const uint16_t* sg, const uint32_t* pu,
                               const uint16_t* su, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, unsigned int* status) {
    if (!w4a16_gemm_sm100_swiglu_takes(M, K, N)) return false;
    if (((uintptr_t)a | (uintptr_t)pg | (uintptr_t)sg | (uintptr_t)pu | (uintptr_t)su | (uintptr_t)y) & 15) return false;
    const int sms = sm_count();
    CUtensorMap tmap;
    if (!make_a_map(&tmap, a, M, K)) return false;
    W4Epilogue ep;
    ep.status = status;
    // 256 rows per tile once that still gives every SM a tile
    if (M > 128 && ((M + 255) / 256) * (N / 128) >= (uint32_t)sms) return launch<2, 256, true>(st, tmap, pg, sg, y, M, K, N, ep, sms, pu, su);
    return launch<1, 256, true>(st, tmap, pg, sg, y, M, K, N, ep, sms, pu, su);
}

}  // namespace gehtp
