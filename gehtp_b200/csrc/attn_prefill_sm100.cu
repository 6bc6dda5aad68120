// Prefill attention on tcgen05 / TMEM: softmax(Q K^T * scale + mask) V, head_dim 128, grouped-query heads.
//
// Same op chain and the same fp16 rounding points of a score as ops_attn_prefill.cu (after the dot
// product, after the scale, after the mask); the probabilities are exp(s - rowmax) / rowsum rounded to
// fp16 before they meet V; the division by the row sum is applied to the fp32 output accumulator (the reference's
// SOFTMAX op, oplist_exec.c:1163-1194, divides first and rounds then: a difference of rounding only).
//
// One CTA = one query head x 128 query rows. Key/value tiles of 128 positions; tiles whose mask is -inf
// everywhere (upper triangle of a causal mask) are skipped. Two passes over the live tiles:
//   pass 1  S = Q K^T per tile -> row maximum (on tiles whose mask is +0 everywhere: the maximum of the raw dot
//           products, pushed through the roundings once per row; nothing is kept of S);
//   pass 2  S again -> P = f16(exp(s - max)), row sum -> O += P V; O / sum at the end.
// Recomputing S costs tensor time, which is plentiful here; it removes the rescaling of the output
// accumulator that an online softmax needs (O stays in TMEM untouched until the end).
//
// Operands: Q, K token-major (head_dim contiguous) are K-major for S = Q K^T; for O = P V the
// contraction runs over key positions: V is read as it lies in memory ([position][head_dim]) and declared
// an MN-major B operand (instruction descriptor bit 16; boxes of 64 positions x 64 head_dim values, see
// umma_desc_v), and P is written by the softmax warps into shared memory in the 128-byte-swizzled K-major
// form tcgen05.mma reads.
//
//   warp 0     TMA producer: Q once, then K tiles (both passes) and V tiles (pass 2), 2-stage rings
//   warp 1     one lane issues tcgen05.mma / tcgen05.commit
//   warp 2     owns the TMEM allocation (512 columns: two S buffers, O)
//   warps 4-11 softmax: warp w works on TMEM lanes 32 (w % 4) .. +31 (one query row per thread) and on
//              the key columns 64 ((w - 4) / 4) .. +63 of a tile; the two warps of a row exchange their
//              tile maxima through shared memory.
// Every mbarrier wait is bounded; on a timeout the CTA raises the engine's status word and winds down.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launchers_attn.h"
#include "sm100_umma.cuh"

namespace gehtp {

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128, TILE_BYTES = 128 * 64 * 2;   // one 128 x 64 fp16 box
constexpr int NTHREADS = 384;

struct __align__(8) ABars {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, p_empty, o_full;
    uint64_t pair[4];         // the two softmax warps of a row quarter meet here (bounded, unlike bar.sync)
    uint32_t tmem_base, abort_flag;
    unsigned long long live, zero;   // bit kt: tile (qt, kt) has a live entry / a mask of +0 everywhere (n_kt <= 64)
    float xmax[2][128];       // tile maxima of the two column halves of a row
    float xsum[2][128];
};

struct SmArgs {
    const uint16_t* mask;        // [heads or 1][seq_q][seq_k] additive fp16, or NULL
    size_t mask_head_stride;
    const uint8_t* skip;         // [ceil(seq_q/64)][ceil(seq_k/64)], 1 = 64 x 64 tile fully masked, or NULL
    const uint8_t* zero;         // same shape, 1 = the mask of the 64 x 64 tile is +0 everywhere, or NULL
    uint16_t* out;               // [seq_q][nh * 128]
    uint32_t seq_q, seq_k, nh, kvh;
    float scale;
    int scale_div;
    unsigned int* status;
};

__device__ __forceinline__ float round_h(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float score_of(float dot, float rscale, float maskv) {
    float s = round_h(dot);
    s = round_h(__fmul_rn(s, rscale));
    return round_h(__fadd_rn(s, maskv));
}

// Two fp32 values -> one half2 word (low half = a) in one instruction, and back. The softmax warps are bound by
// the ALU pipe: the score roundings run on pairs.
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
__device__ __forceinline__ float2 unpack_h2(uint32_t h) { return __half22float2(*(const __half2*)&h); }
// the scores of two neighbouring positions with the roundings of the op chain; mk = their two mask values (half2 word)
template <bool MASKED>
__device__ __forceinline__ float2 score2(float d0, float d1, float rscale, uint32_t mk) {
    float2 f = unpack_h2(pack_h2(d0, d1));
    f = unpack_h2(pack_h2(__fmul_rn(f.x, rscale), __fmul_rn(f.y, rscale)));
    if (MASKED) {
        const float2 m = unpack_h2(mk);
        f = unpack_h2(pack_h2(__fadd_rn(f.x, m.x), __fadd_rn(f.y, m.y)));
    }
    return f;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// P of one row for 64 positions: 2^(s log2e + m_off) rounded to fp16, eight 16-byte chunks; adds the unrounded values to l
template <bool MASKED>
__device__ __forceinline__ void probs64(uint32_t taddr, const uint4 (&mk)[8], float rscale, float m_off, float& l, uint4 (&pk)[8]) {
    const float LOG2E = 1.4426950408889634f;
#pragma unroll
    for (int c = 0; c < 2; c++) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        const uint32_t* m32 = (const uint32_t*)mk + c * 16;
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int e0 = ch * 8 + 2 * i;
                const float2 sc = score2<MASKED>(__uint_as_float(v[e0]), __uint_as_float(v[e0 + 1]), rscale, MASKED ? m32[e0 >> 1] : 0u);
                const float p0 = ex2(fmaf(sc.x, LOG2E, m_off)), p1 = ex2(fmaf(sc.y, LOG2E, m_off));
                l += p0 + p1;
                w[i] = pack_h2(p0, p1);
            }
            pk[c * 4 + ch] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// true: the 128 x 128 tile (qt, kt) has no live entry
__device__ __forceinline__ bool tile_dead(const uint8_t* skip, uint32_t qt, uint32_t kt, uint32_t nq64, uint32_t nk64) {
    if (!skip) return false;
    for (uint32_t a = 0; a < 2; a++)
        for (uint32_t b = 0; b < 2; b++) {
            const uint32_t r = 2 * qt + a, c = 2 * kt + b;
            if (r < nq64 && c < nk64 && !skip[(size_t)r * nk64 + c]) return false;
        }
    return true;
}

// true: the mask of the 128 x 128 tile (qt, kt) is +0 on all its entries
__device__ __forceinline__ bool tile_zero(const uint8_t* zero, uint32_t qt, uint32_t kt, uint32_t nq64, uint32_t nk64) {
    if (!zero) return false;
    for (uint32_t a = 0; a < 2; a++)
        for (uint32_t b = 0; b < 2; b++) {
            const uint32_t r = 2 * qt + a, c = 2 * kt + b;
            if (r < nq64 && c < nk64 && !zero[(size_t)r * nk64 + c]) return false;
        }
    return true;
}

// B-operand descriptor of a V tile as it lies in memory ([position][head_dim], head_dim contiguous = "MN-major"):
// boxes of 64 positions x 64 head_dim values (128-byte rows, 128-byte swizzle); 8-position groups 1024 bytes
// apart (stride byte offset), the second head_dim half 8192 bytes further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_v(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(8192 >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(NTHREADS, 1)
attn_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const SmArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                          // 2 boxes (head_dim halves)
    unsigned char* sK = sQ + 2 * TILE_BYTES;           // 2 stages x 2 boxes
    unsigned char* sV = sK + 4 * TILE_BYTES;           // 2 stages x 2 boxes (position halves)
    unsigned char* sP = sV + 4 * TILE_BYTES;           // 2 boxes (position halves)
    ABars* bars = (ABars*)(sP + 2 * TILE_BYTES);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;     // the longest rows first
    const uint32_t head = blockIdx.y, kvhd = head / (A.nh / A.kvh);
    const uint32_t q0 = qt * BQ;
    const uint32_t n_kt = (A.seq_k + BKV - 1) / BKV;
    const uint32_t nq64 = (A.seq_q + 63) / 64, nk64 = (A.seq_k + 63) / 64;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
            mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
            mbar_init(&bars->s_full[s], 1); mbar_init(&bars->s_empty[s], 8);
        }
        mbar_init(&bars->p_full, 8); mbar_init(&bars->p_empty, 1); mbar_init(&bars->o_full, 1);
        for (int s = 0; s < 4; s++) mbar_init(&bars->pair[s], 2);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 3) {
        // which key tiles this CTA works on, read once (the tables are constants: no need to wait for the predecessor)
        unsigned long long lv = 0, zr = 0;
        for (uint32_t kt = lane; kt < n_kt; kt += 32) {
            if (!tile_dead(A.skip, qt, kt, nq64, nk64)) lv |= 1ull << kt;
            if (tile_zero(A.zero, qt, kt, nq64, nk64)) zr |= 1ull << kt;
        }
        for (int o = 16; o; o >>= 1) { lv |= __shfl_xor_sync(0xffffffffu, lv, o); zr |= __shfl_xor_sync(0xffffffffu, zr, o); }
        if (lane == 0) { bars->live = lv; bars->zero = zr; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;
    const uint32_t tm_o = tmem + 256;
    const unsigned long long live = bars->live, zero_tiles = bars->zero;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            mbar_expect_tx(&bars->q_full, 2 * TILE_BYTES);
            tma_load_2d(sQ, &tmap_q, (int)(head * HD), (int)q0, &bars->q_full);
            tma_load_2d(sQ + TILE_BYTES, &tmap_q, (int)(head * HD + 64), (int)q0, &bars->q_full);
            uint32_t ik = 0, iv = 0;
            for (int pass = 0; pass < 2 && !*abort_flag; pass++)
                for (uint32_t kt = 0; kt < n_kt && !*abort_flag; kt++) {
                    if (!((live >> kt) & 1ull)) continue;
                    {
                        const uint32_t s = ik & 1, ph = (ik >> 1) & 1;
                        if (!mbar_wait(&bars->k_empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                        mbar_expect_tx(&bars->k_full[s], 2 * TILE_BYTES);
                        tma_load_2d(sK + s * 2 * TILE_BYTES, &tmap_k, (int)(kvhd * HD), (int)(kt * BKV), &bars->k_full[s]);
                        tma_load_2d(sK + s * 2 * TILE_BYTES + TILE_BYTES, &tmap_k, (int)(kvhd * HD + 64), (int)(kt * BKV), &bars->k_full[s]);
                        ik++;
                    }
                    if (pass == 1) {
                        const uint32_t s = iv & 1, ph = (iv >> 1) & 1;
                        if (!mbar_wait(&bars->v_empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                        mbar_expect_tx(&bars->v_full[s], 2 * TILE_BYTES);
                        // [position half][head_dim half][64 positions x 128 bytes]
#pragma unroll
                        for (uint32_t b4 = 0; b4 < 4; b4++)
                            tma_load_2d(sV + s * 2 * TILE_BYTES + b4 * (TILE_BYTES / 2), &tmap_v, (int)(kvhd * HD + (b4 & 1) * 64),
                                        (int)(kt * BKV + (b4 >> 1) * 64), &bars->v_full[s]);
                        iv++;
                    }
                }
            if (*abort_flag) {   // copies already requested must land before the CTA may go away
                for (uint32_t j = ik > 2 ? ik - 2 : 0; j < ik; j++) mbar_wait(&bars->k_full[j & 1], (j >> 1) & 1);
                for (uint32_t j = iv > 2 ? iv - 2 : 0; j < iv; j++) mbar_wait(&bars->v_full[j & 1], (j >> 1) & 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t q_base = smem_u32(sQ), k_base = smem_u32(sK), v_base = smem_u32(sV), p_base = smem_u32(sP);
            bool ok = mbar_wait(&bars->q_full, 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t ik = 0, is = 0;
            // S[buf] = Q K_tile^T : 2 head_dim halves x 4 steps of k16
            auto issue_s = [&]() -> bool {
                const uint32_t s = ik & 1, buf = is & 1;
                if (!mbar_wait(&bars->k_full[s], (ik >> 1) & 1)) return false;
                if (!mbar_wait(&bars->s_empty[buf], ((is >> 1) & 1) ^ 1)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t kb = 0; kb < 2; kb++)
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; k4++)
                        umma_f16(tmem + buf * 128, umma_desc(q_base + kb * TILE_BYTES) + (uint64_t)(k4 * 2),
                                 umma_desc(k_base + s * 2 * TILE_BYTES + kb * TILE_BYTES) + (uint64_t)(k4 * 2), idesc_f16(128), (kb | k4) ? 1u : 0u);
                umma_commit(&bars->k_empty[s]);
                umma_commit(&bars->s_full[buf]);
                ik++; is++;
                return true;
            };
            // pass 1
            for (uint32_t kt = 0; ok && kt < n_kt && !*abort_flag; kt++) {
                if (!((live >> kt) & 1ull)) continue;
                ok = issue_s();
            }
            // pass 2: S of the next live tile is issued before P V of the current one
            const uint32_t n_live = (uint32_t)__popcll(live);
            if (ok && n_live && !*abort_flag) ok = issue_s();
            for (uint32_t j = 0; ok && j < n_live && !*abort_flag; j++) {
                if (j + 1 < n_live) ok = issue_s();
                if (!ok) break;
                const uint32_t s = j & 1;
                if (!mbar_wait(&bars->v_full[s], (j >> 1) & 1) || !mbar_wait(&bars->p_full, j & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t kb = 0; kb < 2; kb++)
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; k4++)
                        // 16 positions = two 8-position groups = 2048 bytes per step; bit 16: B is MN-major
                        umma_f16(tm_o, umma_desc(p_base + kb * TILE_BYTES) + (uint64_t)(k4 * 2),
                                 umma_desc_v(v_base + s * 2 * TILE_BYTES + kb * TILE_BYTES + k4 * 2048), idesc_f16(128) | (1u << 16), (j | kb | k4) ? 1u : 0u);
                umma_commit(&bars->v_empty[s]);
                umma_commit(&bars->p_empty);
            }
            if (ok && !*abort_flag) umma_commit(&bars->o_full);
            if (!ok) *abort_flag = 1;
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ softmax and epilogue
        const uint32_t quarter = warp & 3, half = (warp - 4) >> 2;
        const uint32_t row = quarter * 32 + lane;              // query row of the tile = TMEM lane
        const uint32_t qrow = q0 + row;
        const uint32_t lane_addr = (quarter * 32) << 16;
        const uint16_t* mrow = A.mask ? A.mask + (size_t)head * A.mask_head_stride + (size_t)min(qrow, A.seq_q - 1) * A.seq_k : nullptr;
        const bool mvec = ((A.seq_k & 7u) == 0) && (((uintptr_t)A.mask & 15u) == 0);
        const float rscale = A.scale_div ? 1.0f / A.scale : A.scale;   // s * (1 / scale): within an fp32 step of s / scale before the fp16 rounding
        float m_run = -INFINITY, l_run = 0.0f;
        uint32_t is = 0, pair_phase = 0;
        bool ok = true;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // the two warps of a row quarter wait for each other; shared-memory writes before it are visible after it
        auto pair_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->pair[quarter]);
            const bool done = __all_sync(0xffffffffu, mbar_wait(&bars->pair[quarter], pair_phase));
            pair_phase ^= 1;
            return done;
        };
        // mask values of this row for 64 positions from tile column c0 (requested before the scores are waited for)
        auto mask64 = [&](uint32_t kt, uint32_t c0, uint4 (&mk)[8]) {
            const uint32_t key0 = kt * BKV + c0;
            if (mrow && mvec && key0 + 64 <= A.seq_k) {
#pragma unroll
                for (int q4 = 0; q4 < 8; q4++) mk[q4] = __ldg((const uint4*)(mrow + key0) + q4);
            } else {                                            // positions past the sequence count as masked out
                uint16_t* m16 = (uint16_t*)mk;
#pragma unroll
                for (int i = 0; i < 64; i++) m16[i] = key0 + i < A.seq_k ? (mrow ? mrow[key0 + i] : (uint16_t)0) : (uint16_t)0xFC00u;
            }
        };
        for (int pass = 0; pass < 2 && ok; pass++) {
            uint32_t jp = 0;
            for (uint32_t kt = 0; kt < n_kt && ok; kt++) {
                if (!((live >> kt) & 1ull)) continue;
                // a tile whose mask is +0 everywhere and that lies inside the sequence needs no mask values
                const bool plain = (!mrow || ((zero_tiles >> kt) & 1ull)) && (kt + 1) * BKV <= A.seq_k;
                uint4 mk[8];
                if (!plain) mask64(kt, half * 64, mk);
                const uint32_t buf = is & 1;
                ok = !__any_sync(0xffffffffu, *abort_flag != 0);
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[buf], (is >> 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (pass == 0) {
                    // row maximum of the tile. Rounding to fp16 and a positive scale keep the order, so without a mask
                    // the maximum of the scores is the score of the largest dot product.
                    float mt = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t v[32];
                        tmem_ld32(tmem + lane_addr + buf * 128 + half * 64 + c * 32, v);
                        if (plain) {
#pragma unroll
                            for (int i = 0; i < 32; i++) mt = fmaxf(mt, __uint_as_float(v[i]));
                        } else {
                            const uint32_t* m32 = (const uint32_t*)mk + c * 16;
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                const float2 sc = score2<true>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), rscale, m32[i]);
                                mt = fmaxf(mt, fmaxf(sc.x, sc.y));
                            }
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->s_empty[buf]);
                    if (plain) mt = score_of(mt, rscale, 0.0f);
                    m_run = fmaxf(m_run, mt);
                } else {
                    if (jp == 0) {
                        // the two column halves of a row agree on the row maximum once, before the second pass
                        bars->xmax[half][row] = m_run;
                        if (!pair_sync()) { ok = false; break; }
                        m_run = fmaxf(bars->xmax[0][row], bars->xmax[1][row]);
                    }
                    // P of this warp's 64 columns: 8 chunks of 8 positions, 16 bytes each, swizzled by row. The values are
                    // formed first; the buffer (still read by P V of the tile before) is waited for only then.
                    uint4 pk[8];
                    // exp(s - m) as 2^(s log2e - m log2e); a row with no live position (m = -inf) gives zeros through m_off = 0
                    const float m_off = m_run == -INFINITY ? 0.0f : -m_run * 1.4426950408889634f;
                    if (plain) probs64<false>(tmem + lane_addr + buf * 128 + half * 64, mk, rscale, m_off, l_run, pk);
                    else probs64<true>(tmem + lane_addr + buf * 128 + half * 64, mk, rscale, m_off, l_run, pk);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->s_empty[buf]);
                    if (!__all_sync(0xffffffffu, mbar_wait(&bars->p_empty, (jp & 1) ^ 1))) { ok = false; break; }
                    unsigned char* prow = sP + half * TILE_BYTES + row * 128;
#pragma unroll
                    for (uint32_t chunk = 0; chunk < 8; chunk++) *(uint4*)(prow + ((chunk ^ (row & 7u)) << 4)) = pk[chunk];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->p_full);
                    jp++;
                }
                is++;
            }
        }
        // ---- O / row sum -> fp16 -> out; this warp stores head_dim columns 64 half .. +63 of its rows
        float inv_l = 0.0f;
        if (ok) {
            bars->xsum[half][row] = l_run;
            ok = pair_sync();
            const float l = bars->xsum[0][row] + bars->xsum[1][row];
            inv_l = l > 0.0f ? 1.0f / l : 0.0f;
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, 0));
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tmem_ld32(tm_o + lane_addr + half * 64 + c * 32, v);
                if (qrow < A.seq_q) {
                    uint4* dst = (uint4*)(A.out + ((size_t)qrow * A.nh + head) * HD + half * 64 + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)      // a row without a live position never reached the accumulator: zeros
                            w[i] = inv_l == 0.0f ? 0u : (uint32_t)f2h(__uint_as_float(v[8 * q4 + 2 * i]) * inv_l) |
                                                        ((uint32_t)f2h(__uint_as_float(v[8 * q4 + 2 * i + 1]) * inv_l) << 16);
                        dst[q4] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        } else {
            *abort_flag = 1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
        if (lane == 0 && *abort_flag) raise_status(A.status, kStatusAttnTimeout);
    }
}

bool make_map(CUtensorMap* tm, const uint16_t* base, uint64_t inner, uint64_t rows, uint64_t row_stride_elems, uint32_t box_rows = 128) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// false: shape not taken (head_dim other than 128, more than 8192 key positions, unaligned operands, scale <= 0);
// nothing launched.
bool k_attn_prefill_sm100(cudaStream_t st, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask,
                          size_t mask_head_stride, const uint8_t* skip, const uint8_t* zero, float scale, int scale_div, uint32_t seq_q,
                          uint32_t seq_k, uint32_t nh, uint32_t kvh, uint32_t hd, uint16_t* out, unsigned int* status) {
    if (hd != 128 || !seq_q || !seq_k || seq_k > 64 * BKV || !kvh || nh % kvh) return false;
    if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out)) & 15u) return false;
    if (scale <= 0.0f) return false;      // the row maximum is taken before the scale: the scale must keep the order
    CUtensorMap tq, tk, tv;
    if (!make_map(&tq, q, (uint64_t)nh * hd, seq_q, (uint64_t)nh * hd) || !make_map(&tk, k, (uint64_t)kvh * hd, seq_k, (uint64_t)kvh * hd) ||
        !make_map(&tv, v, (uint64_t)kvh * hd, seq_k, (uint64_t)kvh * hd, 64))
        return false;
    const size_t smem = 1024 + 12 * (size_t)TILE_BYTES + sizeof(ABars) + 16;
    static int have[64] = {};
    if (!ensure_dyn_smem(attn_prefill_sm100_kernel, smem, have)) return false;
    SmArgs a{mask, mask_head_stride, skip, zero, out, seq_q, seq_k, nh, kvh, scale, scale_div, status};
    if (launch_pdl(attn_prefill_sm100_kernel, dim3((seq_q + BQ - 1) / BQ, nh), dim3(NTHREADS), smem, st, tq, tk, tv, a) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    g_launches++;
    return true;
}

}  // namespace gehtp
