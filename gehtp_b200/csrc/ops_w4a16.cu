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
#include <cstdlib>
#include <cuda_fp16.h>
#include "common.cuh"
#include "launchers_w4.h"
#include "w4_stream.cuh"

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
// Walk modes of the streaming kernel.
//   WALK_ONE  : every warp owns exactly UNROLL groups; one batch, all offsets
//               are compile-time multiples of the strides (the decode shapes).
//   WALK_FULL : every warp owns a whole number of batches; rolling refill.
//   WALK_ANY  : ragged tail; per-group bounds tests.
enum { WALK_ANY = 0, WALK_FULL = 1, WALK_ONE = 2 };

template <int MT, int UNROLL, bool DUAL, int WALK, bool ROPE = false, bool STAGE = false>
__global__ void __launch_bounds__(MT >= 4 ? 512 : 640)
w4a16_skinny_kernel(const uint16_t* __restrict__ a, const uint4* __restrict__ wp,
                    const uint16_t* __restrict__ sc, const uint4* __restrict__ wp2,
                    const uint16_t* __restrict__ sc2, uint16_t* __restrict__ y, uint32_t M,
                    uint32_t K, uint32_t N, uint32_t kgw, W4Epilogue ep) {
    extern __shared__ float red[];  // [nwarps][NACC][32], then (MT == 1) the activation stage [nwarps][UNROLL][rows][144 B]
    constexpr int NACC = MT * 4 * (DUAL ? 2 : 1);
    constexpr bool FULL = WALK != WALK_ANY, ONE = WALK == WALK_ONE;
    // STAGE (one or two rows of activations): a warp's activations for a batch of UNROLL k groups are copied into
    // shared memory in one go right after the dependency wait (cp.async, all requests in flight together) and the
    // fragments are read from there. Fetched group by group from global memory, every group of a warp costs one L2
    // round trip: the activations have just been written by the kernel before, they are in L2 and nowhere nearer.
    // With more rows the CTAs of an SM share the activations through L1 and the stage only costs occupancy
    // (measured on B200: batch 1 decode step -8 %, batch 8 unchanged, vocabulary projection at 8 rows +35 %).
    static_assert(!STAGE || MT == 1, "the activation stage holds one row tile");
    constexpr uint32_t AROW = 144;        // bytes of a staged row of 64 fp16 (+16: the 8 rows of a group fall on different banks)
    // Programmatic dependent launch: let the next kernel start early, and order
    // this one after its predecessor only once the first batch of weight loads
    // (constants, independent of the predecessor) is in flight.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    // ROPE: a CTA owns two strips of one head that are half a head (64 columns) apart, so that it
    // holds both members of every rotary pair; the first half of its warps walks K for the first
    // strip, the second half for the second.
    const uint32_t nwk = ROPE ? nwarps / 2 : nwarps;            // warps along K
    const uint32_t which = ROPE ? warp / nwk : 0, kwarp = ROPE ? warp % nwk : warp;
    const uint32_t nb = ROPE ? (blockIdx.x / 4) * 8 + blockIdx.x % 4 + which * 4 : blockIdx.x, NB = N / 16, KG = K / 64;
    const uint32_t m0 = blockIdx.y * (8 * MT);
    const uint32_t n_lo = nb * 16 + g;
    const uint32_t kg0 = kwarp * (ONE ? (uint32_t)UNROLL : kgw);
    const uint32_t kg1 = ONE ? kg0 + UNROLL : min(kg0 + kgw, KG);

    float acc[MT][4], acc2[DUAL ? MT : 1][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) { acc[i][c] = 0.0f; if (DUAL) acc2[i][c] = 0.0f; }

    // Per-lane pointers at the warp's first group; group `rel` lies rel strides
    // further (a weight slot is < 4 GB by its format, so 32-bit products do).
    const uint32_t wstride = NB * 512u, sstride = N * 2u;   // bytes per k group
    const char* wl = (const char*)(wp + ((size_t)kg0 * NB + nb) * 32 + lane);
    const char* wl2 = DUAL ? (const char*)(wp2 + ((size_t)kg0 * NB + nb) * 32 + lane) : nullptr;
    const char* sl = (const char*)(sc + (size_t)kg0 * N + n_lo);
    const char* sl2 = DUAL ? (const char*)(sc2 + (size_t)kg0 * N + n_lo) : nullptr;
    // This lane's activation row at the warp's first group. Rows past M read
    // row M-1 instead (no branch in the loop); their results are never stored.
    const char* arow[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) {
        const uint32_t m = min(m0 + i * 8 + g, M - 1);
        arow[i] = (const char*)(a + (size_t)m * K + (size_t)kg0 * 64 + t * 16);
    }

    // Rolling window of UNROLL k groups per warp: the first batch is requested
    // before the dependency wait, and (beyond WALK_ONE) every register slot is
    // refilled as soon as its group has been consumed.
    uint4 wq[UNROLL], wq2[DUAL ? UNROLL : 1];
    uint16_t s0[UNROLL], s1[UNROLL], t0[DUAL ? UNROLL : 1], t1[DUAL ? UNROLL : 1];
    auto fetch = [&](int u, uint32_t rel) {
        const uint32_t wo = rel * wstride, so = rel * sstride;
        wq[u] = __ldcs((const uint4*)(wl + wo));   // streamed once: evict first
        s0[u] = __ldg((const uint16_t*)(sl + so));
        s1[u] = __ldg((const uint16_t*)(sl + so) + 8);
        if (DUAL) {
            wq2[u] = __ldcs((const uint4*)(wl2 + wo));
            t0[u] = __ldg((const uint16_t*)(sl2 + so));
            t1[u] = __ldg((const uint16_t*)(sl2 + so) + 8);
        }
    };
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
        if (FULL || kg0 + u < kg1) {
            fetch(u, (uint32_t)u);
        } else {
            wq[u] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
            s0[u] = 0; s1[u] = 0;
            if (DUAL) { wq2[u] = wq[u]; t0[u] = 0; t1[u] = 0; }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t last = kg1 - kg0 - 1;
    const uint32_t rows = min(M - m0, 8u);                      // STAGE: rows staged per group
    unsigned char* stage = (unsigned char*)(red + nwarps * NACC * 32) + (size_t)warp * UNROLL * rows * AROW;
    // STAGE: groups relb .. relb+UNROLL-1 of this warp into its stage; returns when they have landed
    auto stage_batch = [&](uint32_t relb) {
        __syncwarp();                                           // the batch before has been read
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (!FULL && relb + u > last) break;
            for (uint32_t c = lane; c < rows * 8; c += 32) {
                const uint32_t r = c >> 3, col = c & 7;
                const uint16_t* src = a + (size_t)(m0 + r) * K + (size_t)(kg0 + relb + u) * 64 + col * 8;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(stage + ((size_t)u * rows + r) * AROW + col * 16);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
    };
    // activations of group `rel`: STAGE reads slot rel % UNROLL of the stage (rows past M read row M-1), the other
    // forms fetch from global memory one group ahead of their use
    uint4 bc[MT][2];
    auto load_act = [&](uint4 (&b)[MT][2], uint32_t rel) {
        if (STAGE) {
            const unsigned char* sp = stage + ((size_t)(rel % UNROLL) * rows + min((uint32_t)g, rows - 1)) * AROW + t * 32;
            b[0][0] = *(const uint4*)sp;
            b[0][1] = *(const uint4*)(sp + 16);
            return;
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
            const uint4* ap = (const uint4*)(arow[i] + rel * 128u);   // 64 fp16 per group
            b[i][0] = ld_ordered(ap);
            b[i][1] = ld_ordered(ap + 1);
        }
    };
    // MT <= 2 without a stage: the next group's activations are requested one group ahead; wider
    // row tiles (MT = 4) have no registers for that and load them at their use.
    constexpr bool PRE = MT <= 2 && !STAGE;
    if (PRE) load_act(bc, 0);
    auto batch = [&](uint32_t relb, bool more) {   // groups relb .. relb+UNROLL-1
        if (STAGE) stage_batch(relb);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (!FULL && relb + u > last) break;
            uint4 bn[PRE ? MT : 1][2];
            const bool have_next = PRE && (u + 1 < UNROLL || !ONE);
            if (PRE) {
                if (have_next) load_act(*(uint4(*)[MT][2])&bn, ONE ? (uint32_t)(u + 1) : min(relb + u + 1, last));
            } else {
                load_act(bc, ONE ? (uint32_t)u : relb + u);
            }
            uint32_t af[4][4];
            dequant_word(wq[u].x, af[0]);
            dequant_word(wq[u].y, af[1]);
            dequant_word(wq[u].z, af[2]);
            dequant_word(wq[u].w, af[3]);
            {
                const float slo = h2f(s0[u]), shi = h2f(s1[u]);
#pragma unroll
                for (int i = 0; i < MT; i++) mma_group(acc[i], af, bc[i][0], bc[i][1], slo, shi);
            }
            if (DUAL) {
                dequant_word(wq2[u].x, af[0]);
                dequant_word(wq2[u].y, af[1]);
                dequant_word(wq2[u].z, af[2]);
                dequant_word(wq2[u].w, af[3]);
                const float tlo = h2f(t0[u]), thi = h2f(t1[u]);
#pragma unroll
                for (int i = 0; i < MT; i++) mma_group(acc2[i], af, bc[i][0], bc[i][1], tlo, thi);
            }
            if (!ONE && more && (FULL || relb + UNROLL + u <= last)) fetch(u, relb + UNROLL + u);
            if (have_next) {
#pragma unroll
                for (int i = 0; i < (PRE ? MT : 1); i++) {
                    bc[i][0] = bn[i][0];
                    bc[i][1] = bn[i][1];
                }
            }
        }
    };
    if (ONE) {
        batch(0, false);
    } else {
        for (uint32_t relb = 0; relb <= last; relb += UNROLL) batch(relb, relb + UNROLL <= last);
    }

#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            red[(warp * NACC + i * 4 + c) * 32 + lane] = acc[i][c];
            if (DUAL) red[(warp * NACC + MT * 4 + i * 4 + c) * 32 + lane] = acc2[i][c];
        }
    __syncthreads();
    if (ROPE) {
        // one thread per (row m, column d of the first half): it owns d and d + 64 of its head
        const uint32_t hd = 128, hidx = blockIdx.x / 4, d0 = (blockIdx.x % 4) * 16;
        const uint32_t pos = ep.pos_const == 0xFFFFFFFAu ? *ep.counter : ep.pos_const;
        const uint32_t slot = pos % ep.nslots;
        const uint32_t kv_elems = M * ep.kvh * hd;
        uint16_t* kf = ep.ring + (size_t)slot * kv_elems * 2;
        uint16_t* vf = kf + kv_elems;
        for (uint32_t idx = threadIdx.x; idx < 4 * 32; idx += blockDim.x) {
            float sa = 0.0f, sb = 0.0f;
            for (uint32_t w = 0; w < nwk; w++) {
                sa += red[w * NACC * 32 + idx];
                sb += red[(nwk + w) * NACC * 32 + idx];
            }
            const uint32_t ln = idx & 31, c = idx >> 5;
            const uint32_t d = d0 + (ln >> 2) + ((c & 2) ? 8 : 0);
            const uint32_t m = (ln & 3) * 2 + (c & 1);
            if (m >= M) continue;
            const uint16_t xa = f2h(sa), xb = f2h(sb);          // the matmul's own fp16 outputs
            if (hidx >= ep.nh + ep.kvh) {                        // v head: plain copy into the ring
                const size_t o = ((size_t)m * ep.kvh + (hidx - ep.nh - ep.kvh)) * hd + d;
                vf[o] = xa;
                vf[o + 64] = xb;
                continue;
            }
            const bool is_q = hidx < ep.nh;
            const size_t o = is_q ? ((size_t)m * ep.nh + hidx) * hd + d : ((size_t)m * ep.kvh + (hidx - ep.nh)) * hd + d;
            const uint16_t* ct = is_q ? ep.cos_q : ep.cos_k;
            const uint16_t* st = is_q ? ep.sin_q : ep.sin_k;
            uint16_t* dst = is_q ? ep.q_out : kf;
            const float fa = h2f(xa), fb = h2f(xb);
            // out[d] = x[d] cos - x[d+64] sin ; out[d+64] = x[d+64] cos + x[d] sin, each product rounded to fp16
            const float lo = __fadd_rn(h2f(f2h(__fmul_rn(fa, h2f(ct[o])))), h2f(f2h(__fmul_rn(-fb, h2f(st[o])))));
            const float hi = __fadd_rn(h2f(f2h(__fmul_rn(fb, h2f(ct[o + 64])))), h2f(f2h(__fmul_rn(fa, h2f(st[o + 64])))));
            dst[o] = f2h(lo);
            dst[o + 64] = f2h(hi);
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) ep.posmap[slot] = pos;
        return;
    }
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

// k groups per warp (a multiple of 8). Default 8 (one register batch per warp,
// the widest split of K). When that many warps per CTA would leave the strips
// unable to be resident together (a long K with few columns: register-limited
// to one CTA per SM and more strips than SMs), warps take more batches instead,
// so that the whole grid is one wave.
static uint32_t skinny_kgw(uint32_t KG, uint32_t strips) {
    uint32_t fallback = 0;
    for (uint32_t kgw = 8; kgw <= 256; kgw += 8) {
        const uint32_t nw = (KG + kgw - 1) / kgw;
        if (nw > 20) continue;
        if (!fallback) fallback = kgw;
        const uint32_t threads = nw * 32;
        uint32_t per_sm = 2048 / threads;
        const uint32_t by_regs = 65536 / (80 * threads);
        if (by_regs < per_sm) per_sm = by_regs;
        if (per_sm > 32) per_sm = 32;
        if (per_sm && strips <= 148 * per_sm) return kgw;
        if (kgw >= 32) break;
    }
    return fallback ? fallback : 8;
}

// Launch of a one-row-tile form: dynamic shared memory = the reduction buffer + the activation stage
// (M <= 2: nwarps x UNROLL groups x M rows x 144 bytes), opted in per device when it passes 48 KB.
template <int UNROLL, bool DUAL, int WALK, bool ROPE, typename... Args>
static void launch_skinny1(dim3 grid, dim3 block, uint32_t M, cudaStream_t st, Args... args) {
    static int have[64];
    const uint32_t nwarps = block.x / 32;
    const size_t red = (size_t)nwarps * (DUAL ? 8 : 4) * 32 * sizeof(float);
    // The vocabulary projection (9496 strips) is staged as well: alone, in back-to-back replays, it runs 41 us
    // direct and 50 us staged (the activations stay in L1 there), but inside the batch-1 step the staged form is
    // the faster one by 77 us (1.75 vs 1.82 ms per step, measured twice each way on one B200).
    if (M > 2) {
        launch_pdl(w4a16_skinny_kernel<1, UNROLL, DUAL, WALK, ROPE, false>, grid, block, red, st, args...);
        return;
    }
    const size_t smem = red + (size_t)nwarps * UNROLL * M * 144;
    if (smem > 48 * 1024 && !ensure_dyn_smem(w4a16_skinny_kernel<1, UNROLL, DUAL, WALK, ROPE, true>, 200 * 1024, have)) return;
    launch_pdl(w4a16_skinny_kernel<1, UNROLL, DUAL, WALK, ROPE, true>, grid, block, smem, st, args...);
}

#define SKINNY_ARGS(P1, S1, P2, S2) a, (const uint4*)(P1), S1, (const uint4*)(P2), (const uint16_t*)(S2), y, M, K, N, kgw, ep

void k_w4a16_skinny(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                    uint16_t* y, uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep) {
    if (!M || !N || !K) return;
    const uint32_t KG = K / 64;
    const uint32_t kgw = skinny_kgw(KG, N / 16), nwarps = (KG + kgw - 1) / kgw;
    const dim3 block(nwarps * 32);
    if (M <= 8) {
        const dim3 grid(N / 16, 1);
        if (kgw == 8 && KG % 8 == 0)
            launch_skinny1<8, false, WALK_ONE, false>(grid, block, M, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
        else if (kgw % 8 == 0 && KG % 8 == 0)
            launch_skinny1<8, false, WALK_FULL, false>(grid, block, M, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
        else
            launch_skinny1<8, false, WALK_ANY, false>(grid, block, M, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
    } else if (M <= 16 || nwarps > 16) {
        const dim3 grid(N / 16, (M + 15) / 16);
        const size_t smem = (size_t)nwarps * 8 * 32 * sizeof(float);
        launch_pdl(w4a16_skinny_kernel<2, 4, false, WALK_ANY>, grid, block, smem, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
    } else {
        // 32 rows per CTA: the strip is dequantised once per 32 rows instead of once per 16
        const dim3 grid(N / 16, (M + 31) / 32);
        const size_t smem = (size_t)nwarps * 16 * 32 * sizeof(float);
        launch_pdl(w4a16_skinny_kernel<4, 4, false, WALK_ANY>, grid, block, smem, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
    }
    g_launches++;
}

bool k_w4a16_skinny_qkv_rope(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                             uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep) {
    const uint32_t KG = K / 64;
    if (!M || M > 8 || K % 512 || KG / 8 > 10 || ep.mode != 2 || N != (ep.nh + 2 * ep.kvh) * 128u) return false;
    const uint32_t kgw = 8, nwk = KG / 8;
    uint16_t* y = nullptr;
    const dim3 grid(N / 32, 1), block(2 * nwk * 32);
    launch_skinny1<8, false, WALK_ONE, true>(grid, block, M, st, SKINNY_ARGS(packed, sc, nullptr, nullptr));
    g_launches++;
    return true;
}

// y = swiglu(a.Wg, a.Wu): two weight matrices of the same shape in one pass.
void k_w4a16_skinny_swiglu(cudaStream_t st, const uint16_t* a, const uint32_t* pg, const uint16_t* sg,
                           const uint32_t* pu, const uint16_t* su, uint16_t* y, uint32_t M, uint32_t K,
                           uint32_t N) {
    if (!M || !N || !K) return;
    const uint32_t KG = K / 64;
    uint32_t kgw = skinny_kgw(KG, 0xFFFFFFFFu), nwarps = (KG + kgw - 1) / kgw;
    W4Epilogue ep;
    if (M <= 8) {
        const dim3 grid(N / 16, 1);
        if (KG % 4 == 0 && KG / 4 <= 20) {   // whole 4-group warps: the branch-free variant
            kgw = 4;
            nwarps = KG / 4;
            launch_skinny1<4, true, WALK_ONE, false>(grid, dim3(nwarps * 32), M, st, SKINNY_ARGS(pg, sg, pu, su));
        } else {
            launch_skinny1<4, true, WALK_ANY, false>(grid, dim3(nwarps * 32), M, st, SKINNY_ARGS(pg, sg, pu, su));
        }
    } else {
        const dim3 grid(N / 16, (M + 15) / 16);
        launch_pdl(w4a16_skinny_kernel<2, 2, true, WALK_ANY>, grid, dim3(nwarps * 32), (size_t)nwarps * 16 * 32 * sizeof(float), st, SKINNY_ARGS(pg, sg, pu, su));
    }
    g_launches++;
}

}  // namespace gehtp
