// One-shot all-reduce over NVLink peer memory for the small vectors of a
// tensor-parallel decode step (one row of the hidden state per sequence).
//
// Every rank owns a mailbox in its own HBM: two banks (epoch parity) of one data
// slot and one flag row per source rank. An all-reduce is ONE kernel per rank:
//   push : each CTA copies its chunk of the local partial sums into slot
//          [bank][my rank] of every rank's mailbox (its own included), fences,
//          and stores the epoch into flag [bank][my rank][cta] of every mailbox;
//   wait : the CTA polls its own mailbox until the flags of all ranks for this
//          chunk carry the epoch (bounded: on a timeout it raises the engine's
//          status word and goes on, the step is then reported as failed);
//   sum  : the CTA adds the world slots in rank order in fp32 and stores fp16,
//          so every rank gets the same bits.
// The epoch lives in device memory and is advanced by the last CTA of each
// launch, so a captured CUDA graph replays correctly. Bank k%2 is only written
// again by all-reduce k+2, which a rank can reach only after every peer has
// flagged k+1, i.e. finished reading k: two banks suffice.
//
// Only plain peer loads/stores are used (no multimem, no bulk copies).
#include <cstdio>
#include <cstring>
#include "common.cuh"
#include "engine.h"
#include "launchers.h"
#include "norm_row.cuh"

namespace gehtp {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 64;
constexpr size_t kSlotBytes = 1u << 20;                       // per source rank and bank
constexpr size_t kDataBytes = 2 * kMaxWorld * kSlotBytes;
constexpr size_t kFlagBytes = 2 * kMaxWorld * kMaxCtas * sizeof(uint32_t);
constexpr size_t kLLSlotBytes = 1u << 20;                     // flag-in-data slots: 8 bytes per 4 payload bytes
constexpr size_t kLLBytes = 2 * kMaxWorld * kLLSlotBytes;
constexpr size_t kBoxBytes = kDataBytes + kFlagBytes + kLLBytes;
constexpr uint32_t kSpinLimit = 4u * 1000u * 1000u;           // polls (with a short sleep) before giving up

struct P2PCtx {
    unsigned char* box[kMaxWorld];   // mailbox of every rank as mapped in this process (own one included)
    uint32_t* epoch;                 // [0] epoch of the last finished all-reduce, [1] CTAs done in this launch
    unsigned int* status;
    int rank, world;
    uint32_t spin_limit;             // polls before a wait gives up
};

struct P2PState {
    unsigned char* my_box = nullptr;
    void* peer_base[kMaxWorld] = {};
    uint32_t* epoch = nullptr;
    P2PCtx ctx{};
    bool ready = false;
    unsigned char* loop_box[kMaxWorld] = {};   // loopback bring-up: stand-ins for the peers' mailboxes
    uint32_t spin_limit = kSpinLimit;
} p2p;

__device__ __forceinline__ unsigned char* slot_ptr(unsigned char* box, uint32_t bank, int src) {
    return box + ((size_t)bank * kMaxWorld + src) * kSlotBytes;
}
__device__ __forceinline__ uint32_t* flag_ptr(unsigned char* box, uint32_t bank, int src, uint32_t cta) {
    return (uint32_t*)(box + kDataBytes) + ((size_t)bank * kMaxWorld + src) * kMaxCtas + cta;
}

__device__ __forceinline__ uint2* ll_slot_ptr(unsigned char* box, uint32_t bank, int src) {
    return (uint2*)(box + kDataBytes + kFlagBytes + ((size_t)bank * kMaxWorld + src) * kLLSlotBytes);
}

// vecs: number of 16-byte vectors of the fp16 vector.
__global__ void __launch_bounds__(256)
p2p_allreduce_kernel(P2PCtx c, const uint4* in, uint4* out, uint32_t vecs) {   // in == out is allowed
    const uint32_t epoch = c.epoch[0] + 1, bank = epoch & 1u;
    const uint32_t per = (vecs + gridDim.x - 1) / gridDim.x;
    const uint32_t v0 = blockIdx.x * per, v1 = min(v0 + per, vecs);

    // push
    for (uint32_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        const uint4 x = in[v];
        for (int p = 0; p < c.world; p++) ((uint4*)slot_ptr(c.box[p], bank, c.rank))[v] = x;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < (uint32_t)c.world) {
        uint32_t* f = flag_ptr(c.box[threadIdx.x], bank, c.rank, blockIdx.x);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
    // wait
    if (threadIdx.x < (uint32_t)c.world) {
        const uint32_t* f = flag_ptr(c.box[c.rank], bank, (int)threadIdx.x, blockIdx.x);
        uint32_t seen = 0, it = 0;
        for (; it < c.spin_limit; it++) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if ((int32_t)(seen - epoch) >= 0) break;
            __nanosleep(64);
        }
        if (it == c.spin_limit) raise_status(c.status, kStatusAllReduceTimeout);
    }
    __syncthreads();
    // sum, rank order
    for (uint32_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.0f;
        for (int r = 0; r < c.world; r++) {
            const uint4 x = __ldcg((const uint4*)slot_ptr(c.box[c.rank], bank, r) + v);
            const __half2* h = (const __half2*)&x;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(h[i]);
                acc[2 * i] += f.x;
                acc[2 * i + 1] += f.y;
            }
        }
        uint4 o;
        uint32_t* ow = (uint32_t*)&o;
#pragma unroll
        for (int i = 0; i < 4; i++) ow[i] = (uint32_t)f2h(acc[2 * i]) | ((uint32_t)f2h(acc[2 * i + 1]) << 16);
        out[v] = o;
    }
    // last CTA of the launch publishes the epoch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&c.epoch[1], 1u) == gridDim.x - 1) {
            c.epoch[1] = 0;
            __threadfence();
            c.epoch[0] = epoch;
        }
    }
}

// All-reduce of the addend `r` fused with the residual add and the RMSNorm that
// follow a row-parallel projection. One CTA per row. The exchange carries its
// flag inside the data: every 32-bit word of the row travels as an 8-byte
// {word, epoch} pair written with one store (8-byte stores arrive whole), into
// slot [epoch parity][my rank] of every peer's mailbox; the receiver polls the
// pairs of its own mailbox until each carries the epoch. No fence and no
// separate flag round trip: the exchange costs one NVLink write latency. The
// words are added in rank order in fp32 (every rank gets the same bits), the
// reduced row is stored back to `r`, and f16(a + r) is normalised as in
// rmsnorm_kernel. Polls are bounded; a peer that never writes raises the status word.
template <int BLOCK, int WPT>
__global__ void __launch_bounds__(BLOCK)
p2p_add_rmsnorm_kernel(P2PCtx c, const uint16_t* a, uint16_t* r, const uint16_t* __restrict__ g,
                       const uint16_t* __restrict__ b, uint16_t* sum_out, uint16_t* y, uint32_t width) {
    extern __shared__ float row[];  // width floats
    __shared__ double part[BLOCK / 32];
    __shared__ float s_rms;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = c.epoch[0] + 1, bank = epoch & 1u;
    const size_t base = (size_t)blockIdx.x * width;
    const uint32_t words = width / 2;
    const size_t w0 = (size_t)blockIdx.x * words;
    uint32_t* rw = (uint32_t*)(r + base);
    uint32_t mine[WPT];
    // push this rank's words to every peer
#pragma unroll
    for (int j = 0; j < WPT; j++) {
        const uint32_t w = threadIdx.x + j * BLOCK;
        mine[j] = w < words ? rw[w] : 0u;
        if (w < words)
            for (int p = 0; p < c.world; p++) {
                if (p == c.rank) continue;
                uint2* dst = ll_slot_ptr(c.box[p], bank, c.rank) + w0 + w;
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(mine[j]), "r"(epoch) : "memory");
            }
    }
    // collect the peers' words: all loads of a sweep are issued before any is tested
    uint32_t got[kMaxWorld][WPT];
    uint32_t pending = 0;      // bit q * WPT + j
#pragma unroll
    for (int q = 0; q < kMaxWorld; q++)
#pragma unroll
        for (int j = 0; j < WPT; j++) {
            got[q][j] = 0u;
            if (q < c.world && q != c.rank && threadIdx.x + j * BLOCK < words) pending |= 1u << (q * WPT + j);
        }
    for (uint32_t it = 0; pending && it < c.spin_limit; it++) {
        uint2 v[kMaxWorld][WPT];
#pragma unroll
        for (int q = 0; q < kMaxWorld; q++)
#pragma unroll
            for (int j = 0; j < WPT; j++)
                if (pending & (1u << (q * WPT + j))) {
                    const uint2* src = ll_slot_ptr(c.box[c.rank], bank, q) + w0 + threadIdx.x + j * BLOCK;
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[q][j].x), "=r"(v[q][j].y) : "l"(src) : "memory");
                }
#pragma unroll
        for (int q = 0; q < kMaxWorld; q++)
#pragma unroll
            for (int j = 0; j < WPT; j++)
                if ((pending & (1u << (q * WPT + j))) && v[q][j].y == epoch) {
                    got[q][j] = v[q][j].x;
                    pending &= ~(1u << (q * WPT + j));
                }
        if (pending && it > 64) __nanosleep(64);
    }
    if (pending) raise_status(c.status, kStatusAllReduceTimeout);
    // sum in rank order, back into r
#pragma unroll
    for (int j = 0; j < WPT; j++) {
        const uint32_t w = threadIdx.x + j * BLOCK;
        if (w >= words) continue;
        float lo = 0.0f, hi = 0.0f;
#pragma unroll
        for (int q = 0; q < kMaxWorld; q++) {
            if (q >= c.world) break;
            const uint32_t x = q == c.rank ? mine[j] : got[q][j];
            lo += h2f((uint16_t)(x & 0xffffu));
            hi += h2f((uint16_t)(x >> 16));
        }
        rw[w] = (uint32_t)f2h(lo) | ((uint32_t)f2h(hi) << 16);
    }
    __syncthreads();     // the row of r is complete (and visible to this CTA) before the norm reads it
    rmsnorm_row<BLOCK>(a + base, r + base, g, b, sum_out ? sum_out + base : nullptr, y + base, width, row, part, &s_rms);
    // last CTA of the launch publishes the epoch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&c.epoch[1], 1u) == gridDim.x - 1) {
            c.epoch[1] = 0;
            __threadfence();
            c.epoch[0] = epoch;
        }
    }
}

}  // namespace

bool tp_p2p_ready() { return p2p.ready; }

// y = rmsnorm(f16(a + allreduce(r))) with the reduced r and the sum stored too;
// false when the shape does not fit the mailbox (the caller then runs the
// all-reduce and the norm as two launches).
bool tp_p2p_add_rmsnorm(cudaStream_t st, const uint16_t* a, uint16_t* r, const uint16_t* g, const uint16_t* b,
                        uint16_t* sum_out, uint16_t* y, uint32_t rows, uint32_t width) {
    if (!p2p.ready || !rows || (width & 7u) || (size_t)rows * width * 4 > kLLSlotBytes || width > 2 * 512 * 4) return false;
    if ((((uintptr_t)a) | ((uintptr_t)r) | ((uintptr_t)sum_out) | ((uintptr_t)y)) & 15u) return false;
    if (width <= 2 * 512 * 2)
        launch_pdl(p2p_add_rmsnorm_kernel<512, 2>, dim3(rows), dim3(512), width * sizeof(float), st, p2p.ctx, a, r, g, b, sum_out, y, width);
    else
        launch_pdl(p2p_add_rmsnorm_kernel<512, 4>, dim3(rows), dim3(512), width * sizeof(float), st, p2p.ctx, a, r, g, b, sum_out, y, width);
    g_launches++;
    return true;
}

// In-place all-reduce of `elems` fp16 values; false when the vector does not
// fit the mailbox or is not 16-byte sized/aligned (the caller then uses NCCL).
bool tp_p2p_allreduce_f16(cudaStream_t st, void* buf, size_t elems) {
    if (!p2p.ready) return false;
    const size_t bytes = elems * 2;
    if (bytes > kSlotBytes || (bytes & 15) || ((uintptr_t)buf & 15)) return false;
    const uint32_t vecs = (uint32_t)(bytes / 16);
    uint32_t ctas = (vecs + 511) / 512;       // two vectors per thread
    if (ctas < 1) ctas = 1;
    if (ctas > kMaxCtas) ctas = kMaxCtas;
    p2p_allreduce_kernel<<<ctas, 256, 0, st>>>(p2p.ctx, (const uint4*)buf, (uint4*)buf, vecs);
    g_launches++;
    return true;
}

void tp_p2p_shutdown() {
    if (!p2p.my_box) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < kMaxWorld; r++) {
        if (p2p.peer_base[r]) { cudaIpcCloseMemHandle(p2p.peer_base[r]); p2p.peer_base[r] = nullptr; }
        if (p2p.loop_box[r]) { cudaFree(p2p.loop_box[r]); p2p.loop_box[r] = nullptr; }
    }
    const uint32_t keep_limit = p2p.spin_limit;
    cudaFree(p2p.my_box);
    cudaFree(p2p.epoch);
    p2p = P2PState();
    p2p.spin_limit = keep_limit;
}

}  // namespace gehtp

using namespace gehtp;

extern "C" {

int gehtp_cuda_tp_p2p_export(void* handle_out, size_t handle_bytes) {
    if (!handle_out || handle_bytes < sizeof(cudaIpcMemHandle_t)) return -1;
    if (!ensure_device(nullptr, 0)) return -1;
    if (!p2p.my_box) {
        if (cudaMalloc(&p2p.my_box, kBoxBytes) != cudaSuccess || cudaMalloc(&p2p.epoch, 2 * sizeof(uint32_t)) != cudaSuccess) {
            g.last_error = "tp p2p: mailbox allocation failed";
            cudaGetLastError();
            return -1;
        }
        cudaMemset(p2p.my_box, 0, kBoxBytes);
        cudaMemset(p2p.epoch, 0, 2 * sizeof(uint32_t));
        cudaDeviceSynchronize();
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p2p.my_box) != cudaSuccess) {
        g.last_error = "tp p2p: cudaIpcGetMemHandle failed";
        cudaGetLastError();
        return -1;
    }
    std::memcpy(handle_out, &h, sizeof h);
    return 0;
}

int gehtp_cuda_tp_p2p_import(const void* handles, size_t handle_stride, int world) {
    if (!handles || handle_stride < sizeof(cudaIpcMemHandle_t) || world != g.tp_world || world > kMaxWorld) {
        g.last_error = "tp p2p: bad import arguments (world must match tp_init)";
        return -1;
    }
    P2PCtx c{};
    c.rank = g.tp_rank; c.world = world; c.epoch = p2p.epoch; c.status = g.d_status; c.spin_limit = p2p.spin_limit;
    bool mine = p2p.my_box != nullptr;      // a rank whose export failed still takes part in the agreement below
    if (!mine) g.last_error = "tp p2p: this rank has no mailbox (its export failed)";
    for (int r = 0; r < world && mine; r++) {
        if (r == g.tp_rank) { c.box[r] = p2p.my_box; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const unsigned char*)handles + (size_t)r * handle_stride, sizeof h);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            g.last_error = "tp p2p: cudaIpcOpenMemHandle failed (no peer access between the ranks' GPUs?)";
            cudaGetLastError();
            mine = false;
            break;
        }
        p2p.peer_base[r] = p;
        c.box[r] = (unsigned char*)p;
    }
    // Every rank takes the peer-memory path or none does: a rank that fell back to NCCL while its peers post into
    // mailboxes would leave them polling. The ranks agree here (minimum of the flags over the communicator of
    // tp_init), so the caller needs no agreement of its own; which launches are eligible afterwards depends on row
    // count and width only, which are the same on every rank.
    const int all = tp_all_agree(mine ? 1 : 0);
    if (all != 1) {
        for (int r = 0; r < kMaxWorld; r++)
            if (p2p.peer_base[r]) { cudaIpcCloseMemHandle(p2p.peer_base[r]); p2p.peer_base[r] = nullptr; }
        p2p.ready = false;
        if (mine) g.last_error = all < 0 ? "tp p2p: the ranks could not agree (no communicator: call gehtp_cuda_tp_init first)"
                                         : "tp p2p: another rank could not map the mailboxes; all ranks use NCCL";
        if (g.planned) drop_plan(true);
        return -1;
    }
    p2p.ctx = c;
    p2p.ready = true;
    if (g.planned) drop_plan(true);
    return 0;
}

void gehtp_cuda_set_wait_limit(uint32_t polls) {
    p2p.spin_limit = polls ? polls : kSpinLimit;
    p2p.ctx.spin_limit = p2p.spin_limit;
    if (g.planned) drop_plan(true);   // launches (and a captured graph) carry the limit by value
}

int gehtp_cuda_tp_p2p_loopback(int world) {
    if (world < 2 || world > kMaxWorld) { g.last_error = "tp p2p loopback: world must be 2..8"; return -1; }
    if (!ensure_device(nullptr, 0)) return -1;
    if (g.nccl_comm || p2p.ready) { g.last_error = "tp p2p loopback: tensor parallelism is already set up"; return -1; }
    cudaIpcMemHandle_t unused;
    if (gehtp_cuda_tp_p2p_export(&unused, sizeof unused) != 0) return -1;   // allocates this rank's own mailbox
    P2PCtx c{};
    c.rank = 0; c.world = world; c.epoch = p2p.epoch; c.status = g.d_status; c.spin_limit = p2p.spin_limit;
    c.box[0] = p2p.my_box;
    for (int r = 1; r < world; r++) {
        if (cudaMalloc(&p2p.loop_box[r], kBoxBytes) != cudaSuccess) { cudaGetLastError(); g.last_error = "tp p2p loopback: allocation failed"; return -1; }
        cudaMemset(p2p.loop_box[r], 0, kBoxBytes);
        c.box[r] = p2p.loop_box[r];
    }
    cudaDeviceSynchronize();
    g.tp_rank = 0; g.tp_world = world;
    p2p.ctx = c;
    p2p.ready = true;
    if (g.planned) drop_plan(true);
    return 0;
}

void gehtp_cuda_tp_p2p_disable(void) {
    if (!p2p.ready) return;
    p2p.ready = false;
    if (g.planned) drop_plan(true);
}

}  // extern "C"
