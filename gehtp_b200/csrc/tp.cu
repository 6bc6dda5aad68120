// Tensor parallelism inside one node: the engine owns an NCCL communicator and
// queues an all-reduce on its own stream after the ops the caller names. The
// runlist of each rank is already sharded (column-parallel projections carry
// N/world columns, row-parallel ones K/world rows); which op outputs are partial
// sums comes from the blob's sideband manifest, not from the blob itself.
#include <cstdio>
#include <cstring>
#include <nccl.h>
#include "engine.h"

namespace gehtp {
std::vector<uint8_t> g_allreduce_after;   // per op: 1 = all-reduce its first output
}
using namespace gehtp;

extern "C" {

int gehtp_cuda_tp_unique_id(void* out_id, size_t id_bytes) {
    if (!out_id || id_bytes < sizeof(ncclUniqueId)) return -1;
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return -1;
    std::memcpy(out_id, &id, sizeof id);
    return 0;
}

int gehtp_cuda_tp_init(int rank, int world, const void* nccl_unique_id, size_t id_bytes) {
    if (world < 1 || rank < 0 || rank >= world) return -1;
    if (!ensure_device(nullptr, 0)) return -1;
    g.tp_rank = rank; g.tp_world = world;
    if (world == 1) return 0;
    if (!nccl_unique_id || id_bytes < sizeof(ncclUniqueId)) return -1;
    ncclUniqueId id;
    std::memcpy(&id, nccl_unique_id, sizeof id);
    ncclComm_t comm = nullptr;
    if (ncclCommInitRank(&comm, world, id, rank) != ncclSuccess) { g.last_error = "ncclCommInitRank failed"; return -1; }
    g.nccl_comm = comm;
    return 0;
}

void gehtp_cuda_tp_shutdown(void) {
    tp_p2p_shutdown();
    if (g.nccl_comm) { ncclCommDestroy((ncclComm_t)g.nccl_comm); g.nccl_comm = nullptr; }
    g.tp_world = 1; g.tp_rank = 0;
    g_allreduce_after.clear();
}

int gehtp_cuda_tp_allreduce_after(const uint32_t* op_idx, uint32_t n) {
    g_allreduce_after.clear();
    for (uint32_t i = 0; i < n; i++) {
        if (op_idx[i] >= WT_MAX_OPS) return -1;
        if (g_allreduce_after.size() <= op_idx[i]) g_allreduce_after.resize(op_idx[i] + 1, 0);
        g_allreduce_after[op_idx[i]] = 1;
    }
    if (g.planned) drop_plan(true);
    return 0;
}

}  // extern "C"

namespace gehtp {
// In-place fp16 sum over the ranks, queued on `st`.
int tp_allreduce_f16(cudaStream_t st, void* buf, size_t elems) {
    if (g.tp_world <= 1) return 0;
    if (tp_p2p_allreduce_f16(st, buf, elems)) return 0;   // small vectors: one kernel over peer memory
    if (!g.nccl_comm) return -1;
    ncclResult_t r = ncclAllReduce(buf, buf, elems, ncclHalf, ncclSum, (ncclComm_t)g.nccl_comm, st);
    return r == ncclSuccess ? 0 : -1;
}

// Minimum of a flag over the ranks (NCCL, blocking): 1 only if every rank passed 1. -1: no communicator.
int tp_all_agree(int mine) {
    if (g.tp_world <= 1) return mine ? 1 : 0;
    if (!g.nccl_comm) return -1;
    int* d = nullptr;
    if (cudaMalloc(&d, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    int v = mine ? 1 : 0;
    cudaMemcpyAsync(d, &v, sizeof v, cudaMemcpyHostToDevice, g.stream);
    const ncclResult_t r = ncclAllReduce(d, d, 1, ncclInt32, ncclMin, (ncclComm_t)g.nccl_comm, g.stream);
    cudaMemcpyAsync(&v, d, sizeof v, cudaMemcpyDeviceToHost, g.stream);
    const cudaError_t e = cudaStreamSynchronize(g.stream);
    cudaFree(d);
    return (r == ncclSuccess && e == cudaSuccess) ? v : -1;
}
}  // namespace gehtp
