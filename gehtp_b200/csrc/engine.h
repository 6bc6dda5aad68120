// Engine state shared by the executor's translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <functional>
#include <map>
#include <string>
#include <vector>
#include "gehtp_cuda.h"
#include "launchers.h"
#include "launchers_w4.h"

namespace gehtp {

constexpr uint32_t kMaxTemps = WT_EXEC_MAX_TEMPS;
constexpr uint32_t kNoOff = 0xFFFFFFFFu;

struct KvGeom {
    bool ready = false;
    uint32_t slot_bytes = 0, nslots = 0;
    uint32_t* posmap = nullptr;  // device, nslots entries
};

struct W4Epilogue;

// One runlist op after planning: resolved device pointers baked into `launch`.
struct PlanOp {
    int rc = 0;                 // non-zero: the op fails when reached, with `err`
    std::string err;
    std::function<void(cudaStream_t)> launch;
    std::function<void(cudaStream_t)> launch_local;   // tensor parallel: the op without the all-reduce of its output
    uint32_t engine = WT_ENG_SCALAR;
    uint32_t out_id[2] = {kNoOff, kNoOff};   // temps written, for last-bytes tracking
    uint32_t out_bytes[2] = {0, 0};
    int kv_append_state = -1;   // AUTO append: host counter check / bump
    int kv_gather_state = -1;   // AUTO gather: host counter check
    uint32_t w4_m = 0;          // M of a W4A16 matmul (reported through engine_m)
    // a W4A16 matmul at GEMM row counts: the tcgen05 GEMM with an epilogue of the caller's (false: shape not taken)
    // `a_src` / `a_d` != 0: read the activations from a_src, stored [K / a_d][M][a_d], instead of the op's own operand
    std::function<bool(cudaStream_t, const W4Epilogue&, const uint16_t* a_src, uint32_t a_d)> launch_w4_gemm;
    // fusion: when `fused` is set on op i, it replaces ops [i, i + span)
    std::function<void(cudaStream_t)> fused;
    uint32_t span = 0;
    uint32_t stat = 0;          // index into the stats struct, 0 = none
    bool uses_internal = false; // touches a temp that has no memory in a fused plan
    bool dead_when_fused = false;   // its result is read only by ops that fused chains replace: skipped in whole fused runs
    // a data-movement op whose inputs are weight slots (or results of such ops) and whose output nobody else writes:
    // its result is a constant of the blob, made by the first run that reaches it and kept
    bool const_fold = false, const_done = false;
};

struct W4Packed {
    uint32_t* packed = nullptr;   // device, K*N/2 bytes, strip-major layout
    const uint16_t* scales = nullptr;  // device, [K/64][N], inside the uploaded slot
    uint32_t K = 0, N = 0;
};

struct Engine {
    bool dev_ok = false;
    int device = -1;
    cudaStream_t stream = nullptr;
    std::string last_error;

    // identity of the planned blob
    const wt_blob* blob = nullptr;
    const uint8_t* blob_wbase = nullptr;
    uint32_t blob_nops = 0, blob_nslots = 0;
    bool planned = false;

    uint8_t* d_weights = nullptr;
    size_t weights_bytes = 0;
    std::map<uint32_t, uint8_t*> d_ext;        // EXT_IN / EXT_WGT slots: own buffers
    std::map<uint64_t, W4Packed> w4;            // key = slot | K<<16 ... see executor.cu

    uint8_t* d_arena = nullptr;
    size_t arena_bytes = 0;
    uint8_t* temp_dev[kMaxTemps];
    uint32_t temp_cap[kMaxTemps];
    uint32_t temp_last[kMaxTemps];

    // TEMPOFF table / wt_exec_pool_init
    bool have_static = false;
    uint32_t static_cap = 0, vtcm_cap = 0;
    size_t vtcm_base = 0;               // arena offset of the on-chip-resident region
    uint32_t static_off[kMaxTemps], vtcm_off[kMaxTemps];
    bool user_pool = false;
    uint32_t user_total = 0, user_static = 0;
    std::vector<uint32_t> user_off;

    // persistent states
    bool states_loaded = false;
    uint32_t n_states = 0;
    uint8_t* st_buf[WT_MAX_STATES];
    uint32_t st_bytes[WT_MAX_STATES];
    uint32_t st_count[WT_MAX_STATES];   // host mirror of the AUTO position counters
    uint32_t* d_st_count = nullptr;     // device: WT_MAX_STATES counters, then WT_MAX_STATES arrival counts of the merge kernel
    KvGeom kv[WT_MAX_STATES];

    unsigned int* d_status = nullptr;   // first failing op (1-based) raised by a kernel
    unsigned int* h_status = nullptr;   // pinned

    std::vector<PlanOp> plan;
    uint32_t fused_ops = 0;
    uint32_t const_ops = 0;       // ops of the current plan whose result is made once (const_fold)
    uint32_t demoted_temps = 0;

    // I/O staging
    uint8_t* h_in = nullptr;  size_t h_in_cap = 0;    // pinned
    uint8_t* h_out = nullptr; size_t h_out_cap = 0;   // pinned
    std::map<uint32_t, std::pair<uint8_t*, size_t>> mirrors;  // wt_exec_temp host views
    const uint8_t* ext_in = nullptr;
    const uint8_t* ext_in_dev = nullptr;
    const uint8_t* ext_wgt = nullptr;

    // CUDA graph of a whole run
    cudaGraphExec_t graph = nullptr;
    uint32_t graph_out_temp = kNoOff;
    bool graph_has_in = false, graph_has_out = false;
    uint32_t warm_runs = 0;
    unsigned long long graph_launches = 0;  // kernels inside the captured graph

    // per-unit CUDA event profiling (gehtp_cuda_run_profiled)
    struct ProfEvent { uint32_t op; cudaEvent_t e0, e1; };
    float* prof_ms = nullptr;
    std::vector<ProfEvent> prof_events;
    float prof_attn_ms = 0.0f;      // decode attention kernel alone, last profiled run
    uint32_t prof_attn_n = 0;

    // options
    int opt_fuse = 1, opt_graph = 1, trace_on = 0;
    bool exact_ops = false;       // a dump hook is active: matmuls keep the reference's summation order
    bool skip_dead = false;       // set for the duration of a whole fused run
    bool force_unfused = false;   // a run needed an op that the fused plan gave no memory
    const char* hook_spec = nullptr;
    wt_op_ts* ts_buf = nullptr;
    uint32_t ts_cap = 0;
    wt_exec_stats st{};

    // tensor parallel
    int tp_rank = 0, tp_world = 1;
    void* nccl_comm = nullptr;
};

extern Engine g;

// executor.cu
bool ensure_device(char* err, size_t errn);
int status_message(unsigned int code, char* msg, size_t msg_bytes);
int read_status(char* err, size_t errn);   // after a stream sync: 0, or the failed run's return value with last_error set
// plan.cu
int build_plan(const wt_blob* b, char* err, size_t errn);
void drop_plan(bool keep_states);
// tp.cu
extern std::vector<uint8_t> g_allreduce_after;   // per op: 1 = all-reduce its first output over the ranks
// Fewest rows for which a W4A16 matmul goes to the tcgen05 GEMM (TMA zero-fills the rows a 128-row tile has
// beyond M; with few tiles K is split over the SMs); below it the streaming kernel runs, which re-reads and
// re-dequantises the weights once per 16 or 32 rows. Measured at 64 rows, Qwen3-4B shapes: the batch-64 decode step
// 18.8 -> 18.0 ms with the GEMM. $GEHTP_CUDA_GEMM_MIN_M moves the switch (>= 17).
inline uint32_t w4_gemm_min_rows() {
    static const uint32_t v = [] { const char* e = std::getenv("GEHTP_CUDA_GEMM_MIN_M"); int x = e ? std::atoi(e) : 64; return (uint32_t)(x >= 17 ? x : 64); }();
    return v;
}
int tp_allreduce_f16(cudaStream_t st, void* buf, size_t elems);
int tp_all_agree(int mine);
// tp_p2p.cu
bool tp_p2p_ready();
bool tp_p2p_allreduce_f16(cudaStream_t st, void* buf, size_t elems);
void tp_p2p_shutdown();
bool tp_p2p_add_rmsnorm(cudaStream_t st, const uint16_t* a, uint16_t* r, const uint16_t* g, const uint16_t* b,
                        uint16_t* sum_out, uint16_t* y, uint32_t rows, uint32_t width);
// fuse.cu
void fuse_analyze(const wt_blob* b, const std::vector<PlanOp>& meas, std::vector<uint8_t>& internal, std::vector<uint8_t>& dead);
void fuse_materialize(const wt_blob* b);
// Marks the ops whose result is a constant of the blob (PlanOp::const_fold). addr / maxb: device address and capacity
// of every temp id of the plan.
void fold_constants(const wt_blob* b, uint8_t* const* addr, const uint64_t* maxb);
bool fuse_all_materialized();
void fuse_release();

}  // namespace gehtp
