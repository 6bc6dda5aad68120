// The wt_exec_* C API on CUDA: device set-up, the run loop over a planned op
// list, host<->device I/O staging, per-op timing / hooks / traces, whole-run
// CUDA graphs. Mirrors the calling contract of the reference engine
// (kernels/src/runtime/oplist_exec.c:2499-2602; kernels/include/oplist_exec.h).
#include <cuda_fp16.h>
#include <fcntl.h>
#include <unistd.h>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>
#include "common.cuh"
#include "engine.h"
#include "launchers_attn.h"

namespace gehtp {

Engine g;

static int64_t now_us() {
    return std::chrono::duration_cast<std::chrono::microseconds>(
               std::chrono::steady_clock::now().time_since_epoch()).count();
}

static void set_err(char* err, size_t errn, const char* msg) {
    g.last_error = msg;
    if (err && errn) std::snprintf(err, errn, "%s", msg);
}

bool ensure_device(char* err, size_t errn) {
    if (g.dev_ok) { cudaSetDevice(g.device); return true; }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); set_err(err, errn, "no CUDA device"); return false; }
    int dev = g.device;
    if (dev < 0) { const char* e = std::getenv("GEHTP_CUDA_DEVICE"); dev = e ? std::atoi(e) : 0; }
    if (dev >= n || cudaSetDevice(dev) != cudaSuccess) { set_err(err, errn, "no CUDA device"); return false; }
    g.device = dev;
    if (cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking) != cudaSuccess) { set_err(err, errn, "no CUDA device"); return false; }
    cudaMalloc(&g.d_st_count, 2 * WT_MAX_STATES * sizeof(uint32_t));
    cudaMemset(g.d_st_count, 0, 2 * WT_MAX_STATES * sizeof(uint32_t));
    cudaMalloc(&g.d_status, sizeof(unsigned int));
    cudaMemset(g.d_status, 0, sizeof(unsigned int));
    cudaMallocHost(&g.h_status, sizeof(unsigned int));
    *g.h_status = 0;
    if (const char* e = std::getenv("GEHTP_CUDA_FUSE")) g.opt_fuse = std::atoi(e);
    if (const char* e = std::getenv("GEHTP_CUDA_GRAPH")) g.opt_graph = std::atoi(e);
    for (uint32_t i = 0; i < kMaxTemps; i++) { g.temp_dev[i] = nullptr; g.temp_cap[i] = 0; g.temp_last[i] = 0; g.static_off[i] = kNoOff; g.vtcm_off[i] = kNoOff; }
    g.dev_ok = true;
    return true;
}

static void grow_pinned(uint8_t*& p, size_t& cap, size_t need) {
    if (need <= cap) return;
    if (p) cudaFreeHost(p);
    cap = (need + 4095) / 4096 * 4096;
    if (cudaMallocHost(&p, cap) != cudaSuccess) { p = nullptr; cap = 0; }
}

// "opidx:temp,opidx:temp" dump after op `ii` of the current range
// (exec_hook_dump, oplist_exec.c:117-166).
static void hook_dump(uint32_t ii) {
    static const char* env_hook = nullptr;
    static bool env_tried = false;
    const char* hook = g.hook_spec;
    if (!hook) {
        if (!env_tried) { env_hook = std::getenv("GEHTP_HOOK"); env_tried = true; }
        hook = env_hook;
    }
    if (!hook || !hook[0]) return;
    const char* tok = hook;
    while (*tok) {
        const char* comma = std::strchr(tok, ',');
        size_t len = comma ? (size_t)(comma - tok) : std::strlen(tok);
        std::string item(tok, len);
        size_t col = item.rfind(':');
        if (col != std::string::npos) {
            uint32_t hi = (uint32_t)std::strtoul(item.substr(0, col).c_str(), nullptr, 0);
            uint32_t ht = (uint32_t)std::strtoul(item.substr(col + 1).c_str(), nullptr, 0);
            if (hi == ii && ht < kMaxTemps && g.temp_cap[ht]) {
                uint32_t nbytes = g.temp_last[ht];
                std::vector<uint8_t> host(nbytes);
                cudaStreamSynchronize(g.stream);
                cudaMemcpy(host.data(), g.temp_dev[ht], nbytes, cudaMemcpyDeviceToHost);
                char fn[128];
                std::snprintf(fn, sizeof fn, "/tmp/hook_%u_%u.f16.raw", hi, ht);
                int fd = open(fn, O_WRONLY | O_CREAT | O_TRUNC, 0666);
                if (fd >= 0) {
                    size_t off = 0;
                    while (off < nbytes) {
                        ssize_t w = write(fd, host.data() + off, nbytes - off);
                        if (w <= 0) break;
                        off += (size_t)w;
                    }
                    close(fd);
                }
            }
        }
        if (!comma) break;
        tok = comma + 1;
    }
}

static FILE* g_trace_fp = nullptr;
// Per-op trace lines in the reference's format (oplist_exec.c:2521-2561):
//   pre<ii> code=<opcode> a=<arg0>,<arg1>,<arg2>,<arg3> pool=<bytes>     before the op
//   op<ii> code=<opcode> rc=<rc> us=<host microseconds, -1 without op_us>  after it
// appended to $GEHTP_TRACE_FILE (default /tmp/gehtp_optrace.txt). The file is reopened when the
// variable changes.
static std::string g_trace_name;
static FILE* trace_file() {
    const char* fn = std::getenv("GEHTP_TRACE_FILE");
    const std::string want = fn ? fn : "/tmp/gehtp_optrace.txt";
    if (g_trace_fp && want != g_trace_name) { std::fclose(g_trace_fp); g_trace_fp = nullptr; }
    if (!g_trace_fp) { g_trace_fp = std::fopen(want.c_str(), "a"); g_trace_name = want; }
    return g_trace_fp;
}
static void trace_pre(uint32_t ii, const wt_op& op) {
    if (FILE* f = trace_file()) {
        std::fprintf(f, "pre%u code=%u a=%u,%u,%u,%u pool=%u\n", ii, (unsigned)op.opcode, op.args[0], op.args[1], op.args[2],
                     op.args[3], (unsigned)g.arena_bytes);
        std::fflush(f);
    }
}
static void trace_post(uint32_t ii, const wt_op& op, int rc, long long us) {
    if (FILE* f = trace_file()) {
        std::fprintf(f, "op%u code=%u rc=%d us=%lld\n", ii, (unsigned)op.opcode, rc, us);
        std::fflush(f);
    }
}

static bool hooks_active() {
    if (g.hook_spec) return g.hook_spec[0] != 0;
    const char* e = std::getenv("GEHTP_HOOK");
    return e && e[0];
}

static void bump_stat(uint32_t stat) {
    uint32_t* f = &g.st.ops;
    if (stat) f[stat - 1]++;
    if (stat == 6) g.st.pin_skipped++;  // there is no on-chip weight cache to fill
}

static int ensure_plan(const wt_blob* b, char* err, size_t errn) {
    if (g.planned && (g.blob != b || g.blob_wbase != b->weight_base || g.blob_nops != b->n_ops ||
                      g.blob_nslots != b->n_slots)) {
        drop_plan(true);
        g.force_unfused = false;
    }
    if (g.planned) return 0;
    int rc = build_plan(b, err, errn);
    if (rc != 0) { drop_plan(true); if (err) g.last_error = err; }
    return rc;
}

// Host-side part of an op that the device cannot check before it is queued:
// the AUTO position counters of the KV states (oplist_exec.c:2166-2173, 2198-2207).
static int host_precheck(const PlanOp& p, char* err, size_t errn) {
    char m[160];
    if (p.kv_append_state >= 0) {
        uint32_t si = (uint32_t)p.kv_append_state;
        if (g.st_count[si] >= g.kv[si].nslots) {
            std::snprintf(m, sizeof m, "kv append state %u count=%u >= nslots=%u (context too long)", si, g.st_count[si], g.kv[si].nslots);
            set_err(err, errn, m);
            return -1;
        }
        g.st_count[si]++;
    }
    if (p.kv_gather_state >= 0) {
        uint32_t si = (uint32_t)p.kv_gather_state;
        if (g.st_count[si] == 0u || g.st_count[si] > g.kv[si].nslots) {
            std::snprintf(m, sizeof m, "kv gather state %u count=%u bad (append first?)", si, g.st_count[si]);
            set_err(err, errn, m);
            return -1;
        }
    }
    return 0;
}

static void note_outputs(const PlanOp& p) {
    for (int k = 0; k < 2; k++) {
        uint32_t id = p.out_id[k];
        if (id == kNoOff) continue;
        g.temp_last[id] = p.out_bytes[k];
        if (g.temp_cap[id] < p.out_bytes[k]) g.temp_cap[id] = p.out_bytes[k];
    }
}

constexpr int kNeedUnfused = -1000;

// Queues ops [first, first+count) on the engine stream. Returns 0 or the
// 1-based index of the op that failed before launch.
static int queue_range(uint32_t first, uint32_t count, bool fuse, bool per_op_sync, uint32_t* engine_m,
                       int64_t* op_us, char* err, size_t errn) {
    const int64_t t_run0 = now_us();
    const bool hooks = hooks_active();
    std::vector<PlanOp*> pending;
    cudaStreamCaptureStatus cap_state = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(g.stream, &cap_state) != cudaSuccess || cap_state != cudaStreamCaptureStatusNone;
    if (hooks) fuse = false;   // dumps need every intermediate temp
    g.exact_ops = hooks;
    for (uint32_t ii = 0; ii < count;) {
        const uint32_t i = first + ii;
        PlanOp& p = g.plan[i];
        uint32_t span = 1;
        const bool use_fused = fuse && p.fused && p.span >= 1 && ii + p.span <= count;
        if (use_fused) span = p.span;
        const int64_t t0 = now_us();
        int rc = 0;
        uint32_t fail = i;
        if (g.trace_on) for (uint32_t k = 0; k < span; k++) trace_pre(ii + k, g.blob->ops[i + k]);
        for (uint32_t k = 0; k < span && !rc; k++) {
            PlanOp& q = g.plan[i + k];
            if (!use_fused && q.uses_internal) return kNeedUnfused;
            if (q.rc) { set_err(err, errn, q.err.c_str()); rc = -1; fail = i + k; break; }
            if (host_precheck(q, err, errn)) { rc = -1; fail = i + k; break; }
            if (q.w4_m) *engine_m = q.w4_m;
            bump_stat(q.stat);
            g.st.ops++;
            note_outputs(q);
            pending.push_back(&q);
        }
        {
            cudaEvent_t ev0 = nullptr, ev1 = nullptr;
            if (g.prof_ms && !rc) {
                cudaEventCreate(&ev0); cudaEventCreate(&ev1);
                g.prof_events.push_back({i, ev0, ev1});
                cudaEventRecord(ev0, g.stream);
            }
            if (!rc) {
                if (use_fused) p.fused(g.stream);
                else for (PlanOp* q : pending) {
                    if (!q->launch || (g.skip_dead && q->dead_when_fused)) continue;
                    if (q->const_fold && q->const_done) continue;        // a constant of the blob, made by an earlier run
                    q->launch(g.stream);
                    if (q->const_fold && !capturing) q->const_done = true;   // inside a capture the launch has not run yet
                }
            }
            if (ev1) cudaEventRecord(ev1, g.stream);
            pending.clear();
        }

        if (!rc && (per_op_sync || hooks)) {
            cudaError_t ce = cudaStreamSynchronize(g.stream);
            if (ce != cudaSuccess) { set_err(err, errn, cudaGetErrorString(ce)); rc = -1; }
        }
        if (!rc && hooks) for (uint32_t k = 0; k < span; k++) hook_dump(ii + k);
        const int64_t t1 = now_us();
        for (uint32_t k = 0; k < span; k++) {
            if (op_us) op_us[ii + k] = k == 0 ? t1 - t0 : 0;
            if (g.ts_buf && i + k < g.ts_cap) {
                wt_op_ts& ts = g.ts_buf[i + k];
                ts.start_us = (uint32_t)(t0 - t_run0);
                ts.dur_us = k == 0 ? (uint32_t)(t1 - t0) : 0;
                ts.dma_us = 0; ts.dma_bytes = 0;
                ts.engine = g.plan[i + k].engine;
            }
        }
        if (g.trace_on)
            for (uint32_t k = 0; k < span && i + k <= fail; k++)
                trace_post(ii + k, g.blob->ops[i + k], (rc && i + k == fail) ? rc : 0, op_us ? (long long)op_us[ii + k] : -1);
        if (rc) return (int)fail + 1;
        ii += span;
    }
    return 0;
}

// Device status word -> error string and return value. A KV gather that found another
// position in its ring slot leaves the 1-based index of its op, which is also the run's
// return value (oplist_exec.c:2562); a bounded wait that ran out inside a kernel cannot be
// pinned on one op and returns -1, the reference's value for engine-level failures (:2504-2506).
int status_message(unsigned int code, char* m, size_t mn) {
    switch (code) {
    case kStatusAllReduceTimeout:
        std::snprintf(m, mn, "tensor-parallel all-reduce timed out waiting for a peer rank");
        return -1;
    case kStatusAttnTimeout:
        std::snprintf(m, mn, "decode attention timed out waiting for a K/V tile copy");
        return -1;
    case kStatusGemmTimeout:
        std::snprintf(m, mn, "tcgen05 GEMM timed out on a pipeline barrier (output incomplete)");
        return -1;
    default:
        if (code & 0x80000000u) { std::snprintf(m, mn, "device status 0x%08x", code); return -1; }
        std::snprintf(m, mn, "kv gather miss (state bug) at op %u", code - 1);
        return (int)code;
    }
}

// Ends a run: waits for the stream and turns a device-raised status into the
// reference's error return.
static int finish_run(char* err, size_t errn) {
    cudaMemcpyAsync(g.h_status, g.d_status, sizeof(unsigned int), cudaMemcpyDeviceToHost, g.stream);
    cudaError_t ce = cudaStreamSynchronize(g.stream);
    if (ce != cudaSuccess) { set_err(err, errn, cudaGetErrorString(ce)); return -1; }
    if (*g.h_status) {
        unsigned int code = *g.h_status;
        *g.h_status = 0;
        cudaMemsetAsync(g.d_status, 0, sizeof(unsigned int), g.stream);
        char m[128];
        const int rc = status_message(code, m, sizeof m);
        set_err(err, errn, m);
        return rc;
    }
    return 0;
}

int read_status(char* err, size_t errn) {
    unsigned int code = 0;
    if (!g.d_status || cudaMemcpy(&code, g.d_status, sizeof code, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (!code) return 0;
    cudaMemset(g.d_status, 0, sizeof code);
    char m[128];
    const int rc = status_message(code, m, sizeof m);
    set_err(err, errn, m);
    return rc;
}

static void stage_inputs(const wt_blob* b, const void* in_host, const void* in_dev) {
    for (auto& kv : g.d_ext) {
        const wt_slot& sl = b->slots[kv.first];
        if (sl.addr != WT_SLOT_EXT_IN) continue;
        if (in_host) {
            grow_pinned(g.h_in, g.h_in_cap, sl.len);
            std::memcpy(g.h_in, in_host, sl.len);
            cudaMemcpyAsync(kv.second, g.h_in, sl.len, cudaMemcpyHostToDevice, g.stream);
        } else if (in_dev) {
            cudaMemcpyAsync(kv.second, in_dev, sl.len, cudaMemcpyDeviceToDevice, g.stream);
        }
    }
}

static int run_impl(const wt_blob* b, uint32_t first, uint32_t count, const void* in_host,
                    const void* in_dev, void* out_host, void* out_dev, uint32_t out_temp, bool sync_end,
                    uint32_t* engine_m, int64_t* op_us, char* err, size_t errn) {
    uint32_t dummy_m = 0;
    if (!engine_m) engine_m = &dummy_m;
    *engine_m = 0;
    if (!b) { set_err(err, errn, "null blob"); return -1; }
    if (!ensure_device(err, errn)) return -1;
    if ((uint64_t)first + count > b->n_ops) { set_err(err, errn, "range oob"); return -1; }
    if (ensure_plan(b, err, errn) != 0) return -1;

    const bool timing = op_us || g.ts_buf;
    const bool whole = first == 0 && count == b->n_ops;
    const bool has_in = in_host || in_dev;
    const bool eager_only = timing || hooks_active() || g.trace_on || !g.opt_graph || !whole || g.prof_ms;

    int rc = 0;
    // Device-side input and output copies stay outside the graph (their pointers
    // may change from run to run); host staging goes through fixed pinned buffers
    // and is part of it.
    if (!eager_only && g.graph && (g.graph_out_temp != out_temp || g.graph_has_in != (in_host != nullptr) ||
                                   g.graph_has_out != (out_host != nullptr))) {
        cudaGraphExecDestroy(g.graph);   // same blob, different I/O binding: capture again
        g.graph = nullptr;
    }
    if (!eager_only && g.graph) {
        // replay: host bookkeeping first, then one launch
        for (uint32_t i = 0; i < b->n_ops; i++) {
            PlanOp& q = g.plan[i];
            if (q.rc) { set_err(err, errn, q.err.c_str()); return (int)i + 1; }
            if (host_precheck(q, err, errn)) return (int)i + 1;
            if (q.w4_m) *engine_m = q.w4_m;
            bump_stat(q.stat);
            g.st.ops++;
            note_outputs(q);
        }
        if (in_host) {
            for (auto& kv : g.d_ext)
                if (b->slots[kv.first].addr == WT_SLOT_EXT_IN) std::memcpy(g.h_in, in_host, b->slots[kv.first].len);
        }
        if (in_dev) stage_inputs(b, nullptr, in_dev);
        cudaGraphLaunch(g.graph, g.stream);
        g_launches += g.graph_launches;
        if (out_dev && out_temp < kMaxTemps && g.temp_cap[out_temp])
            cudaMemcpyAsync(out_dev, g.temp_dev[out_temp], g.temp_last[out_temp], cudaMemcpyDeviceToDevice, g.stream);
        if (!sync_end) return 0;
        rc = finish_run(err, errn);
        if (rc == 0 && out_host && out_temp < kMaxTemps) std::memcpy(out_host, g.h_out, g.temp_last[out_temp]);
        return rc;
    }

    // a run that could be graphed later is captured on its second eager pass
    const bool capture = !eager_only && !g.graph && g.warm_runs >= 1;
    uint32_t out_bytes_planned = 0;
    if (capture) {
        if (in_host)
            for (auto& kv : g.d_ext)
                if (b->slots[kv.first].addr == WT_SLOT_EXT_IN) grow_pinned(g.h_in, g.h_in_cap, b->slots[kv.first].len);
        if (out_host && out_temp < kMaxTemps) {
            // the size the output temp has after a whole run is known from the previous run
            out_bytes_planned = g.temp_last[out_temp];
            grow_pinned(g.h_out, g.h_out_cap, out_bytes_planned ? out_bytes_planned : 4);
        }
        if (in_dev) stage_inputs(b, nullptr, in_dev);
        if (cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            g.opt_graph = 0;
            return run_impl(b, first, count, in_host, in_dev, out_host, out_dev, out_temp, sync_end, engine_m, op_us, err, errn);
        }
    }
    const unsigned long long launches0 = g_launches;
    if (capture) { if (in_host) stage_inputs(b, in_host, nullptr); }
    else if (has_in) stage_inputs(b, in_host, in_dev);
    g.skip_dead = whole && g.opt_fuse != 0 && !hooks_active();
    rc = queue_range(first, count, g.opt_fuse != 0, timing, engine_m, op_us, err, errn);
    g.skip_dead = false;
    if (rc == kNeedUnfused) {
        // an op inside a fused chain has to run on its own: plan again with every temp in memory
        if (capture) { cudaGraph_t gr = nullptr; cudaStreamEndCapture(g.stream, &gr); if (gr) cudaGraphDestroy(gr); cudaGetLastError(); }
        cudaStreamSynchronize(g.stream);
        g.force_unfused = true;
        auto old_ext = std::move(g.d_ext);   // injected inputs and temps written so far outlive the re-plan
        g.d_ext.clear();
        uint8_t* old_arena = g.d_arena;
        g.d_arena = nullptr;
        std::vector<uint8_t*> old_dev(g.temp_dev, g.temp_dev + kMaxTemps);
        std::vector<uint32_t> old_cap(g.temp_cap, g.temp_cap + kMaxTemps), old_last(g.temp_last, g.temp_last + kMaxTemps);
        drop_plan(true);
        int prc = ensure_plan(b, err, errn);
        for (uint32_t t = 0; prc == 0 && t < kMaxTemps; t++) {
            if (!old_cap[t] || !old_dev[t] || !g.temp_dev[t]) continue;
            cudaMemcpyAsync(g.temp_dev[t], old_dev[t], old_cap[t], cudaMemcpyDeviceToDevice, g.stream);
            g.temp_cap[t] = old_cap[t];
            g.temp_last[t] = old_last[t];
        }
        for (auto& kv : old_ext) {
            auto it = g.d_ext.find(kv.first);
            if (prc == 0 && it != g.d_ext.end())
                cudaMemcpyAsync(it->second, kv.second, b->slots[kv.first].len, cudaMemcpyDeviceToDevice, g.stream);
        }
        cudaStreamSynchronize(g.stream);
        for (auto& kv : old_ext) cudaFree(kv.second);
        if (old_arena) cudaFree(old_arena);
        if (prc != 0) return -1;
        return run_impl(b, first, count, in_host, in_dev, out_host, out_dev, out_temp, sync_end, engine_m, op_us, err, errn);
    }
    if (capture) {
        if (rc == 0 && out_host && out_temp < kMaxTemps && g.temp_cap[out_temp])
            cudaMemcpyAsync(g.h_out, g.temp_dev[out_temp], g.temp_last[out_temp], cudaMemcpyDeviceToHost, g.stream);
        cudaGraph_t graph = nullptr;
        cudaError_t ce = cudaStreamEndCapture(g.stream, &graph);
        if (rc != 0 || ce != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            g.opt_graph = 0;  // this blob cannot be graphed; stay eager
            if (rc != 0) return rc;
            // host counters were advanced while capturing: undo, then run eagerly
            for (uint32_t i = 0; i < b->n_ops; i++)
                if (g.plan[i].kv_append_state >= 0) g.st_count[g.plan[i].kv_append_state]--;
            return run_impl(b, first, count, in_host, in_dev, out_host, out_dev, out_temp, sync_end, engine_m, op_us, err, errn);
        }
        ce = cudaGraphInstantiate(&g.graph, graph, 0);
        cudaGraphDestroy(graph);
        if (ce != cudaSuccess) {
            g.graph = nullptr; g.opt_graph = 0; cudaGetLastError();
            for (uint32_t i = 0; i < b->n_ops; i++)
                if (g.plan[i].kv_append_state >= 0) g.st_count[g.plan[i].kv_append_state]--;
            return run_impl(b, first, count, in_host, in_dev, out_host, out_dev, out_temp, sync_end, engine_m, op_us, err, errn);
        }
        g.graph_launches = g_launches - launches0;
        g.graph_out_temp = out_temp; g.graph_has_in = in_host != nullptr; g.graph_has_out = out_host != nullptr;
        cudaGraphLaunch(g.graph, g.stream);
        if (out_dev && out_temp < kMaxTemps && g.temp_cap[out_temp])
            cudaMemcpyAsync(out_dev, g.temp_dev[out_temp], g.temp_last[out_temp], cudaMemcpyDeviceToDevice, g.stream);
        if (!sync_end) return 0;
        rc = finish_run(err, errn);
        if (rc == 0 && out_host && out_temp < kMaxTemps) std::memcpy(out_host, g.h_out, g.temp_last[out_temp]);
        return rc;
    }
    if (rc != 0) { cudaStreamSynchronize(g.stream); return rc; }
    if (whole) g.warm_runs++;
    if (out_dev && out_temp < kMaxTemps && g.temp_cap[out_temp])
        cudaMemcpyAsync(out_dev, g.temp_dev[out_temp], g.temp_last[out_temp], cudaMemcpyDeviceToDevice, g.stream);
    if (out_host && out_temp < kMaxTemps && g.temp_cap[out_temp]) {
        grow_pinned(g.h_out, g.h_out_cap, g.temp_last[out_temp]);
        cudaMemcpyAsync(g.h_out, g.temp_dev[out_temp], g.temp_last[out_temp], cudaMemcpyDeviceToHost, g.stream);
    }
    if (!sync_end) return 0;
    rc = finish_run(err, errn);
    if (rc == 0 && out_host && out_temp < kMaxTemps && g.temp_cap[out_temp])
        std::memcpy(out_host, g.h_out, g.temp_last[out_temp]);
    return rc;
}

}  // namespace gehtp

using namespace gehtp;

extern "C" {

int wt_exec_run_range(const struct wt_blob* b, uint32_t first, uint32_t count, uint32_t* engine_m,
                      int64_t* op_us, char* err, size_t errn) {
    return run_impl(b, first, count, g.ext_in, nullptr, nullptr, nullptr, kNoOff, true, engine_m, op_us, err, errn);
}

int wt_exec_run(const struct wt_blob* b, uint32_t* engine_m, int64_t* op_us, char* err, size_t errn) {
    std::memset(&g.st, 0, sizeof g.st);
    if (!b) { set_err(err, errn, "null blob"); return -1; }
    return run_impl(b, 0, b->n_ops, g.ext_in, nullptr, nullptr, nullptr, kNoOff, true, engine_m, op_us, err, errn);
}

int wt_exec_run_io(const struct wt_blob* b, const void* in_ptr, void* out_ptr, uint32_t out_temp,
                   uint32_t* engine_m, int64_t* op_us, char* err, size_t errn) {
    std::memset(&g.st, 0, sizeof g.st);
    if (!b) { set_err(err, errn, "null blob"); return -1; }
    return run_impl(b, 0, b->n_ops, in_ptr, nullptr, out_ptr, nullptr, out_temp, true, engine_m, op_us, err, errn);
}

int gehtp_cuda_run_dev(const struct wt_blob* b, const void* in_dev, void* out_dev, uint32_t out_temp,
                       char* err, size_t errn) {
    std::memset(&g.st, 0, sizeof g.st);
    if (!b) { set_err(err, errn, "null blob"); return -1; }
    return run_impl(b, 0, b->n_ops, nullptr, in_dev, nullptr, out_dev, out_temp, false, nullptr, nullptr, err, errn);
}

uint8_t* wt_exec_temp(uint32_t id) {
    if (!g.dev_ok || id >= kMaxTemps || !g.temp_cap[id] || !g.temp_dev[id]) return nullptr;
    auto& m = g.mirrors[id];
    size_t need = g.temp_cap[id];
    if (m.second < need) {
        if (m.first) cudaFreeHost(m.first);
        m.first = nullptr;
        if (cudaMallocHost(&m.first, need) != cudaSuccess) { m.second = 0; return nullptr; }
        m.second = need;
    }
    cudaSetDevice(g.device);
    cudaStreamSynchronize(g.stream);
    if (cudaMemcpy(m.first, g.temp_dev[id], need, cudaMemcpyDeviceToHost) != cudaSuccess) return nullptr;
    return m.first;
}

uint32_t wt_exec_temp_bytes(uint32_t id) { return id < kMaxTemps ? g.temp_cap[id] : 0; }
uint32_t wt_exec_temp_last_bytes(uint32_t id) { return id < kMaxTemps ? g.temp_last[id] : 0; }

void wt_exec_shutdown(void) {
    std::memset(&g.st, 0, sizeof g.st);
    if (!g.dev_ok) return;
    cudaSetDevice(g.device);
    cudaStreamSynchronize(g.stream);
    drop_plan(true);
    g.force_unfused = false;
    g.user_pool = false;
    g.user_off.clear();
}

void wt_exec_state_reset(void) {
    if (!g.dev_ok) return;
    cudaSetDevice(g.device);
    for (uint32_t i = 0; i < g.n_states; i++) {
        cudaMemsetAsync(g.st_buf[i], 0, g.st_bytes[i], g.stream);
        g.st_count[i] = 0;
        if (g.kv[i].ready) cudaMemsetAsync(g.kv[i].posmap, 0xFF, (size_t)g.kv[i].nslots * 4, g.stream);
    }
    cudaMemsetAsync(g.d_st_count, 0, 2 * WT_MAX_STATES * sizeof(uint32_t), g.stream);
    cudaStreamSynchronize(g.stream);
}

void wt_exec_pool_init(uint8_t* base, uint32_t total_cap, uint32_t static_cap, const uint32_t* offsets) {
    if (base) {
        g.user_pool = true;
        g.user_total = total_cap;
        g.user_static = static_cap;
    } else if (!offsets) {
        g.user_pool = false;
    }
    g.user_off.clear();
    if (offsets) g.user_off.assign(offsets, offsets + kMaxTemps);
    if (g.planned) drop_plan(true);
}

void wt_exec_get_stats(struct wt_exec_stats* st) { if (st) *st = g.st; }
void wt_exec_set_ext_weights(const void* wgt_ptr) { g.ext_wgt = (const uint8_t*)wgt_ptr; }
void wt_exec_set_ts(struct wt_op_ts* buf, uint32_t cap) { g.ts_buf = buf; g.ts_cap = buf ? cap : 0; }
void wt_exec_set_trace(int on) { g.trace_on = on ? 1 : 0; }
void wt_exec_set_hook(const char* spec) { g.hook_spec = spec; }

// One JSON line per slot, then per op, then a summary line.
void wt_w3_report(const char* blob_name, const uint8_t* buf, size_t size, const struct wt_blob* w,
                  void (*emit)(const char* line, void* ud), void* ud) {
    if (!emit || !w) return;
    (void)buf;
    char line[512];
    std::snprintf(line, sizeof line, "{\"blob\":\"%s\",\"bytes\":%zu,\"ver\":%u,\"n_slots\":%u,\"n_ops\":%u,\"weight_off\":%u}",
                  blob_name ? blob_name : "", size, (unsigned)w->ver, w->n_slots, w->n_ops, w->weight_off);
    emit(line, ud);
    for (uint32_t i = 0; i < w->n_slots; i++) {
        const wt_slot& s = w->slots[i];
        std::snprintf(line, sizeof line, "{\"slot\":%u,\"len\":%u,\"count\":%u,\"offset\":%llu,\"addr\":%u}", i, s.len,
                      s.count, (unsigned long long)s.offset, s.addr);
        emit(line, ud);
    }
    for (uint32_t i = 0; i < w->n_ops; i++) {
        const wt_op& op = w->ops[i];
        int n = std::snprintf(line, sizeof line, "{\"op\":%u,\"opcode\":%u,\"args\":[", i, (unsigned)op.opcode);
        for (uint16_t a2 = 0; a2 < op.n_args && n < (int)sizeof line - 16; a2++)
            n += std::snprintf(line + n, sizeof line - n, a2 ? ",%u" : "%u", op.args[a2]);
        std::snprintf(line + n, sizeof line - n, "]}");
        emit(line, ud);
    }
}

// ---- CUDA-side configuration ----
int gehtp_cuda_set_device(int ordinal) {
    if (g.dev_ok && g.device != ordinal) return -1;
    g.device = ordinal;
    return ensure_device(nullptr, 0) ? 0 : -1;
}
void gehtp_cuda_set_fusion(int on) {
    if ((g.opt_fuse != (on ? 1 : 0) || g.force_unfused) && g.planned) drop_plan(true);
    g.opt_fuse = on ? 1 : 0;
    g.force_unfused = false;
}
void gehtp_cuda_set_graph(int on) {
    g.opt_graph = on ? 1 : 0;
    if (!on && g.graph) { cudaGraphExecDestroy(g.graph); g.graph = nullptr; }
}
uint64_t gehtp_cuda_launch_count(void) { return g_launches; }
uint32_t gehtp_cuda_fused_ops(void) { return g.fused_ops; }
uint32_t gehtp_cuda_const_ops(void) { return g.const_ops; }
uint32_t gehtp_cuda_demoted_temps(void) { return g.demoted_temps; }
void* gehtp_cuda_stream(void) { return ensure_device(nullptr, 0) ? (void*)g.stream : nullptr; }
void* gehtp_cuda_temp_dev(uint32_t id) { return (id < kMaxTemps && g.temp_cap[id]) ? g.temp_dev[id] : nullptr; }
int gehtp_cuda_sync(void) {
    if (!g.dev_ok) return -1;
    cudaSetDevice(g.device);
    return (int)cudaStreamSynchronize(g.stream);
}
const char* gehtp_cuda_last_error(void) { return g.last_error.c_str(); }
int gehtp_cuda_status_message(uint32_t code, char* msg, size_t msg_bytes) {
    char m[128];
    const int rc = status_message(code, m, sizeof m);
    if (msg && msg_bytes) std::snprintf(msg, msg_bytes, "%s", m);
    return rc;
}
// Eager run with a CUDA event pair around every launch unit; op_ms[i] gets the
// device time of the unit that starts at op i (0 for ops inside a fused unit).
int gehtp_cuda_run_profiled(const struct wt_blob* b, const void* in_ptr, uint32_t out_temp, float* op_ms,
                            uint32_t cap, char* err, size_t errn) {
    std::memset(&g.st, 0, sizeof g.st);
    if (!b || !op_ms) { set_err(err, errn, "null argument"); return -1; }
    for (uint32_t i = 0; i < cap; i++) op_ms[i] = 0.0f;
    g.prof_ms = op_ms;
    g.prof_events.clear();
    // The stream is held back by a host node until every launch of the pass is
    // queued (bounded: 200 ms), so the event pairs measure kernels running back
    // to back, not the host's launch pace.
    attn_prof_begin();
    static std::atomic<int> go;
    go.store(0);
    cudaLaunchHostFunc(g.stream, [](void* p) {
        auto* f = (std::atomic<int>*)p;
        for (int i = 0; i < 2000 && !f->load(); i++) std::this_thread::sleep_for(std::chrono::microseconds(100));
    }, &go);
    int rc = run_impl(b, 0, b->n_ops, in_ptr, nullptr, nullptr, nullptr, out_temp, false, nullptr, nullptr, err, errn);
    go.store(1);
    if (rc == 0) rc = finish_run(err, errn);
    else cudaStreamSynchronize(g.stream);
    g.prof_ms = nullptr;
    attn_prof_end(&g.prof_attn_ms, &g.prof_attn_n);
    for (auto& e : g.prof_events) {
        float ms = 0.0f;
        if (rc == 0 && e.op < cap && cudaEventElapsedTime(&ms, e.e0, e.e1) == cudaSuccess) op_ms[e.op] = ms;
        cudaEventDestroy(e.e0); cudaEventDestroy(e.e1);
    }
    g.prof_events.clear();
    return rc;
}

// Summed device time and launch count of the decode attention kernel alone in the last
// gehtp_cuda_run_profiled (its launch unit also holds the rotary/append and merge kernels).
void gehtp_cuda_profiled_attn(float* total_ms, uint32_t* launches) {
    if (total_ms) *total_ms = g.prof_attn_ms;
    if (launches) *launches = g.prof_attn_n;
}

// Loads `bytes` of a persistent state from host or device memory and, for a KV
// state, marks positions [0, n_positions) as resident (ring slot p holds
// position p) and sets the state's position counter to n_positions.
int gehtp_cuda_state_load(const struct wt_blob* b, uint32_t idx, const void* src, size_t bytes, int src_is_device,
                          uint32_t kv_elems, uint32_t n_positions, char* err, size_t errn) {
    if (!ensure_device(err, errn)) return -1;
    if (b && ensure_plan(b, err, errn) != 0) return -1;
    if (idx >= g.n_states || bytes > g.st_bytes[idx]) { set_err(err, errn, "state load: bad index or size"); return -1; }
    if (src && bytes)
        cudaMemcpyAsync(g.st_buf[idx], src, bytes, src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, g.stream);
    if (kv_elems) {
        KvGeom& k = g.kv[idx];
        if (!k.ready) {
            uint32_t slot_bytes = kv_elems * 4u;
            if (slot_bytes < 256u || (slot_bytes & 127u) || g.st_bytes[idx] % slot_bytes) { set_err(err, errn, "state load: kv geometry bad"); return -1; }
            k.slot_bytes = slot_bytes; k.nslots = g.st_bytes[idx] / slot_bytes;
            if (cudaMalloc(&k.posmap, (size_t)k.nslots * 4) != cudaSuccess) { set_err(err, errn, "kv posmap alloc"); return -1; }
            k.ready = true;
        }
        if (n_positions > k.nslots) { set_err(err, errn, "state load: more positions than ring slots"); return -1; }
        std::vector<uint32_t> pm(k.nslots, 0xFFFFFFFFu);
        for (uint32_t p = 0; p < n_positions; p++) pm[p] = p;
        cudaMemcpyAsync(k.posmap, pm.data(), (size_t)k.nslots * 4, cudaMemcpyHostToDevice, g.stream);
        cudaMemcpyAsync(g.d_st_count + idx, &n_positions, 4, cudaMemcpyHostToDevice, g.stream);
        g.st_count[idx] = n_positions;
        cudaStreamSynchronize(g.stream);
    }
    cudaError_t ce = cudaStreamSynchronize(g.stream);
    if (ce != cudaSuccess) { set_err(err, errn, cudaGetErrorString(ce)); return -1; }
    return 0;
}

// Sets the position counter of a KV state (positions at or past it stay in the
// ring but are no longer attended; the next append overwrites them).
int gehtp_cuda_state_set_count(uint32_t idx, uint32_t n_positions) {
    if (!g.dev_ok || idx >= g.n_states || !g.kv[idx].ready || n_positions > g.kv[idx].nslots) return -1;
    cudaSetDevice(g.device);
    cudaMemcpyAsync(g.d_st_count + idx, &n_positions, 4, cudaMemcpyHostToDevice, g.stream);
    cudaStreamSynchronize(g.stream);
    g.st_count[idx] = n_positions;
    return 0;
}

// Copies a persistent state to host memory (bytes <= its size).
int gehtp_cuda_state_read(uint32_t idx, void* dst, size_t bytes) {
    if (!g.dev_ok || idx >= g.n_states || bytes > g.st_bytes[idx]) return -1;
    cudaSetDevice(g.device);
    cudaStreamSynchronize(g.stream);
    return cudaMemcpy(dst, g.st_buf[idx], bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

// ---- state files in the layout of the reference's host golden ("HDS1") ----
// compiler/src/ops/host_decode_state.cpp:14-62 writes
//   "HDS1", u32 n = 42, u32 kv_count[6], f32 kv_k[6][64][512], f32 kv_v[6][64][512],
//   f32 conv_win[18][3 * 6144], f32 delta_s[18][16 * 128 * 128]
// (dimensions: compiler/include/hnnx/host_decode_state.hpp:17-27); the device state table
// numbers them kv 0..5, conv 6..23, delta 24..41 (compiler/tools/wtop_ops/wtop_ops.hpp:478-492).
// A KV state here is a ring of fp16 slots [K face | V face]; the file holds positions
// 0..count-1 as fp32 (every fp16 value is exact in fp32, and a file written by the host
// golden from fp16 inputs rounds back without loss).
namespace {
constexpr uint32_t kHdsKv = 6, kHdsConv = 18, kHdsDelta = 18, kHdsKvElems = 512, kHdsKvMax = 64;
constexpr uint32_t kHdsConvBytes = 3u * 6144u * 4u, kHdsDeltaBytes = 16u * 128u * 128u * 4u;
constexpr uint32_t kHdsSlotBytes = kHdsKvElems * 4u;   // fp16 K face + fp16 V face

int hds_check_table(char* err, size_t errn) {
    if (g.n_states != kHdsKv + kHdsConv + kHdsDelta) { set_err(err, errn, "state file: state table does not hold 42 states"); return -1; }
    for (uint32_t i = 0; i < g.n_states; i++) {
        bool ok = i < kHdsKv ? (g.st_bytes[i] >= kHdsSlotBytes && g.st_bytes[i] % kHdsSlotBytes == 0 &&
                                (!g.kv[i].ready || g.kv[i].slot_bytes == kHdsSlotBytes))
                : i < kHdsKv + kHdsConv ? g.st_bytes[i] == kHdsConvBytes
                                        : g.st_bytes[i] == kHdsDeltaBytes;
        if (!ok) {
            char m[96]; std::snprintf(m, sizeof m, "state file: state %u has %u bytes, not the file's shape", i, g.st_bytes[i]);
            set_err(err, errn, m); return -1;
        }
    }
    return 0;
}
}  // namespace

int gehtp_cuda_state_save_hds1(const struct wt_blob* b, const char* path, char* err, size_t errn) {
    if (!path) { set_err(err, errn, "null argument"); return -1; }
    if (!ensure_device(err, errn)) return -1;
    if (b && ensure_plan(b, err, errn) != 0) return -1;
    if (hds_check_table(err, errn) != 0) return -1;
    cudaStreamSynchronize(g.stream);
    uint32_t counts[WT_MAX_STATES];
    if (cudaMemcpy(counts, g.d_st_count, sizeof(uint32_t) * g.n_states, cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_err(err, errn, "state file: counter read failed"); return -1;
    }
    std::vector<float> kf((size_t)kHdsKv * kHdsKvMax * kHdsKvElems, 0.0f), vf(kf.size(), 0.0f);
    uint32_t kv_count[kHdsKv];
    for (uint32_t i = 0; i < kHdsKv; i++) {
        kv_count[i] = 0;
        if (!g.kv[i].ready) continue;
        const uint32_t nslots = g.kv[i].nslots;
        std::vector<uint32_t> pm(nslots);
        std::vector<uint16_t> ring((size_t)g.st_bytes[i] / 2);
        if (cudaMemcpy(pm.data(), g.kv[i].posmap, (size_t)nslots * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
            cudaMemcpy(ring.data(), g.st_buf[i], g.st_bytes[i], cudaMemcpyDeviceToHost) != cudaSuccess) {
            set_err(err, errn, "state file: KV read failed"); return -1;
        }
        // appends at explicit positions leave the AUTO counter at 0: the count is then the run of
        // resident positions from 0
        uint32_t n = counts[i];
        if (!n) while (n < nslots && pm[n] == n) n++;
        if (n > kHdsKvMax) { set_err(err, errn, "state file: a KV state holds more than 64 positions"); return -1; }
        kv_count[i] = n;
        for (uint32_t p = 0; p < n; p++) {
            const uint32_t s = p % nslots;
            if (pm[s] != p) { set_err(err, errn, "state file: a KV position below the counter is not resident"); return -1; }
            const uint16_t* slot = ring.data() + (size_t)s * kHdsKvElems * 2;
            float* kd = kf.data() + ((size_t)i * kHdsKvMax + p) * kHdsKvElems;
            float* vd = vf.data() + ((size_t)i * kHdsKvMax + p) * kHdsKvElems;
            for (uint32_t e = 0; e < kHdsKvElems; e++) {
                kd[e] = __half2float(__ushort_as_half(slot[e]));
                vd[e] = __half2float(__ushort_as_half(slot[kHdsKvElems + e]));
            }
        }
    }
    FILE* f = std::fopen(path, "wb");
    if (!f) { set_err(err, errn, "state file: cannot open for writing"); return -1; }
    const uint32_t n = g.n_states;
    bool ok = std::fwrite("HDS1", 1, 4, f) == 4 && std::fwrite(&n, 4, 1, f) == 1 &&
              std::fwrite(kv_count, 4, kHdsKv, f) == kHdsKv &&
              std::fwrite(kf.data(), 4, kf.size(), f) == kf.size() && std::fwrite(vf.data(), 4, vf.size(), f) == vf.size();
    std::vector<uint8_t> img(kHdsDeltaBytes);
    for (uint32_t i = kHdsKv; ok && i < n; i++) {
        ok = cudaMemcpy(img.data(), g.st_buf[i], g.st_bytes[i], cudaMemcpyDeviceToHost) == cudaSuccess &&
             std::fwrite(img.data(), 1, g.st_bytes[i], f) == g.st_bytes[i];
    }
    ok = (std::fclose(f) == 0) && ok;
    if (!ok) { set_err(err, errn, "state file: write failed"); return -1; }
    return 0;
}

// 0 = loaded, 1 = no such file (states untouched), -1 = bad file or a state table of another shape, as
// host_decode_state_load reports them. The file is read and checked as a whole before the first state is
// written, so a bad file leaves the states untouched; a device copy that fails midway (reported through err)
// leaves the states before it loaded.
int gehtp_cuda_state_load_hds1(const struct wt_blob* b, const char* path, char* err, size_t errn) {
    if (!path) { set_err(err, errn, "null argument"); return -1; }
    if (!ensure_device(err, errn)) return -1;
    if (b && ensure_plan(b, err, errn) != 0) return -1;
    if (hds_check_table(err, errn) != 0) return -1;
    FILE* f = std::fopen(path, "rb");
    if (!f) return 1;
    char magic[4];
    uint32_t n = 0, kv_count[kHdsKv];
    std::vector<float> kf((size_t)kHdsKv * kHdsKvMax * kHdsKvElems), vf(kf.size());
    std::vector<uint8_t> rest((size_t)kHdsConv * kHdsConvBytes + (size_t)kHdsDelta * kHdsDeltaBytes);
    bool ok = std::fread(magic, 1, 4, f) == 4 && !std::memcmp(magic, "HDS1", 4) && std::fread(&n, 4, 1, f) == 1 &&
              n == g.n_states && std::fread(kv_count, 4, kHdsKv, f) == kHdsKv &&
              std::fread(kf.data(), 4, kf.size(), f) == kf.size() && std::fread(vf.data(), 4, vf.size(), f) == vf.size() &&
              std::fread(rest.data(), 1, rest.size(), f) == rest.size();
    std::fclose(f);
    for (uint32_t i = 0; ok && i < kHdsKv; i++) ok = kv_count[i] <= kHdsKvMax && kv_count[i] <= g.st_bytes[i] / kHdsSlotBytes;
    if (!ok) { set_err(err, errn, "state file: bad magic, size or counts"); return -1; }
    for (uint32_t i = 0; i < kHdsKv; i++) {
        std::vector<uint16_t> ring((size_t)g.st_bytes[i] / 2, 0);
        for (uint32_t p = 0; p < kv_count[i]; p++) {
            uint16_t* slot = ring.data() + (size_t)p * kHdsKvElems * 2;
            const float* ks = kf.data() + ((size_t)i * kHdsKvMax + p) * kHdsKvElems;
            const float* vs = vf.data() + ((size_t)i * kHdsKvMax + p) * kHdsKvElems;
            for (uint32_t e = 0; e < kHdsKvElems; e++) {
                slot[e] = __half_as_ushort(__float2half_rn(ks[e]));
                slot[kHdsKvElems + e] = __half_as_ushort(__float2half_rn(vs[e]));
            }
        }
        if (gehtp_cuda_state_load(nullptr, i, ring.data(), g.st_bytes[i], 0, kHdsKvElems, kv_count[i], err, errn) != 0) return -1;
    }
    const uint8_t* src = rest.data();
    for (uint32_t i = kHdsKv; i < n; i++) {
        if (gehtp_cuda_state_load(nullptr, i, src, g.st_bytes[i], 0, 0, 0, err, errn) != 0) return -1;
        src += g.st_bytes[i];
    }
    return 0;
}

// Capture whatever the caller queues on the engine stream between begin and
// end into a CUDA graph, replay it `reps` times and report the mean device time
// of one replay (CUDA events on the engine stream). For timing short kernels
// without per-launch host overhead.
int gehtp_cuda_capture_begin(void) {
    if (!ensure_device(nullptr, 0)) return -1;
    return cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess ? 0 : -1;
}
int gehtp_cuda_capture_end_replay(int reps, float* ms_per_replay) {
    if (!g.dev_ok) return -1;
    cudaGraph_t graph = nullptr;
    if (cudaStreamEndCapture(g.stream, &graph) != cudaSuccess || !graph) { cudaGetLastError(); return -1; }
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { cudaGetLastError(); return -1; }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaGraphLaunch(exec, g.stream);                 // warm
    cudaEventRecord(e0, g.stream);
    for (int i = 0; i < reps; i++) cudaGraphLaunch(exec, g.stream);
    cudaEventRecord(e1, g.stream);
    e = cudaStreamSynchronize(g.stream);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    if (ms_per_replay) *ms_per_replay = reps > 0 ? ms / reps : 0.0f;
    return e == cudaSuccess ? 0 : -1;
}

size_t gehtp_w4a16_slot_bytes(uint32_t K, uint32_t N) { return (size_t)K * N / 2 + (size_t)2 * (K / GEHTP_W4_GROUP) * N; }

}  // extern "C"
