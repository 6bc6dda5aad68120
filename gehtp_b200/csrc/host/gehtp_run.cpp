// gehtp_run: host runners for WTOP blobs on the CUDA executor, speaking the file
// protocols of the reference's two device-side runners so that its drivers
// (`gehtp run`, persistent_runtime.py) can point at a CUDA box unchanged.
//
//   gehtp_run job   <job.txt>   one run, or a decode loop (kernels/examples/42_gehtp_runner/main.c)
//   gehtp_run serve <job.txt>   request/response file queue (kernels/examples/42_gehtp_persistent/main.c)
//
// job.txt holds "key value" lines.
//   job  : blob, input, output, out_temp; optional trace (0/1), hook (dump spec), steps (n > 1: inputs
//          are <input>.<i>, outputs <output>.<i>), weights_size, op_ts (path of the per-op timestamp file,
//          default <output>.op_ts.bin), state_file (an "HDS1" decode-state file: loaded before the
//          first run when it exists, written after the last one, the way the reference's host golden
//          uses GEHTP_HOST_STATE, compiler/src/ir/graph_prepare.cpp:720,1155). External weights are
//          looked for beside the blob: <blob minus ".wtop">.weights.bin.
//   serve: blob, req, resp, out, out_temp, in_bytes; optional idle_exit_s, weights_size, trace.
//          A request file is a 4-byte big-endian header length, a JSON header
//          {"op": "run|reset|ping|shutdown", "want_out": 0|1, ...} and, for run, the input body; it is
//          unlinked when claimed. The response file is 4-byte big-endian length + JSON
//          {"rc":0,"token":n,"steps":u,"step_us":u} (token = arg-max of the fp16 output temp).
// op_ts file: 'WTS1' u32 | version 2 u32 | n_ops u32 | pad u32 | wall_us u64 | n_ops x wt_op_ts.
// Exit status 0 = PASS.
#include <chrono>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>
#include <sys/stat.h>
#include <unistd.h>
#include "gehtp_cuda.h"
#include "wtop_format.h"

namespace {

void logf(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vfprintf(stdout, fmt, ap);
    va_end(ap);
    std::fputc('\n', stdout);
    std::fflush(stdout);
}

int64_t now_us() {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

bool read_file(const std::string& path, std::vector<uint8_t>& out, size_t expect = 0) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    std::fseek(f, 0, SEEK_END);
    long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (sz <= 0 || (expect && (size_t)sz != expect)) { std::fclose(f); return false; }
    out.resize((size_t)sz);
    size_t got = std::fread(out.data(), 1, out.size(), f);
    std::fclose(f);
    return got == out.size();
}

bool write_file(const std::string& path, const void* data, size_t n) {
    std::string tmp = path + ".part";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return false;
    bool ok = std::fwrite(data, 1, n, f) == n;
    ok = std::fclose(f) == 0 && ok;
    return ok && std::rename(tmp.c_str(), path.c_str()) == 0;   // readers never see a half-written file
}

struct Job {
    std::vector<std::pair<std::string, std::string>> kv;
    bool load(const std::string& path) {
        std::vector<uint8_t> raw;
        if (!read_file(path, raw)) return false;
        std::string text(raw.begin(), raw.end()), line;
        size_t p = 0;
        while (p <= text.size()) {
            size_t e = text.find('\n', p);
            line = text.substr(p, e == std::string::npos ? std::string::npos : e - p);
            if (!line.empty() && line.back() == '\r') line.pop_back();
            size_t sp = line.find(' ');
            if (sp != std::string::npos && sp > 0) kv.emplace_back(line.substr(0, sp), line.substr(sp + 1));
            if (e == std::string::npos) break;
            p = e + 1;
        }
        return true;
    }
    const char* get(const char* key) const {
        for (auto& e : kv) if (e.first == key) return e.second.c_str();
        return nullptr;
    }
    long num(const char* key, long dflt) const { const char* v = get(key); return v ? std::strtol(v, nullptr, 10) : dflt; }
};

struct Loaded {
    std::vector<uint8_t> blob_bytes, ext_weights;
    wt_blob* blob = nullptr;
    ~Loaded() { std::free(blob); }
};

// blob + optional external weights; false = failure already logged
bool load_blob(const Job& job, Loaded& L) {
    const char* bp = job.get("blob");
    if (!bp || !read_file(bp, L.blob_bytes)) { logf("[FAIL] read blob %s", bp ? bp : "(no blob key)"); return false; }
    L.blob = (wt_blob*)std::calloc(1, sizeof(wt_blob));          // a few MB: never on the stack
    if (!L.blob) { logf("[FAIL] wt_blob alloc"); return false; }
    int prc = wt_parse(L.blob_bytes.data(), L.blob_bytes.size(), L.blob);
    if (prc != WT_OK) { logf("[FAIL] wt_parse: %s", wt_err_str(prc)); return false; }
    std::string wp(bp);
    if (wp.size() > 5 && wp.compare(wp.size() - 5, 5, ".wtop") == 0) wp.resize(wp.size() - 5);
    wp += ".weights.bin";
    struct stat st;
    if (stat(wp.c_str(), &st) == 0) {
        size_t want = (size_t)job.num("weights_size", 0);
        if (read_file(wp, L.ext_weights, want)) {
            wt_exec_set_ext_weights(L.ext_weights.data());
            logf("[ext-weights] %s loaded (%zu bytes)", wp.c_str(), L.ext_weights.size());
        } else {
            logf("[ext-weights] %s unreadable or not %zu bytes (inline weights only)", wp.c_str(), want);
        }
    }
    wt_exec_set_trace(job.num("trace", 0) ? 1 : 0);
    return true;
}

bool dump_temp(const std::string& path, uint32_t temp) {
    uint32_t n = wt_exec_temp_last_bytes(temp);
    const uint8_t* p = wt_exec_temp(temp);
    return n && p && write_file(path, p, n);
}

int run_step(const wt_blob* b, const std::string& in_path, const std::string& out_path, uint32_t out_temp) {
    std::vector<uint8_t> in;
    char err[160] = {0};
    if (!read_file(in_path, in)) { logf("[FAIL] read step input %s", in_path.c_str()); return -1; }
    int rc = wt_exec_run_io(b, in.data(), nullptr, out_temp, nullptr, nullptr, err, sizeof err);
    if (rc) { logf("[FAIL] step run rc=%d %s", rc, err); return rc; }
    if (!dump_temp(out_path, out_temp)) { logf("[FAIL] out temp %u empty or %s unwritable", out_temp, out_path.c_str()); return -1; }
    return 0;
}

// "first load, last save" of the decode states through an HDS1 file
bool state_file_load(const wt_blob* b, const char* path) {
    if (!path) return true;
    char err[160] = {0};
    int rc = gehtp_cuda_state_load_hds1(b, path, err, sizeof err);
    if (rc < 0) { logf("[FAIL] state file %s: %s", path, err); return false; }
    logf(rc == 0 ? "[state] loaded %s" : "[state] %s absent, states start at zero", path);
    return true;
}
bool state_file_save(const wt_blob* b, const char* path) {
    if (!path) return true;
    char err[160] = {0};
    if (gehtp_cuda_state_save_hds1(b, path, err, sizeof err) != 0) { logf("[FAIL] state file %s: %s", path, err); return false; }
    logf("[state] saved %s", path);
    return true;
}

int mode_job(const std::string& job_path) {
    Job job;
    if (!job.load(job_path)) { logf("[FAIL] read %s", job_path.c_str()); return 1; }
    const char *in_p = job.get("input"), *out_p = job.get("output"), *temp_s = job.get("out_temp");
    if (!job.get("blob") || !in_p || !out_p || !temp_s) { logf("[FAIL] job file lacks one of blob/input/output/out_temp"); return 1; }
    const uint32_t out_temp = (uint32_t)std::strtoul(temp_s, nullptr, 10);
    const int64_t t_read0 = now_us();
    Loaded L;
    if (!load_blob(job, L)) return 1;
    if (const char* hook = job.get("hook")) { wt_exec_set_hook(hook); logf("[hook] tensor dump spec: %s", hook); }
    const char* state_p = job.get("state_file");
    if (!state_file_load(L.blob, state_p)) { wt_exec_shutdown(); return 1; }
    const int64_t t_read1 = now_us();
    const long steps = job.num("steps", 1);
    if (steps > 1) {
        logf("[decode-loop] %ld steps (out_temp %u)", steps, out_temp);
        const int64_t t0 = now_us();
        int bad = 0;
        for (long i = 0; i < steps && !bad; i++) {
            const int64_t ts = now_us();
            int r = run_step(L.blob, std::string(in_p) + "." + std::to_string(i), std::string(out_p) + "." + std::to_string(i), out_temp);
            logf("[decode-loop] step %ld rc=%d us=%lld", i, r, (long long)(now_us() - ts));
            bad = r != 0;
        }
        logf("[decode-loop] total us=%lld%s", (long long)(now_us() - t0), bad ? " (FAIL)" : "");
        if (!bad && !state_file_save(L.blob, state_p)) bad = 1;
        wt_exec_shutdown();
        logf(bad ? "[FAIL] gehtp_run overall" : "[PASS] gehtp_run overall");
        return bad;
    }
    std::vector<uint8_t> in;
    if (!read_file(in_p, in)) { logf("[FAIL] read input %s", in_p); return 1; }
    const uint32_t n_ops = L.blob->n_ops;
    std::vector<int64_t> op_us(n_ops, 0);
    std::vector<wt_op_ts> op_ts(n_ops);
    if (n_ops) wt_exec_set_ts(op_ts.data(), n_ops);
    char err[160] = {0};
    const int64_t t0 = now_us();
    int rc = wt_exec_run_io(L.blob, in.data(), nullptr, out_temp, nullptr, n_ops ? op_us.data() : nullptr, err, sizeof err);
    const int64_t wall = now_us() - t0;
    if (rc) { logf("[FAIL] wt_exec_run_io rc=%d %s", rc, err); wt_exec_shutdown(); return 1; }
    // per-opcode totals, in the runner's log format
    constexpr int kMaxCode = 64;
    int64_t tot[kMaxCode] = {0}, mx[kMaxCode] = {0}, sum = 0, top = 0;
    uint32_t cnt[kMaxCode] = {0};
    int top_i = -1;
    for (uint32_t i = 0; i < n_ops; i++) {
        uint32_t c = L.blob->ops[i].opcode;
        if (c < kMaxCode) { tot[c] += op_us[i]; cnt[c]++; if (op_us[i] > mx[c]) mx[c] = op_us[i]; }
        sum += op_us[i];
        if (op_us[i] > top) { top = op_us[i]; top_i = (int)i; }
    }
    logf("[timing] ops=%u sum_op_us=%lld wall_us=%lld ops_per_sec=%.1f", n_ops, (long long)sum, (long long)wall,
         wall > 0 ? (double)n_ops * 1e6 / (double)wall : 0.0);
    for (int c = 0; c < kMaxCode; c++)
        if (cnt[c]) logf("op_timing code=%d n=%u total_us=%lld avg_us=%.1f max_us=%lld", c, cnt[c], (long long)tot[c],
                         (double)tot[c] / cnt[c], (long long)mx[c]);
    if (top_i >= 0) logf("[timing] slowest op#%d code=%u us=%lld", top_i, L.blob->ops[top_i].opcode, (long long)top);
    {
        std::string tsp = job.get("op_ts") ? job.get("op_ts") : std::string(out_p) + ".op_ts.bin";
        std::vector<uint8_t> file(24 + (size_t)n_ops * sizeof(wt_op_ts), 0);
        const uint32_t ver = 2;
        const uint64_t wall_u = (uint64_t)wall;
        std::memcpy(file.data(), "WTS1", 4);
        std::memcpy(file.data() + 4, &ver, 4);
        std::memcpy(file.data() + 8, &n_ops, 4);
        std::memcpy(file.data() + 16, &wall_u, 8);
        if (n_ops) std::memcpy(file.data() + 24, op_ts.data(), (size_t)n_ops * sizeof(wt_op_ts));
        logf(write_file(tsp, file.data(), file.size()) ? "[prof] op_ts file %u ops" : "[prof] op_ts file write FAIL", n_ops);
    }
    const int64_t t_w0 = now_us();
    bool ok = dump_temp(out_p, out_temp);
    logf("[run] seg_us read=%lld exec=%lld write=%lld", (long long)(t_read1 - t_read0), (long long)wall, (long long)(now_us() - t_w0));
    if (!ok) logf("[FAIL] out temp %u empty or %s unwritable", out_temp, out_p);
    else logf("[out] %u bytes -> %s", wt_exec_temp_last_bytes(out_temp), out_p);
    if (ok && !state_file_save(L.blob, state_p)) ok = false;
    wt_exec_shutdown();
    logf(ok ? "[PASS] gehtp_run overall" : "[FAIL] gehtp_run overall");
    return ok ? 0 : 1;
}

// ---- serve mode helpers
bool json_str(const std::string& h, const char* key, std::string& out) {
    std::string k = std::string("\"") + key + "\"";
    size_t p = h.find(k);
    if (p == std::string::npos) return false;
    p = h.find(':', p + k.size());
    if (p == std::string::npos) return false;
    p = h.find('"', p);
    if (p == std::string::npos) return false;
    size_t e = h.find('"', p + 1);
    if (e == std::string::npos) return false;
    out = h.substr(p + 1, e - p - 1);
    return true;
}
long json_int(const std::string& h, const char* key, long dflt) {
    std::string k = std::string("\"") + key + "\"";
    size_t p = h.find(k);
    if (p == std::string::npos) return dflt;
    p = h.find(':', p + k.size());
    return p == std::string::npos ? dflt : std::strtol(h.c_str() + p + 1, nullptr, 10);
}
bool write_resp(const std::string& path, const std::string& json) {
    std::vector<uint8_t> f(4 + json.size());
    uint32_t n = (uint32_t)json.size();
    f[0] = (uint8_t)(n >> 24); f[1] = (uint8_t)(n >> 16); f[2] = (uint8_t)(n >> 8); f[3] = (uint8_t)n;
    std::memcpy(f.data() + 4, json.data(), json.size());
    return write_file(path, f.data(), f.size());
}
float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, bits;
    if (e == 0) {
        if (!m) bits = sign;
        else { int sh = 0; while (!(m & 1024u)) { m <<= 1; sh++; } bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13); }
    } else if (e == 31u) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
int argmax_f16(const uint8_t* p, uint32_t bytes) {
    int best = -1;
    float bv = 0.0f;
    for (uint32_t i = 0; i + 1 < bytes; i += 2) {
        uint16_t h;
        std::memcpy(&h, p + i, 2);
        float v = half_to_float(h);
        if (v != v) continue;
        if (best < 0 || v > bv) { best = (int)(i / 2); bv = v; }
    }
    return best;
}
std::string json_escape(const char* s) {
    std::string o;
    for (; *s; s++) {
        if (*s == '"' || *s == '\\') { o += '\\'; o += *s; }
        else if ((unsigned char)*s < 0x20) o += ' ';
        else o += *s;
    }
    return o;
}

int mode_serve(const std::string& job_path) {
    Job job;
    if (!job.load(job_path)) { logf("[FAIL] read %s", job_path.c_str()); return 1; }
    const char *req_p = job.get("req"), *resp_p = job.get("resp"), *out_p = job.get("out"), *temp_s = job.get("out_temp");
    if (!job.get("blob") || !req_p || !resp_p || !out_p || !temp_s || !job.get("in_bytes")) {
        logf("[FAIL] job file lacks one of blob/req/resp/out/out_temp/in_bytes");
        return 1;
    }
    const uint32_t out_temp = (uint32_t)std::strtoul(temp_s, nullptr, 10);
    const size_t in_bytes = (size_t)job.num("in_bytes", 0);
    const long idle_exit_s = job.num("idle_exit_s", 0);
    Loaded L;
    if (!load_blob(job, L)) return 1;
    logf("[serve] blob %s out_temp %u in_bytes %zu idle_exit_s %ld", job.get("blob"), out_temp, in_bytes, idle_exit_s);
    uint32_t steps = 0;
    int64_t last = now_us();
    std::vector<uint8_t> req, body(in_bytes ? in_bytes : 1);
    for (;;) {
        struct stat st;
        if (stat(req_p, &st) != 0 || st.st_size < 4) {
            if (idle_exit_s > 0 && now_us() - last > (int64_t)idle_exit_s * 1000000) { logf("[idle] %lds without a request, exit", idle_exit_s); break; }
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
            continue;
        }
        // a request that is still being written has a header length its size does not cover yet
        bool whole = false;
        for (int tries = 0; tries < 2500 && !whole; tries++) {
            if (read_file(req_p, req) && req.size() >= 4) {
                size_t hl = ((size_t)req[0] << 24) | ((size_t)req[1] << 16) | ((size_t)req[2] << 8) | req[3];
                std::string hdr = req.size() >= 4 + hl ? std::string((const char*)req.data() + 4, hl) : std::string();
                std::string op;
                if (!hdr.empty() && json_str(hdr, "op", op) && (op != "run" || req.size() >= 4 + hl + in_bytes)) whole = true;
            }
            if (!whole) std::this_thread::sleep_for(std::chrono::milliseconds(2));
        }
        unlink(req_p);
        last = now_us();
        if (!whole) { write_resp(resp_p, "{\"rc\":-1,\"err\":\"short_request\"}"); continue; }
        const size_t hl = ((size_t)req[0] << 24) | ((size_t)req[1] << 16) | ((size_t)req[2] << 8) | req[3];
        const std::string hdr((const char*)req.data() + 4, hl);
        std::string op;
        json_str(hdr, "op", op);
        if (op == "ping") write_resp(resp_p, "{\"rc\":0,\"pong\":1}");
        else if (op == "reset") { wt_exec_state_reset(); steps = 0; logf("[reset] state cleared"); write_resp(resp_p, "{\"rc\":0,\"reset\":1}"); }
        else if (op == "shutdown") { write_resp(resp_p, "{\"rc\":0,\"bye\":1}"); break; }
        else if (op == "run") {
            if (req.size() - 4 - hl > body.size()) { write_resp(resp_p, "{\"rc\":-1,\"err\":\"body_too_big\"}"); continue; }
            std::memcpy(body.data(), req.data() + 4 + hl, req.size() - 4 - hl);
            char err[160] = {0};
            const int64_t t0 = now_us();
            int rc = wt_exec_run_io(L.blob, body.data(), nullptr, out_temp, nullptr, nullptr, err, sizeof err);
            const int64_t us = now_us() - t0;
            char resp[320];
            if (rc) {
                std::snprintf(resp, sizeof resp, "{\"rc\":%d,\"err\":\"%s\"}", rc, json_escape(err).c_str());
                logf("[run] FAIL rc=%d err=%s", rc, err);
            } else {
                int tok = argmax_f16(wt_exec_temp(out_temp), wt_exec_temp_last_bytes(out_temp));
                if (json_int(hdr, "want_out", 0) && !dump_temp(out_p, out_temp)) logf("[warn] out file not written");
                steps++;
                std::snprintf(resp, sizeof resp, "{\"rc\":0,\"token\":%d,\"steps\":%u,\"step_us\":%lld}", tok, steps, (long long)us);
            }
            write_resp(resp_p, resp);
        } else write_resp(resp_p, "{\"rc\":-1,\"err\":\"bad_op\"}");
    }
    wt_exec_shutdown();
    logf("[PASS] gehtp_run serve done (%u steps)", steps);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 3 || (std::strcmp(argv[1], "job") && std::strcmp(argv[1], "serve"))) {
        std::fprintf(stderr, "usage: gehtp_run job|serve <job.txt>\n");
        return 2;
    }
    return std::strcmp(argv[1], "job") == 0 ? mode_job(argv[2]) : mode_serve(argv[2]);
}
