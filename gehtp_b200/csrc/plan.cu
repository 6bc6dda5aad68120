// Turns a parsed runlist into a launch plan: every op is validated and its
// operands resolved to device addresses once, when the blob is first run.
//
// Memory plan. One device arena holds, in this order: the static temp pool of
// the blob's TEMPOFF table (its offsets are used as they are), the region for
// temps the table marks as on-chip resident, and one region per remaining temp
// sized to the largest tensor that temp id ever holds. Every size is known from
// the op arguments, so the plan is built by walking the op list twice: a
// measuring walk (sizes, first-write / last-read of each temp) and a building
// walk (addresses baked into the launch closures). Table entries whose live
// ranges overlap in time while their byte ranges overlap in the pool are moved
// out of the static pool, because the emitter binds an offset to a temp *id*
// that it later recycles for other tensors.
//
// Validation and error strings follow the per-op routines of the reference
// executor (kernels/src/runtime/oplist_exec.c, cited at each case).
#include <cstdio>
#include <cstring>
#include "engine.h"

namespace gehtp {

namespace {

struct LiveRange { uint32_t w, r; };  // written at op w, last read at op r

struct Planner {
    const wt_blob* b;
    bool build;
    uint32_t opi = 0;
    bool written[kMaxTemps];
    // 64-bit: a temp that only exists inside a fused chain may exceed the 4 GB a
    // materialised temp is limited to (e.g. the GQA-expanded K/V faces at batch 64)
    uint64_t cap[kMaxTemps], last[kMaxTemps];
    // measuring walk results
    uint64_t maxb[kMaxTemps];
    bool oversize[kMaxTemps];
    std::vector<LiveRange> live[kMaxTemps];
    // building walk inputs
    uint8_t* addr[kMaxTemps];
    bool in_static[kMaxTemps], in_vtcm[kMaxTemps];
    bool internal[kMaxTemps];   // exists only inside fused chains: no memory
    PlanOp* cur = nullptr;

    uint8_t* dummy() const { return (uint8_t*)(uintptr_t)256; }

    const uint8_t* slot_ptr(uint32_t s) const {
        if (s >= b->n_slots) return nullptr;
        const wt_slot& sl = b->slots[s];
        if (sl.addr == WT_SLOT_EXT_IN || sl.addr == WT_SLOT_EXT_WGT) {
            if (sl.addr == WT_SLOT_EXT_WGT && !g.ext_wgt) return nullptr;
            if (!build) return dummy();
            auto it = g.d_ext.find(s);
            return it == g.d_ext.end() ? nullptr : it->second;
        }
        return build ? g.d_weights + sl.offset : dummy();
    }

    // ref_ptr, oplist_exec.c:189-203
    const uint8_t* ref(uint32_t arg) {
        if (arg & 0x8000u) return slot_ptr(arg & 0x7FFFu);
        if ((arg & 0xE000u) == WT_REF_STATE_FLAG) {
            uint32_t s = arg & 0x1FFFu;
            return s < g.n_states ? g.st_buf[s] : nullptr;
        }
        uint32_t t;
        if (arg & 0x4000u) {
            t = arg & 0x3FFFu;
            if (t >= kMaxTemps || g.vtcm_off[t] == kNoOff) return nullptr;
            if (!build) { touch(t); return dummy(); }
            return g.d_arena + g.vtcm_base + g.vtcm_off[t];
        }
        t = arg;
        if (t >= kMaxTemps || !written[t]) return nullptr;
        touch(t);
        if (build && internal[t]) { if (cur) cur->uses_internal = true; return dummy(); }
        return build ? addr[t] : dummy();
    }
    void touch(uint32_t t) {
        if (!build && !live[t].empty()) live[t].back().r = opi;
    }
    // ref_elem_count, oplist_exec.c:209-213
    uint32_t ref_count(uint32_t arg) const {
        if (arg & 0x8000u) { uint32_t s = arg & 0x7FFFu; return s < b->n_slots ? b->slots[s].count : 0; }
        if (arg & 0x4000u) return 0;
        return arg < kMaxTemps ? (uint32_t)(last[arg] / 2u) : 0;
    }
    // temp_get, oplist_exec.c:257-335
    uint8_t* temp_get(uint32_t id, uint64_t bytes64, PlanOp& p) {
        if (id >= kMaxTemps || bytes64 > (1ull << 40)) return nullptr;
        // Above 4 GB (the reference's temp sizes are 32-bit) only as a temp that fusion removes.
        if (bytes64 > 0xFFFFFFFFull) {
            if (!build) oversize[id] = true;
            else if (!internal[id]) return nullptr;
        }
        const uint64_t bytes = bytes64;
        bool vt = g.vtcm_off[id] != kNoOff, stc = !vt && g.have_static && g.static_off[id] != kNoOff;
        if (vt && (uint64_t)g.vtcm_off[id] + bytes > g.vtcm_cap) return nullptr;
        if (stc && (!build || in_static[id]) && (uint64_t)g.static_off[id] + bytes > g.static_cap) return nullptr;
        if (vt || stc) cap[id] = bytes;
        else if (!written[id] || cap[id] < bytes) cap[id] = bytes;
        last[id] = bytes;
        written[id] = true;
        for (int k = 0; k < 2; k++)
            if (p.out_id[k] == kNoOff || p.out_id[k] == id) { p.out_id[k] = id; p.out_bytes[k] = (uint32_t)(bytes > 0xFFFFFFFFull ? 0xFFFFFFFFull : bytes); break; }
        if (!build) {
            if (bytes > maxb[id]) maxb[id] = bytes;
            live[id].push_back({opi, opi});
            return dummy();
        }
        if (internal[id]) { p.uses_internal = true; return dummy(); }
        return addr[id];
    }
};

#define FAIL(...)                                            \
    do {                                                     \
        char _m[160];                                        \
        std::snprintf(_m, sizeof _m, __VA_ARGS__);           \
        p.rc = -1; p.err = _m; return;                       \
    } while (0)

// KV ring geometry of a state, derived from the op's K/V width on first use
// (state_kvc, oplist_exec.c:2119-2151).
KvGeom* kv_geom(uint32_t state_ref, uint32_t kv_elems, PlanOp& p) {
    auto fail = [&](const char* fmt, uint32_t a, uint32_t b2, uint32_t c) -> KvGeom* {
        char m[160]; std::snprintf(m, sizeof m, fmt, a, b2, c); p.rc = -1; p.err = m; return nullptr;
    };
    if ((state_ref & 0xE000u) != WT_REF_STATE_FLAG) return fail("kv state_ref not 0x6000|idx (0x%X)", state_ref, 0, 0);
    uint32_t i = state_ref & 0x1FFFu;
    if (i >= g.n_states) return fail("kv state idx %u oob", i, 0, 0);
    uint32_t slot_bytes = kv_elems * 4u;
    KvGeom& k = g.kv[i];
    if (!k.ready) {
        if (slot_bytes < 256u || (slot_bytes & 127u) || g.st_bytes[i] % slot_bytes != 0u)
            return fail("kv state %u geometry bad (slot=%u total=%u)", i, slot_bytes, g.st_bytes[i]);
        k.slot_bytes = slot_bytes;
        k.nslots = g.st_bytes[i] / slot_bytes;
        if (cudaMalloc(&k.posmap, (size_t)k.nslots * 4) != cudaSuccess) return fail("kv posmap alloc", 0, 0, 0);
        cudaMemsetAsync(k.posmap, 0xFF, (size_t)k.nslots * 4, g.stream);
        k.ready = true;
    } else if (k.slot_bytes != slot_bytes) {
        return fail("kv state %u slot_bytes mismatch (%u vs %u)", i, k.slot_bytes, slot_bytes);
    }
    return &k;
}

W4Packed* w4_prepare(Planner& P, uint32_t w_ref, uint32_t K, uint32_t N, PlanOp& p) {
    uint32_t s = w_ref & 0x7FFFu;
    uint64_t key = (uint64_t)s | ((uint64_t)K << 16) | ((uint64_t)N << 40);
    auto it = g.w4.find(key);
    if (it != g.w4.end()) return &it->second;
    if (!P.build) return nullptr;
    W4Packed w;
    w.K = K; w.N = N;
    const uint8_t* slot = P.slot_ptr(s);
    size_t nb = (size_t)K * N / 2;
    if (cudaMalloc(&w.packed, nb) != cudaSuccess) { p.rc = -1; p.err = "w4 packed alloc"; return nullptr; }
    k_w4_repack(g.stream, slot, w.packed, K, N);
    w.scales = (const uint16_t*)(slot + nb);
    return &(g.w4[key] = w);
}

void plan_op(Planner& P, const wt_op& op, PlanOp& p) {
    const wt_blob* b = P.b;
    const uint32_t* a = op.args;
    switch (op.opcode) {
    case OP_NOP: p.stat = 2; return;
    case OP_PIN: {  // xop_pin, oplist_exec.c:2310-2325: no on-chip cache to fill on a GPU
        if (a[0] >= b->n_slots) FAIL("pin slot oob");
        p.stat = 6;
        return;
    }
    case OP_MATMUL_W4A16: {  // group-64 form, see gehtp_cuda.h; legacy: oplist_exec.c:438-529
        p.stat = 3;
        uint32_t M = a[3], K = a[4], N = a[5];
        if (!(a[1] & 0x8000u) || (a[1] & 0x7FFFu) >= b->n_slots) FAIL("w4a16 weight ref is not a slot");
        const wt_slot& ws = b->slots[a[1] & 0x7FFFu];
        if ((uint64_t)ws.len == (uint64_t)K * N / 2u) FAIL("legacy W4A16 slot form unsupported on CUDA");
        if (!M || !K || !N || (K % 64u) || (N % 16u)) FAIL("w4a16 shape m%u k%u n%u", M, K, N);
        if ((uint64_t)ws.len != gehtp_w4a16_slot_bytes(K, N)) FAIL("w slot size mismatch");
        const uint16_t* act = (const uint16_t*)P.ref(a[0]);
        if (!act) FAIL("w4a16 act ref fail");
        if ((a[0] & 0x8000u) && b->slots[a[0] & 0x7FFFu].len != M * K * 2u) FAIL("act slot size mismatch");
        if (!P.slot_ptr(a[1] & 0x7FFFu)) FAIL("w4a16 weight slot has no data");
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)M * N * 2u, p);
        if (!y) FAIL("temp %u alloc", a[2]);
        p.w4_m = M;
        p.engine = WT_ENG_HMX;
        W4Packed* w = w4_prepare(P, a[1], K, N, p);
        if (p.rc) return;
        if (P.build) {
            const uint32_t* pk = w->packed; const uint16_t* sc = w->scales;
            p.launch = [=](cudaStream_t st) {
                W4Epilogue ep;
                ep.status = g.d_status;
                if (M >= w4_gemm_min_rows() && k_w4a16_gemm_sm100(st, act, pk, sc, y, M, K, N, ep)) return;
                k_w4a16_skinny(st, act, pk, sc, y, M, K, N, ep);
            };
            if (M >= w4_gemm_min_rows())
                p.launch_w4_gemm = [=](cudaStream_t st, const W4Epilogue& ep, const uint16_t* a_src, uint32_t a_d) {
                    return k_w4a16_gemm_sm100(st, a_d ? a_src : act, pk, sc, y, M, K, N, ep, 0, a_d);
                };
        }
        return;
    }
    case OP_RMSNORM_F16:
        p.stat = 4;
        FAIL("legacy crouton rmsnorm (opcode 2) unsupported on CUDA");
    case OP_SILU_F16: {  // exec_silu, :594-610
        p.stat = 5;
        uint32_t x_t = a[0], n = a[2];
        if (x_t >= kMaxTemps || !P.written[x_t]) FAIL("silu src temp %u empty", x_t);
        if (P.cap[x_t] != n * 2u) FAIL("silu n_elem mismatch (%u vs face %u)", n, P.cap[x_t] / 2u);
        const uint16_t* x = (const uint16_t*)P.ref(x_t);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)n * 2u, p);
        if (!y) FAIL("silu temp %u alloc", a[1]);
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_unary(st, x, y, n, 12); };
        return;
    }
    case OP_IM2COL: {  // exec_im2col, :615-645
        p.stat = 8;
        const uint16_t* act = (const uint16_t*)P.ref(a[0]);
        if (!act) FAIL("im2col act ref empty");
        uint64_t K = (uint64_t)a[5] * a[6] * a[4];
        uint16_t* cols = (uint16_t*)P.temp_get(a[1], (uint64_t)a[13] * a[14] * K * 2u, p);
        if (!cols) FAIL("im2col temp alloc");
        p.engine = WT_ENG_HVX;
        if (P.build) {
            std::vector<uint32_t> args(a, a + 15);
            p.launch = [=](cudaStream_t st) { k_im2col(st, act, cols, args.data()); };
        }
        return;
    }
    case OP_CONV2D_F16: {  // exec_conv2d, :761-800
        p.stat = 9;
        uint32_t M = a[4], K = a[5], N = a[6];
        const uint16_t* cols = (const uint16_t*)P.ref(a[0]);
        const uint16_t* wp = (const uint16_t*)P.slot_ptr(a[1]);
        const uint16_t* bp = (const uint16_t*)P.slot_ptr(a[2]);
        if (!cols || !wp || !bp) FAIL("conv2d ref empty");
        if (b->slots[a[1]].len != K * N * 2u || b->slots[a[2]].len != N * 2u) FAIL("conv2d w/b slot size mismatch");
        uint16_t* out = (uint16_t*)P.temp_get(a[3], (uint64_t)a[9] * a[10] * N * 2u, p);
        if (!out) FAIL("conv2d temp alloc");
        p.engine = WT_ENG_HVX;
        uint32_t oy0 = a[7], ox0 = a[8], oW = a[10], co0 = a[11], con = a[12];
        if (P.build) p.launch = [=](cudaStream_t st) { k_conv2d(st, cols, wp, bp, out, M, K, N, oy0, ox0, oW, co0, con); };
        return;
    }
    case OP_ADD_F16: {  // exec_add, :807-829
        p.stat = 10;
        uint32_t n = a[3];
        const uint16_t* x0 = (const uint16_t*)P.ref(a[0]);
        const uint16_t* x1 = (const uint16_t*)P.ref(a[1]);
        if (!x0 || !x1) FAIL("add ref empty");
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)n * 2u, p);
        if (!y) FAIL("add temp alloc");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_binary(st, x0, x1, y, n, 0, false); };
        return;
    }
    case OP_SPILL: {  // exec_spill, :849-863
        p.stat = 11;
        uint32_t bytes = a[3] * 2u;
        const uint8_t* src = P.ref(a[0]);
        if (!src) FAIL("spill src empty");
        const uint8_t* pool = P.slot_ptr(a[1]);
        if (!pool || a[1] >= b->n_slots || (uint64_t)b->slots[a[1]].len < (uint64_t)a[2] + bytes) FAIL("spill pool oob");
        uint8_t* dst = (uint8_t*)pool + a[2];
        if (P.build) p.launch = [=](cudaStream_t st) { k_copy_bytes(st, src, dst, bytes); };
        return;
    }
    case OP_FILL: {  // exec_fill, :864-883
        p.stat = 12;
        uint32_t bytes = a[3] * 2u;
        const uint8_t* pool = P.slot_ptr(a[0]);
        if (!pool || a[0] >= b->n_slots || (uint64_t)b->slots[a[0]].len < (uint64_t)a[1] + bytes) FAIL("fill pool oob");
        const uint8_t* src = pool + a[1];
        uint8_t* dst = (a[2] & 0x8000u) ? (uint8_t*)P.slot_ptr(a[2] & 0x7FFFu) : P.temp_get(a[2], bytes, p);
        if (!dst) FAIL("fill dst empty");
        if (P.build) p.launch = [=](cudaStream_t st) { k_copy_bytes(st, src, dst, bytes); };
        return;
    }
    case OP_DMA: {  // exec_dma, :937-980 (engine faces do not exist here)
        uint32_t bytes = a[2], so = a[3], dof = a[4], fs = a[6], fd = a[7];
        if (bytes == 0) return;
        if ((fs > 3u && fs != WT_DMA_FENCE_NONE) || (fd > 3u && fd != WT_DMA_FENCE_NONE)) FAIL("dma fence arg bad");
        auto resolve = [&](uint32_t r, uint32_t off, bool is_dst) -> uint8_t* {
            if ((r & 0xC000u) == 0xC000u) return nullptr;
            if (r & 0x8000u) {
                uint32_t s = r & 0x7FFFu;
                const uint8_t* sp = P.slot_ptr(s);
                if (!sp || s >= b->n_slots || (uint64_t)off + bytes > b->slots[s].len) return nullptr;
                return (uint8_t*)sp + off;
            }
            if (r & 0x4000u) {
                uint32_t t = r & 0x3FFFu;
                if (t >= kMaxTemps || g.vtcm_off[t] == kNoOff) return nullptr;
                if ((uint64_t)g.vtcm_off[t] + off + bytes > g.vtcm_cap) return nullptr;
                return (uint8_t*)P.ref(r) + off;
            }
            if (r >= kMaxTemps) return nullptr;
            if (is_dst) { uint8_t* q = P.temp_get(r, (uint64_t)off + bytes, p); return q ? q + off : nullptr; }
            if (!P.written[r] || (uint64_t)off + bytes > P.cap[r]) return nullptr;
            return (uint8_t*)P.ref(r) + off;
        };
        uint8_t* src = resolve(a[0], so, false);
        uint8_t* dst = resolve(a[1], dof, true);
        if (!src || !dst) FAIL("dma ref fail");
        if (P.build) p.launch = [=](cudaStream_t st) { k_copy_bytes(st, src, dst, bytes); };
        return;
    }
    case OP_TRANSPOSE_F16: {  // exec_transpose, :983-1009
        p.stat = 13;
        uint32_t H = a[2], W = a[3], C = a[4], perm = a[5];
        const uint16_t* src = (const uint16_t*)P.ref(a[0]);
        if (!src) FAIL("transpose src ref empty");
        uint16_t* dst = (uint16_t*)P.temp_get(a[1], (uint64_t)H * W * C * 2u, p);
        if (!dst) FAIL("transpose temp alloc");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_transpose_hwc(st, src, dst, H, W, C, perm); };
        return;
    }
    case OP_UNARY_F16: {  // exec_unary, :1013-1079
        uint32_t n = a[2], sub = a[3];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)n * 2u, p);
        if (!x || !y) FAIL("unary ref fail");
        if (sub > 16u) FAIL("unary unknown subtype %u", sub);
        p.engine = WT_ENG_HVX;
        if (P.build) {
            if (sub == 14 && n >= 32u) p.launch = [=](cudaStream_t st) { k_copy_bytes(st, x, y, (size_t)n * 2u); };
            else p.launch = [=](cudaStream_t st) { k_unary(st, x, y, n, sub); };
        }
        return;
    }
    case OP_BINARY_F16: {  // exec_binary, :1081-1161
        uint32_t n = a[3], sub = a[4];
        p.engine = WT_ENG_HVX;
        if (sub == 8) {
            const uint16_t* c = (const uint16_t*)P.ref(a[0]);
            const uint16_t* tv = (const uint16_t*)P.ref(a[1]);
            const uint16_t* fv = (const uint16_t*)P.ref(a[2]);
            uint32_t cn = P.ref_count(a[0]), an = P.ref_count(a[1]), fn = P.ref_count(a[2]);
            uint32_t nn = cn > an ? cn : an;
            nn = fn > nn ? fn : nn;
            uint16_t* y = (uint16_t*)P.temp_get(a[3], (uint64_t)nn * 2u, p);
            if (!c || !tv || !fv || !y || nn == 0) FAIL("select ref fail");
            if (P.build) p.launch = [=](cudaStream_t st) { k_select(st, c, cn, tv, an, fv, fn, y, nn); };
            return;
        }
        const uint16_t* x0 = (const uint16_t*)P.ref(a[0]);
        const uint16_t* x1 = (const uint16_t*)P.ref(a[1]);
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)n * 2u, p);
        if (!x0 || !x1 || !y) FAIL("binary ref fail");
        bool guard = n < 32u;
        if (P.build) p.launch = [=](cudaStream_t st) { k_binary(st, x0, x1, y, n, sub, guard); };
        return;
    }
    case OP_SOFTMAX_F16: {  // exec_softmax, :1163-1194
        uint32_t rows = a[2], n = a[3];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)rows * n * 2u, p);
        if (!x || !y) FAIL("softmax ref fail");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_softmax(st, x, y, rows, n); };
        return;
    }
    case OP_CONCAT_F16: {  // exec_concat, :1196-1220
        uint32_t out_t = a[8], n_seg = a[10], n_elems = a[11];
        uint32_t sizes[4] = {a[12], a[13], a[14], a[15]};
        uint32_t total = 0;
        for (uint32_t i = 0; i < n_seg && i < 4; i++) total += sizes[i];
        if (total == 0 || n_elems % total != 0) FAIL("concat shape");
        uint32_t outer = n_elems / total;
        uint16_t* y = (uint16_t*)P.temp_get(out_t, (uint64_t)n_elems * 2u, p);
        if (!y) FAIL("concat out fail");
        const uint16_t* xs[4] = {nullptr, nullptr, nullptr, nullptr};
        for (uint32_t k = 0; k < n_seg && k < 4; k++) {
            xs[k] = (const uint16_t*)P.ref(a[k]);
            if (!xs[k]) FAIL("concat in fail");
        }
        p.engine = WT_ENG_HVX;
        if (P.build) {
            const uint16_t *x0 = xs[0], *x1 = xs[1], *x2 = xs[2], *x3 = xs[3];
            uint32_t s0 = sizes[0], s1 = sizes[1], s2 = sizes[2], s3 = sizes[3];
            p.launch = [=](cudaStream_t st) {
                const uint16_t* xv[4] = {x0, x1, x2, x3};
                uint32_t sv[4] = {s0, s1, s2, s3}, start = 0;
                for (uint32_t k = 0; k < n_seg && k < 4; k++) {
                    k_concat_seg(st, xv[k], y, outer, sv[k], total, start);
                    start += sv[k];
                }
            };
        }
        return;
    }
    case OP_SPLIT_F16: {  // exec_split, :1222-1256
        uint32_t x_t = a[0], n_seg = a[10], split_index = a[15];
        uint32_t sizes[4] = {a[11], a[12], a[13], a[14]};
        const uint16_t* x = (const uint16_t*)P.ref(x_t);
        if (!x) FAIL("split in fail");
        uint32_t total = 0;
        for (uint32_t i = 0; i < n_seg && i < 4; i++) total += sizes[i];
        if (total == 0) FAIL("split shape");
        uint32_t x_elems = 0;
        if ((x_t & 0x8000u) == 0 && x_t < kMaxTemps) x_elems = P.cap[x_t] / 2u;
        if (x_elems == 0) FAIL("split x size");
        uint32_t outer = x_elems / total, off = 0;
        p.engine = WT_ENG_HVX;
        for (uint32_t k = 0; k < n_seg && k < 4; k++) {
            if (k == split_index) {
                uint16_t* yk = (uint16_t*)P.temp_get(a[1], (uint64_t)outer * sizes[k] * 2u, p);
                if (!yk) FAIL("split out fail");
                uint32_t seg = sizes[k], o2 = off;
                if (P.build) p.launch = [=](cudaStream_t st) { k_split_seg(st, x, yk, outer, seg, total, o2); };
            }
            off += sizes[k];
        }
        return;
    }
    case OP_REDUCE_F16: {  // exec_reduce, :1258-1299
        uint32_t n = a[2], axis = a[3], sub = a[4];
        uint32_t d[4] = {a[5], a[6], a[7], a[8]};
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        if (!x) FAIL("reduce in fail");
        if (axis >= 4 || sub > 3) FAIL("reduce axis/subtype bad (axis=%u sub=%u)", axis, sub);
        uint32_t L = d[axis] ? d[axis] : 1, inner = 1;
        for (uint32_t k = axis + 1; k < 4; k++) inner *= d[k];
        if ((uint64_t)L * inner == 0 || n % (L * inner) != 0) FAIL("reduce geom (n=%u L=%u inner=%u)", n, L, inner);
        uint32_t outer = n / (L * inner);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)outer * inner * 2u, p);
        if (!y) FAIL("reduce out fail");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_reduce(st, x, y, outer, L, inner, sub); };
        return;
    }
    case OP_PAD_F16: {  // exec_pad, :1301-1318
        uint32_t outer = a[2], in_inner = a[3], out_inner = a[4], before = a[5];
        uint16_t pv = (uint16_t)a[6];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)outer * out_inner * 2u, p);
        if (!x || !y) FAIL("pad ref fail");
        if (before + in_inner > out_inner) FAIL("pad geom");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_pad(st, x, y, outer, in_inner, out_inner, before, pv); };
        return;
    }
    case OP_CUMSUM_F32: {  // exec_cumsum, :1320-1347
        uint32_t rows = a[2], n = a[3], excl = a[5], rev = a[6];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)rows * n * 2u, p);
        if (!x || !y) FAIL("cumsum ref fail");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_cumsum(st, x, y, rows, n, excl, rev); };
        return;
    }
    case OP_CONV1D_SSM_F16: {  // exec_conv1d_ssm, :1349-1376
        uint32_t seq = a[3], C = a[4], k = a[5];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        const uint16_t* w = (const uint16_t*)P.slot_ptr(a[1] & 0x7FFFu);
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)seq * C * 2u, p);
        if (!x || !w || !y) FAIL("ssm ref fail");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_conv1d_ssm(st, x, w, y, seq, C, k); };
        return;
    }
    case OP_GATHER_F16: {  // exec_gather, :1378-1432
        uint32_t n = a[3], packed = a[4];
        uint32_t axis = packed & 0xFF, xrank = (packed >> 8) & 0xFF, irank = (packed >> 16) & 0xFF;
        const uint16_t* tbl = (const uint16_t*)P.ref(a[0]);
        const int32_t* idx = (const int32_t*)P.ref(a[1]);
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)n * 2u, p);
        if (!tbl || !idx || !y) FAIL("gather ref fail");
        if (axis >= irank || irank > 5 || xrank > 5 || xrank == 0) FAIL("gather axis/rank bad (a=%u x=%u i=%u)", axis, xrank, irank);
        p.engine = WT_ENG_HVX;
        if (P.build) {
            std::vector<uint32_t> td(a + 5, a + 10), xd(a + 10, a + 15);
            p.launch = [=](cudaStream_t st) { k_gather(st, tbl, idx, y, n, axis, xrank, irank, td.data(), xd.data()); };
        }
        return;
    }
    case OP_SCATTER_ND_F16: {  // exec_scatter_nd, :1438-1470
        const uint16_t* data = (const uint16_t*)P.ref(a[0]);
        const int32_t* idxs = (const int32_t*)P.ref(a[1]);
        const uint16_t* upd = (const uint16_t*)P.ref(a[2]);
        uint32_t n = a[4], rank = a[5], K = a[11], n_idx = a[12], block = a[13];
        uint16_t* y = (uint16_t*)P.temp_get(a[3], (uint64_t)n * 2u, p);
        if (!data || !idxs || !upd || !y) FAIL("scatter_nd ref fail");
        if (rank < 1 || rank > 5 || K < 1 || K > rank) FAIL("scatter_nd rank/K");
        p.engine = WT_ENG_HVX;
        if (P.build) {
            std::vector<uint32_t> od(5, 1u);
            for (uint32_t i = 0; i < 5; i++) od[i] = (i < rank) ? a[6 + i] : 1u;
            p.launch = [=](cudaStream_t st) {
                k_copy_bytes(st, data, y, (size_t)n * 2u);
                k_scatter_nd(st, idxs, upd, y, n, K, n_idx, block, od.data());
            };
        }
        return;
    }
    case OP_ARGMAX_F16: {  // exec_argmax, :1990-2004
        uint32_t n = a[2];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        int32_t* y = (int32_t*)P.temp_get(a[1], 4u, p);
        if (!x || !y) FAIL("argmax ref fail");
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_argmax(st, x, y, n); };
        return;
    }
    case OP_KV_APPEND_F16: {  // exec_kv_append, :2154-2176
        const uint16_t* k = (const uint16_t*)P.ref(a[0]);
        const uint16_t* v = (const uint16_t*)P.ref(a[1]);
        uint32_t kn = P.ref_count(a[0]), vn = P.ref_count(a[1]);
        if (!k || !v || !kn || kn != vn) FAIL("kv append ref fail");
        KvGeom* c = kv_geom(a[2], kn, p);
        if (!c) return;
        uint32_t si = a[2] & 0x1FFFu, pos = a[3];
        if (pos == WT_KV_POS_AUTO) p.kv_append_state = (int)si;
        p.engine = WT_ENG_HVX;
        uint16_t* ring = (uint16_t*)g.st_buf[si];
        uint32_t* posmap = c->posmap; uint32_t* ctr = g.d_st_count + si; uint32_t ns = c->nslots;
        if (P.build) p.launch = [=](cudaStream_t st) { k_kv_append(st, k, v, ring, posmap, ctr, kn, ns, pos); };
        return;
    }
    case OP_KV_GATHER_F16: {  // exec_kv_gather, :2183-2231
        uint32_t n_kv = a[3], nh = a[4], kvh = a[5], hd = a[6];
        if (!nh || !kvh || !hd || nh % kvh != 0u) FAIL("kv gather gqa bad (h=%u kvh=%u hd=%u)", nh, kvh, hd);
        KvGeom* c = kv_geom(a[0], kvh * hd, p);
        if (!c) return;
        uint32_t si = a[0] & 0x1FFFu, pstride = n_kv;
        if (n_kv == WT_KV_POS_AUTO) { p.kv_gather_state = (int)si; pstride = c->nslots; }
        uint16_t* kT = a[1] ? (uint16_t*)P.temp_get(a[1], (uint64_t)nh * hd * pstride * 2u, p) : nullptr;
        uint16_t* vo = a[2] ? (uint16_t*)P.temp_get(a[2], (uint64_t)nh * pstride * hd * 2u, p) : nullptr;
        if ((!kT && a[1]) || (!vo && a[2])) FAIL("kv gather out alloc");
        p.engine = WT_ENG_HVX;
        const uint16_t* ring = (const uint16_t*)g.st_buf[si];
        const uint32_t* posmap = c->posmap; const uint32_t* ctr = g.d_st_count + si; uint32_t ns = c->nslots;
        unsigned int code = P.opi + 1;
        if (P.build) p.launch = [=](cudaStream_t st) {
            k_kv_gather(st, ring, posmap, ctr, kT, vo, n_kv, pstride, nh, kvh, hd, ns, g.d_status, code);
        };
        return;
    }
    case OP_MATMUL_F16:
    case OP_MATMUL_F16_SPLIT: {  // exec_matmul_f16, :1709-1813
        uint32_t M = a[3], K = a[4], N_full, n0, N, flags;
        if (op.opcode == OP_MATMUL_F16_SPLIT) { N_full = a[5]; n0 = a[6]; N = a[7]; flags = a[8]; }
        else { N_full = N = a[5]; n0 = 0; flags = a[6]; }
        int t0 = (int)(flags & 1u), t1 = (flags & 2u) ? 1 : 0;
        uint32_t Bn = (flags & 4u) ? (flags >> 16) : 1u;
        if (Bn == 0) Bn = 1;
        uint32_t Balloc = (flags >> 16) ? (flags >> 16) : 1u;
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        const uint16_t* w = (const uint16_t*)P.ref(a[1]);
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)M * N_full * Balloc * 2u, p);
        if (!x || !w || !y) FAIL("matmul_f16 ref fail");
        p.engine = WT_ENG_HVX;
        // Weights stored [N, K], one matrix: tensor cores (M >= 128) or the streaming GEMV (M < 32), unless
        // the one-kernel-per-op plan or a dump hook asks for the reference's summation order bit for bit.
        const bool nk = t1 && !t0 && !(flags & 4u);
        if (nk) p.engine = M >= 128 ? WT_ENG_HMX : WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) {
            if (nk && g.opt_fuse && !g.exact_ops &&
                k_matmul_f16_nk(st, x, w + (size_t)n0 * K, y + n0, M, K, N, N_full, g.d_status)) return;
            k_matmul_f16(st, x, w, y, M, K, N, n0, N_full, t0, t1, Bn);
        };
        return;
    }
    case OP_RMSNORM2_F16: {  // exec_rmsnorm2, :1817-1872
        uint32_t w_s = a[1] & 0x7FFFu, b_s = a[2] & 0x7FFFu, n = a[4];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        const uint16_t* wv = (const uint16_t*)P.slot_ptr(w_s);
        const uint16_t* bv = (const uint16_t*)P.slot_ptr(b_s);
        uint16_t* y = (uint16_t*)P.temp_get(a[3], (uint64_t)n * 2u, p);
        if (!x || !wv || !y) FAIL("rmsnorm2 ref fail");
        uint32_t rw = b->slots[w_s].len / 2u;
        if (rw == 0 || n % rw != 0) FAIL("rmsnorm2 shape n%u rw%u", n, rw);
        uint32_t m = n / rw;
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_rmsnorm(st, x, wv, bv, y, m, rw); };
        return;
    }
    case OP_BROADCAST_F16: {  // exec_broadcast, :1876-1907
        uint32_t n = a[2], b_elems = a[3];
        uint32_t in_d[4] = {a[4], a[5], a[6], a[7]}, out_d[4] = {a[8], a[9], a[10], a[11]};
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)n * 2u, p);
        if (!x || !y || b_elems == 0) FAIL("broadcast ref fail");
        uint32_t r = 4;
        while (r > 0 && out_d[r - 1] == 1) r--;
        uint32_t ir = 4;
        if (r == 0) r = 1;
        if (ir > r) ir = r;
        std::vector<uint32_t> istr(4, 1u), ostr(4, 1u), ind(in_d, in_d + 4);
        for (int i = (int)ir - 2; i >= 0; i--) istr[i] = istr[i + 1] * in_d[i + 1];
        for (int i = (int)r - 2; i >= 0; i--) ostr[i] = ostr[i + 1] * out_d[i + 1];
        for (auto& o : ostr) if (!o) o = 1;
        uint32_t lead = r - ir;
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_broadcast(st, x, y, n, r, lead, ind.data(), istr.data(), ostr.data()); };
        return;
    }
    case OP_TRANSPOSE_GEN_F16: {  // exec_transpose_gen, :1910-1948
        uint32_t rk = a[2], perm = a[7];
        uint32_t dims[4] = {a[3], a[4], a[5], a[6]};
        const uint16_t* s16 = (const uint16_t*)P.ref(a[0]);
        if (rk < 2 || rk > 4) FAIL("transpose_gen rank %u", rk);
        uint64_t n = 1;
        for (uint32_t i = 0; i < rk; i++) n *= dims[i];
        uint16_t* dst = (uint16_t*)P.temp_get(a[1], (uint64_t)(uint32_t)n * 2u, p);
        if (!s16 || !dst) FAIL("transpose_gen ref fail");
        std::vector<uint32_t> pv = {perm & 0xFF, (perm >> 8) & 0xFF, (perm >> 16) & 0xFF, (perm >> 24) & 0xFF};
        std::vector<uint32_t> si(4, 1u), so(4, 1u);
        for (int i = (int)rk - 2; i >= 0; i--) {
            si[i] = si[i + 1] * dims[i + 1];
            uint32_t pd = pv[i + 1] >= rk ? 1u : dims[pv[i + 1]];
            so[i] = so[i + 1] * pd;
        }
        for (auto& s : si) if (!s) s = 1;
        uint32_t nn = (uint32_t)n;
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_transpose_gen(st, s16, dst, nn, rk, si.data(), so.data(), pv.data()); };
        return;
    }
    case OP_STRIDED_SLICE_F16: {  // exec_slice, :1950-1988
        uint32_t n_out = a[2], rk = a[3];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        uint16_t* y = (uint16_t*)P.temp_get(a[1], (uint64_t)n_out * 2u, p);
        if (!x || !y) FAIL("slice ref fail");
        if (rk < 1 || rk > 3) FAIL("slice rank %u", rk);
        std::vector<uint32_t> bb = {a[4], a[5], a[6]}, ee = {a[7], a[8], a[9]}, ss = {a[10], a[11], a[12]}, dd = {a[13], a[14], a[15]};
        std::vector<uint32_t> od(3, 1u), istr(3, 1u), ostr(3, 1u);
        for (uint32_t ax = 0; ax < rk; ax++) {
            if (ss[ax] == 0) ss[ax] = 1;
            uint32_t span = (ee[ax] > bb[ax]) ? ee[ax] - bb[ax] : 0;
            od[ax] = (span + ss[ax] - 1) / ss[ax];
        }
        for (int i = (int)rk - 2; i >= 0; i--) { istr[i] = istr[i + 1] * dd[i + 1]; ostr[i] = ostr[i + 1] * od[i + 1]; }
        for (auto& o : ostr) if (!o) o = 1;
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_slice(st, x, y, n_out, rk, bb.data(), ss.data(), istr.data(), ostr.data()); };
        return;
    }
    case OP_CONV1D_SSM_STEP_F16: {  // exec_conv1d_ssm_step, :2235-2257
        uint32_t C = a[4], dc = a[5];
        const uint16_t* x = (const uint16_t*)P.ref(a[0]);
        const uint16_t* w = (const uint16_t*)P.ref(a[1]);
        uint16_t* y = (uint16_t*)P.temp_get(a[2], (uint64_t)C * 2u, p);
        if (!x || !y || !w) FAIL("ssm step ref fail");
        if ((a[1] & 0x7FFFu) >= b->n_slots || b->slots[a[1] & 0x7FFFu].len != dc * C * 2u) FAIL("ssm step w slot len mismatch");
        if (dc < 2 || C == 0) FAIL("ssm step shape C=%u dc=%u", C, dc);
        if ((a[3] & 0xE000u) != WT_REF_STATE_FLAG) FAIL("ssm step state_ref bad");
        uint32_t si = a[3] & 0x1FFFu;
        if (si >= g.n_states || g.st_bytes[si] < (uint64_t)(dc - 1u) * C * 4u) FAIL("ssm step state %u too small", si);
        float* win = (float*)g.st_buf[si];
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) { k_conv1d_step(st, x, w, y, win, C, dc); };
        return;
    }
    case OP_DELTA_CHUNK_F16: {  // exec_delta_chunk, :2261-2288
        uint32_t c = a[7], ntok = a[8], H = a[9], D = a[10], q_raw = a[11];
        const uint16_t* k = (const uint16_t*)P.ref(a[0]);
        const uint16_t* v = (const uint16_t*)P.ref(a[1]);
        const uint16_t* q = (const uint16_t*)P.ref(a[2]);
        const uint16_t* be = (const uint16_t*)P.ref(a[3]);
        const uint16_t* gg = (const uint16_t*)P.ref(a[4]);
        uint16_t* y = (uint16_t*)P.temp_get(a[5], (uint64_t)H * ntok * D * 2u, p);
        if (!k || !v || !q || !be || !gg || !y) FAIL("delta ref fail");
        if (!H || !D || !ntok || !c || c > ntok || c > 64u) FAIL("delta shape (c=%u ntok=%u H=%u D=%u)", c, ntok, H, D);
        if ((a[6] & 0xE000u) != WT_REF_STATE_FLAG) FAIL("delta state_ref bad");
        uint32_t si = a[6] & 0x1FFFu;
        if (si >= g.n_states || g.st_bytes[si] < (uint64_t)H * D * D * 4u) FAIL("delta state %u too small", si);
        if ((uint64_t)4 * c * (D + 1) * 4 + 17408 > 227u * 1024u) FAIL("delta chunk c=%u D=%u exceeds shared memory", c, D);
        float* S = (float*)g.st_buf[si];
        p.engine = WT_ENG_HVX;
        if (P.build) p.launch = [=](cudaStream_t st) {
            // fused plans take the tensor-core form; the one-kernel-per-op plan keeps the scalar loops in the reference's order
            if (g.opt_fuse && !g.exact_ops && k_delta_chunk_mma(st, k, v, q, be, gg, y, S, c, ntok, H, D, q_raw)) return;
            k_delta_chunk(st, k, v, q, be, gg, y, S, c, ntok, H, D, q_raw);
        };
        return;
    }
    default:
        FAIL("opcode %u unhandled", (unsigned)op.opcode);
    }
}

// TEMPOFF table: [cap][reserve = vtcm_kb<<16 | bump_kb][n] n x {tid, off, size}
// (wt_exec_load_tempoff, oplist_exec.c:2012-2066).
int load_tempoff(const wt_blob* b, char* err, size_t errn) {
    for (uint32_t i = 0; i < kMaxTemps; i++) { g.static_off[i] = kNoOff; g.vtcm_off[i] = kNoOff; }
    g.have_static = false; g.static_cap = 0; g.vtcm_cap = 0;
    if (g.user_pool) {
        g.have_static = !g.user_off.empty();
        g.static_cap = g.user_static ? g.user_static : g.user_total;
        for (uint32_t i = 0; i < kMaxTemps && i < g.user_off.size(); i++) g.static_off[i] = g.user_off[i];
        return 0;
    }
    for (uint32_t s = 0; s < b->n_slots; s++) {
        if (b->slots[s].addr != WT_SLOT_TEMPOFF) continue;
        const uint8_t* p = b->weight_base + b->slots[s].offset;
        uint32_t len = b->slots[s].len;
        if (len < 12u) { std::snprintf(err, errn, "tempoff slot short"); return -1; }
        uint32_t cap = wt_rd_u32(p), reserve = wt_rd_u32(p + 4), n = wt_rd_u32(p + 8);
        if ((uint64_t)len < 12ull + (uint64_t)n * 12u) { std::snprintf(err, errn, "tempoff table short"); return -1; }
        if (cap == 0 || cap > 0x80000000u) { std::snprintf(err, errn, "tempoff cap bad"); return -1; }
        uint32_t vtcm_cap = (reserve >> 16) * 1024u;
        for (uint32_t i = 0; i < n; i++) {
            const uint8_t* e = p + 12 + (size_t)i * 12;
            uint32_t tid = wt_rd_u32(e), off = wt_rd_u32(e + 4), sz = wt_rd_u32(e + 8);
            uint32_t clean = tid & 0x3FFFu;
            if (clean >= kMaxTemps) { std::snprintf(err, errn, "tempoff tid bad %u", clean); return -1; }
            if (tid & WT_REF_VTCM_FLAG) {
                if (vtcm_cap == 0 || (uint64_t)off + sz > vtcm_cap) {
                    std::snprintf(err, errn, "tempoff vtcm entry bad (tid %u off %u sz %u vtcm_cap %u)", clean, off, sz, vtcm_cap);
                    return -1;
                }
                g.vtcm_off[clean] = off;
            } else {
                if ((uint64_t)off + sz > cap) {
                    std::snprintf(err, errn, "tempoff entry bad (tid %u off %u sz %u cap %u)", clean, off, sz, cap);
                    return -1;
                }
                g.static_off[clean] = off;
            }
        }
        g.have_static = true; g.static_cap = cap; g.vtcm_cap = vtcm_cap;
        break;
    }
    return 0;
}

// STATE table: [n] n x {bytes}; buffers are zeroed once and live until the
// process ends or a blob with a different table is run
// (wt_exec_load_states, oplist_exec.c:2071-2102). A state may be up to
// 4 GiB - 1 here (the reference stops at 1 GiB).
int load_states(const wt_blob* b, char* err, size_t errn) {
    for (uint32_t s = 0; s < b->n_slots; s++) {
        if (b->slots[s].addr != WT_SLOT_STATE) continue;
        const uint8_t* p = b->weight_base + b->slots[s].offset;
        uint32_t len = b->slots[s].len;
        if (len < 4u) { std::snprintf(err, errn, "state slot short"); return -1; }
        uint32_t n = wt_rd_u32(p);
        if (n == 0 || n > WT_MAX_STATES || (uint64_t)len < 4ull + (uint64_t)n * 4u) {
            std::snprintf(err, errn, "state slot table bad (n=%u len=%u)", n, len);
            return -1;
        }
        // Same table as the states already resident: keep them (decode semantics).
        // A different table means a different model: the old states are released.
        bool same = g.states_loaded && g.n_states == n;
        for (uint32_t i = 0; same && i < n; i++) same = g.st_bytes[i] == wt_rd_u32(p + 4 + (size_t)i * 4);
        if (same) return 0;
        for (uint32_t i = 0; i < g.n_states; i++) {
            cudaFree(g.st_buf[i]); g.st_buf[i] = nullptr;
            if (g.kv[i].posmap) cudaFree(g.kv[i].posmap);
            g.kv[i] = KvGeom();
        }
        g.n_states = 0;
        cudaMemsetAsync(g.d_st_count, 0, 2 * WT_MAX_STATES * sizeof(uint32_t), g.stream);
        for (uint32_t i = 0; i < n; i++) {
            uint32_t bytes = wt_rd_u32(p + 4 + (size_t)i * 4);
            if (bytes == 0) { std::snprintf(err, errn, "state %u bytes bad %u", i, bytes); return -1; }
            if (cudaMalloc(&g.st_buf[i], bytes) != cudaSuccess) {
                cudaGetLastError();
                std::snprintf(err, errn, "state %u alloc %u", i, bytes);
                return -1;
            }
            cudaMemsetAsync(g.st_buf[i], 0, bytes, g.stream);
            g.st_bytes[i] = bytes;
            g.st_count[i] = 0;
            g.n_states = i + 1;
        }
        break;
    }
    g.states_loaded = true;
    return 0;
}

bool ranges_clash(const std::vector<LiveRange>& x, const std::vector<LiveRange>& y) {
    for (const auto& a : x)
        for (const auto& c : y)
            if (a.w <= c.r && c.w <= a.r) return true;
    return false;
}

}  // namespace

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int build_plan(const wt_blob* b, char* err, size_t errn) {
    char scratch[200];
    if (!err) { err = scratch; errn = sizeof scratch; }
    if (load_tempoff(b, err, errn) != 0) return -1;
    if (load_states(b, err, errn) != 0) return -1;

    // device copies of the slot data
    if (b->weight_bytes) {
        if (cudaMalloc(&g.d_weights, b->weight_bytes) != cudaSuccess) { std::snprintf(err, errn, "weights alloc %zu", b->weight_bytes); return -1; }
        g.weights_bytes = b->weight_bytes;
        cudaMemcpyAsync(g.d_weights, b->weight_base, b->weight_bytes, cudaMemcpyHostToDevice, g.stream);
    }
    for (uint32_t s = 0; s < b->n_slots; s++) {
        const wt_slot& sl = b->slots[s];
        if (sl.addr != WT_SLOT_EXT_IN && sl.addr != WT_SLOT_EXT_WGT) continue;
        if (sl.addr == WT_SLOT_EXT_WGT && !g.ext_wgt) continue;
        uint8_t* d = nullptr;
        if (cudaMalloc(&d, align_up(sl.len, 256)) != cudaSuccess) { std::snprintf(err, errn, "ext slot %u alloc", s); return -1; }
        const uint8_t* src = sl.addr == WT_SLOT_EXT_WGT ? g.ext_wgt + sl.offset
                             : (sl.offset + sl.len <= b->weight_bytes ? b->weight_base + sl.offset : nullptr);
        if (src) cudaMemcpyAsync(d, src, sl.len, cudaMemcpyHostToDevice, g.stream);
        else cudaMemsetAsync(d, 0, sl.len, g.stream);
        g.d_ext[s] = d;
    }

    // measuring walk
    std::vector<Planner> holder(1);
    Planner& P = holder[0];
    auto reset_walk = [&](bool build) {
        P.b = b; P.build = build;
        std::memset(P.written, 0, sizeof P.written);
        std::memset(P.cap, 0, sizeof P.cap);
        std::memset(P.last, 0, sizeof P.last);
    };
    reset_walk(false);
    std::memset(P.maxb, 0, sizeof P.maxb);
    std::memset(P.internal, 0, sizeof P.internal);
    std::memset(P.oversize, 0, sizeof P.oversize);
    std::vector<PlanOp> meas(b->n_ops);
    for (uint32_t i = 0; i < b->n_ops; i++) { P.opi = i; P.cur = &meas[i]; plan_op(P, b->ops[i], meas[i]); }
    const bool fusing = g.opt_fuse && !g.force_unfused;
    std::vector<uint8_t> dead_ops;
    if (fusing) {
        std::vector<uint8_t> internal;
        fuse_analyze(b, meas, internal, dead_ops);
        for (uint32_t i = 0; i < kMaxTemps; i++) P.internal[i] = internal[i] != 0;
    }

    // static-pool entries that would overwrite each other while both are live
    g.demoted_temps = 0;
    for (uint32_t i = 0; i < kMaxTemps; i++) P.in_static[i] = g.have_static && g.static_off[i] != kNoOff && g.vtcm_off[i] == kNoOff;
    if (g.have_static) {
        std::vector<uint32_t> ids;
        for (uint32_t i = 0; i < kMaxTemps; i++) if (P.in_static[i] && P.maxb[i]) ids.push_back(i);
        for (size_t x = 0; x < ids.size(); x++)
            for (size_t y = x + 1; y < ids.size(); y++) {
                uint32_t i = ids[x], j = ids[y];
                if (!P.in_static[i] || !P.in_static[j]) continue;
                uint64_t a0 = g.static_off[i], a1 = a0 + P.maxb[i], b0 = g.static_off[j], b1 = b0 + P.maxb[j];
                if (a0 < b1 && b0 < a1 && ranges_clash(P.live[i], P.live[j])) {
                    P.in_static[j] = false;
                    g.demoted_temps++;
                }
            }
        if (g.demoted_temps && g.trace_on)
            std::fprintf(stderr, "[gehtp] %u temps moved out of the static pool (offset table aliases live tensors)\n", g.demoted_temps);
    }

    // arena: static pool | on-chip-resident region | one region per other temp
    g.vtcm_base = align_up((size_t)g.static_cap, 256);
    size_t off = g.vtcm_base + align_up((size_t)g.vtcm_cap, 256);
    std::vector<size_t> toff(kMaxTemps, 0);
    for (uint32_t i = 0; i < kMaxTemps; i++) {
        if (!P.maxb[i] || P.in_static[i] || g.vtcm_off[i] != kNoOff) continue;
        if (P.internal[i]) { P.maxb[i] = 0; continue; }
        toff[i] = off;
        off += align_up(P.maxb[i], 256);
    }
    g.arena_bytes = off ? off : 256;
    if (cudaMalloc(&g.d_arena, g.arena_bytes) != cudaSuccess) { std::snprintf(err, errn, "temp arena alloc %zu", g.arena_bytes); return -1; }
    cudaMemsetAsync(g.d_arena, 0, g.arena_bytes, g.stream);
    for (uint32_t i = 0; i < kMaxTemps; i++) {
        if (g.vtcm_off[i] != kNoOff) P.addr[i] = g.d_arena + g.vtcm_base + g.vtcm_off[i];
        else if (P.in_static[i]) P.addr[i] = g.d_arena + g.static_off[i];
        else P.addr[i] = P.maxb[i] ? g.d_arena + toff[i] : nullptr;
        g.temp_dev[i] = nullptr; g.temp_cap[i] = 0; g.temp_last[i] = 0;
    }

    // building walk
    reset_walk(true);
    g.plan.assign(b->n_ops, PlanOp());
    for (uint32_t i = 0; i < b->n_ops; i++) { P.opi = i; P.cur = &g.plan[i]; plan_op(P, b->ops[i], g.plan[i]); }
    // tensor parallel: outputs named as partial sums are all-reduced right after their op
    if (g.tp_world > 1)
        for (uint32_t i = 0; i < b->n_ops && i < g_allreduce_after.size(); i++) {
            PlanOp& p = g.plan[i];
            if (!g_allreduce_after[i] || p.rc || !p.launch || p.out_id[0] == kNoOff) continue;
            void* buf = P.addr[p.out_id[0]];
            size_t elems = p.out_bytes[0] / 2;
            auto inner = p.launch;
            p.launch_local = inner;
            p.launch = [=](cudaStream_t st) { inner(st); tp_allreduce_f16(st, buf, elems); };
        }
    // run-time temp table starts empty; addresses appear as ops execute
    for (uint32_t i = 0; i < kMaxTemps; i++) g.temp_dev[i] = P.addr[i];

    g.fused_ops = 0;
    g.const_ops = 0;
    if (fusing) {
        fuse_materialize(b);
        // only when every chain really got its kernel: a chain left op-by-op still reads those results
        if (fuse_all_materialized())
            for (uint32_t i = 0; i < b->n_ops && i < dead_ops.size(); i++) g.plan[i].dead_when_fused = dead_ops[i] != 0;
        fold_constants(b, P.addr, P.maxb);
    }
    cudaError_t ce = cudaStreamSynchronize(g.stream);
    if (ce != cudaSuccess) { std::snprintf(err, errn, "plan upload: %s", cudaGetErrorString(ce)); return -1; }
    g.blob = b; g.blob_wbase = b->weight_base; g.blob_nops = b->n_ops; g.blob_nslots = b->n_slots;
    g.planned = true;
    return 0;
}

void drop_plan(bool keep_states) {
    if (g.graph) { cudaGraphExecDestroy(g.graph); g.graph = nullptr; }
    g.plan.clear();
    g.planned = false; g.blob = nullptr; g.warm_runs = 0;
    if (g.d_weights) { cudaFree(g.d_weights); g.d_weights = nullptr; }
    for (auto& kv : g.d_ext) cudaFree(kv.second);
    g.d_ext.clear();
    for (auto& kv : g.w4) cudaFree(kv.second.packed);
    g.w4.clear();
    fuse_release();
    if (g.d_arena) { cudaFree(g.d_arena); g.d_arena = nullptr; }
    g.arena_bytes = 0;
    for (uint32_t i = 0; i < kMaxTemps; i++) { g.temp_dev[i] = nullptr; g.temp_cap[i] = 0; g.temp_last[i] = 0; }
    for (auto& m : g.mirrors) cudaFreeHost(m.second.first);
    g.mirrors.clear();
    (void)keep_states;
}

}  // namespace gehtp
