// Plan-time fusion: recognises op chains of the runlist and replaces each by one to three launches. The chains
// are the shapes the reference's emitter decomposes ONNX graphs into (one op per node):
//
//   decode attention    SPLIT x3, rotary on q and k (mul / slice / slice / neg / concat / mul / add, twice),
//                       KV_APPEND (AUTO position), KV_GATHER K^T and V, batched MATMUL_F16 scores, BINARY scale by a
//                       broadcast constant, ADD mask, SOFTMAX, batched MATMUL_F16 with V
//                                               -> rotary + append (in the q|k|v projection's epilogue where it can),
//                                                  split-KV attention kernel, merge kernel
//   SwiGLU              W4A16 gate, UNARY sigmoid, BINARY mul, W4A16 up, BINARY mul
//                                               -> one GEMV over both matrices (few rows), one tcgen05 GEMM with both
//                                                  accumulators in TMEM (64 rows and up), or two GEMMs + one
//                                                  elementwise kernel (widths the GEMM does not take)
//   residual + norm     ADD followed by RMSNORM2 of its result -> one kernel; behind a W4A16 GEMM: in the kernel that
//                       adds the GEMM's split-K runs
//   rotary              the 7-op rotary chain on its own -> one kernel
//   prefill attention   TRANSPOSE_GEN x3, scores, scale, mask, SOFTMAX, P V, TRANSPOSE_GEN -> tcgen05 attention
//   prefill q|k|v head  SPLIT x3 + two rotary chains (17 ops) -> one kernel
//   transposition + GEMM  [heads][rows][d] -> [rows][heads d] in front of a W4A16 GEMM -> the GEMM reads the
//                       untransposed tensor through a three-dimensional tensor map
// and marks the data-movement ops whose result is a constant of the blob (fold_constants).
//
// A chain is fused only when every intermediate temp is consumed inside the
// chain and the chain's ops are contiguous in the list. Temps that exist only
// inside fused chains get no arena memory; running such an op on its own
// (run_range pieces, dump hooks) makes the engine rebuild the plan unfused.
#include <algorithm>
#include <cstring>
#include <map>
#include <utility>
#include "engine.h"
#include "launchers_attn.h"
#include "launchers_w4.h"

namespace gehtp {

namespace {

struct Graph {
    const wt_blob* b;
    std::vector<std::vector<uint32_t>> users;   // op -> ops reading one of its outputs
    std::vector<int> producer_of_arg[WT_MAX_ARGS];  // [arg][op] -> producing op or -1
};

// argument positions that read a tensor, per opcode
int input_args(const wt_op& op, int out[8]) {
    int n = 0;
    auto add = [&](int i) { out[n++] = i; };
    switch (op.opcode) {
    case OP_MATMUL_W4A16: case OP_ADD_F16: case OP_GATHER_F16: case OP_KV_APPEND_F16:
    case OP_MATMUL_F16: case OP_MATMUL_F16_SPLIT: case OP_CONV1D_SSM_STEP_F16:
        add(0); add(1); break;
    case OP_BINARY_F16: add(0); add(1); if (op.args[4] == 8) add(2); break;
    case OP_SCATTER_ND_F16: add(0); add(1); add(2); break;
    case OP_DELTA_CHUNK_F16: for (int i = 0; i < 5; i++) add(i); break;
    case OP_CONCAT_F16: for (uint32_t i = 0; i < op.args[10] && i < 4; i++) add((int)i); break;
    case OP_SILU_F16: case OP_UNARY_F16: case OP_SOFTMAX_F16: case OP_STRIDED_SLICE_F16: case OP_SPLIT_F16:
    case OP_REDUCE_F16: case OP_CUMSUM_F32: case OP_CONV1D_SSM_F16: case OP_ARGMAX_F16: case OP_RMSNORM2_F16:
    case OP_BROADCAST_F16: case OP_TRANSPOSE_GEN_F16: case OP_PAD_F16: case OP_TRANSPOSE_F16: case OP_IM2COL:
    case OP_CONV2D_F16: case OP_SPILL: case OP_DMA:
        add(0); break;
    default: break;
    }
    return n;
}

bool is_temp_ref(uint32_t a) { return (a & 0xC000u) == 0 && a < kMaxTemps; }

void build_graph(const wt_blob* b, const std::vector<PlanOp>& meas, Graph& G) {
    G.b = b;
    G.users.assign(b->n_ops, {});
    for (auto& v : G.producer_of_arg) v.assign(b->n_ops, -1);
    std::vector<int> cur(kMaxTemps, -1);
    for (uint32_t i = 0; i < b->n_ops; i++) {
        const wt_op& op = b->ops[i];
        int ia[8];
        int n = input_args(op, ia);
        for (int k = 0; k < n; k++) {
            uint32_t a = op.args[ia[k]];
            if (!is_temp_ref(a) || cur[a] < 0) continue;
            G.producer_of_arg[ia[k]][i] = cur[a];
            G.users[cur[a]].push_back(i);
        }
        for (int k = 0; k < 2; k++)
            if (meas[i].out_id[k] != kNoOff) cur[meas[i].out_id[k]] = (int)i;
    }
}

struct Rope {
    bool ok = false;
    int src_op = -1;          // producer of x
    uint32_t x, cos_b, sin_b, rows, hd, out_op;
    std::vector<uint32_t> ops;
};

// out = ADD(xc, xs); xc = MUL(x, cos); xs = MUL(CONCAT(NEG(SLICE(x, h:)), SLICE(x, :h)), sin)
Rope match_rope(const Graph& G, int add_op) {
    Rope r;
    const wt_blob* b = G.b;
    if (add_op < 0 || b->ops[add_op].opcode != OP_ADD_F16) return r;
    int xc = G.producer_of_arg[0][add_op], xs = G.producer_of_arg[1][add_op];
    if (xc < 0 || xs < 0) return r;
    auto is_mul = [&](int i) { return b->ops[i].opcode == OP_BINARY_F16 && b->ops[i].args[4] == 2; };
    if (!is_mul(xc) || !is_mul(xs)) return r;
    int cat = G.producer_of_arg[0][xs];
    if (cat < 0 || b->ops[cat].opcode != OP_CONCAT_F16) return r;
    const wt_op& c = b->ops[cat];
    if (c.args[10] != 2 || c.args[12] != c.args[13]) return r;
    uint32_t h = c.args[12], hd = 2 * h;
    int neg = G.producer_of_arg[0][cat], x1 = G.producer_of_arg[1][cat];
    if (neg < 0 || x1 < 0 || b->ops[neg].opcode != OP_UNARY_F16 || b->ops[neg].args[3] != 0) return r;
    int x2 = G.producer_of_arg[0][neg];
    if (x2 < 0 || b->ops[x1].opcode != OP_STRIDED_SLICE_F16 || b->ops[x2].opcode != OP_STRIDED_SLICE_F16) return r;
    const wt_op &s1 = b->ops[x1], &s2 = b->ops[x2], &m = b->ops[xc];
    uint32_t x = m.args[0];
    if (s1.args[0] != x || s2.args[0] != x) return r;
    uint32_t n = b->ops[add_op].args[3];
    if (n % hd) return r;
    uint32_t rows = n / hd;
    // rank-2 slices [rows, hd] -> columns [0,h) and [h,hd), unit strides
    auto slice_ok = [&](const wt_op& s, uint32_t c0, uint32_t c1) {
        return s.args[3] == 2 && s.args[4] == 0 && s.args[5] == c0 && s.args[7] == rows && s.args[8] == c1 &&
               s.args[10] <= 1 && s.args[11] <= 1 && s.args[13] == rows && s.args[14] == hd && s.args[2] == rows * h;
    };
    if (!slice_ok(s1, 0, h) || !slice_ok(s2, h, hd)) return r;
    if (m.args[3] != n || b->ops[xs].args[3] != n || c.args[11] != n || b->ops[neg].args[2] != rows * h) return r;
    r.ok = true;
    r.x = x; r.cos_b = m.args[1]; r.sin_b = b->ops[xs].args[1]; r.rows = rows; r.hd = hd; r.out_op = (uint32_t)add_op;
    r.src_op = G.producer_of_arg[0][xc];
    r.ops = {(uint32_t)xc, (uint32_t)x1, (uint32_t)x2, (uint32_t)neg, (uint32_t)cat, (uint32_t)xs, (uint32_t)add_op};
    return r;
}

struct Span {
    int kind;                // 0 decode attention, 1 swiglu, 2 add+norm, 3 rotary, 4 prefill attention,
                             // 5 prefill split + rotary of q|k|v, 6 swiglu tail behind two GEMMs,
                             // 7 [head][row][d] -> [row][head * d] transposition in front of a W4A16 GEMM,
                             // 8 per-row SLICE + ARGMAX of a matrix joined by a CONCAT tree (greedy sampling of a batch)
    uint32_t first, count;
    std::vector<uint32_t> ops;
    // attention
    uint32_t qkv, cos_q, sin_q, cos_k, sin_k, q_out, mask, ctx, state, B, nh, kvh, hd, nslots, pos;
    float scale; int scale_div;
    // swiglu
    uint32_t a_ref, wg, wu, y, M, K, N;
    // add+norm
    uint32_t add_a, add_b, sum_t, gamma_s, beta_s, norm_y, n;
    // rotary on its own (kind 3): x, cos_q, sin_q, y, rows = M, hd
    // prefill attention (kind 4): q/k/v inputs, mask operand (+ constant mask slot when known), ctx, seq_q = M, seq_k = N
    uint32_t pq, pk, pv, mask_slot; bool mask_is_slot;
    // decode attention: index of the W4A16 q|k|v projection when it sits right before the chain and
    // nothing but the chain reads its output (its epilogue can then do the rotary + append), else -1
    int qkv_lin = -1;
    // kind 5, split + rotary of a prefill block: qkv in, q_out / k_out / v_out, B = tokens
    // kind 6, SwiGLU around two GEMMs: ops gate_op and up_op keep their launches, a_ref/y as kind 1, n values
    uint32_t k_out, v_out, gate_op, up_op, gate_t, up_t;
    std::vector<uint32_t> keep;   // ops inside the span whose outputs stay materialised (besides the last)
};

bool contiguous(std::vector<uint32_t>& ops, uint32_t& first) {
    std::sort(ops.begin(), ops.end());
    ops.erase(std::unique(ops.begin(), ops.end()), ops.end());
    first = ops.front();
    return ops.back() - ops.front() + 1 == ops.size();
}

// every op of the span except `outs` is read only by ops of the span
bool closed(const Graph& G, const std::vector<uint32_t>& ops, std::initializer_list<uint32_t> outs) {
    for (uint32_t o : ops) {
        if (std::find(outs.begin(), outs.end(), o) != outs.end()) continue;
        for (uint32_t u : G.users[o])
            if (!std::binary_search(ops.begin(), ops.end(), u)) return false;
    }
    return true;
}

bool const_scalar(const Graph& G, int bc_op, float& v) {
    const wt_blob* b = G.b;
    if (bc_op < 0 || b->ops[bc_op].opcode != OP_BROADCAST_F16) return false;
    uint32_t src = b->ops[bc_op].args[0];
    if (!(src & 0x8000u) || b->ops[bc_op].args[3] != 1) return false;
    const wt_slot& s = b->slots[src & 0x7FFFu];
    if (s.addr != 0 || s.len < 2) return false;
    uint16_t h;
    std::memcpy(&h, b->weight_base + s.offset, 2);
    // fp16 -> fp32 on the host
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, bits;
    if (e == 0) {
        if (!m) bits = sign;
        else { int sh = 0; while (!(m & 1024u)) { m <<= 1; sh++; } bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13); }
    } else if (e == 31u) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    std::memcpy(&v, &bits, 4);
    return true;
}

bool match_attention(const Graph& G, uint32_t ia, Span& sp) {
    const wt_blob* b = G.b;
    const wt_op& ap = b->ops[ia];
    if (ap.opcode != OP_KV_APPEND_F16 || ap.args[3] != WT_KV_POS_AUTO) return false;
    uint32_t state = ap.args[2];
    Rope rk = match_rope(G, G.producer_of_arg[0][ia]);
    int vsplit = G.producer_of_arg[1][ia];
    if (!rk.ok || vsplit < 0 || rk.src_op < 0) return false;
    const wt_op &ks = b->ops[rk.src_op], &vs = b->ops[vsplit];
    if (ks.opcode != OP_SPLIT_F16 || vs.opcode != OP_SPLIT_F16 || ks.args[0] != vs.args[0]) return false;
    if (ks.args[10] != 3 || ks.args[15] != 1 || vs.args[15] != 2 || vs.args[10] != 3) return false;
    uint32_t s0 = ks.args[11], s1 = ks.args[12], s2 = ks.args[13], hd = rk.hd;
    if (s1 != s2 || s0 % hd || s1 % hd || vs.args[11] != s0 || vs.args[12] != s1 || vs.args[13] != s2) return false;
    uint32_t nh = s0 / hd, kvh = s1 / hd;
    if (!kvh || nh % kvh || rk.rows % kvh) return false;
    uint32_t B = rk.rows / kvh;
    // ops after the append, in list order
    uint32_t j = ia + 1;
    uint32_t kT = 0, vv = 0;
    std::vector<uint32_t> ops;
    while (j < b->n_ops && b->ops[j].opcode == OP_KV_GATHER_F16 && b->ops[j].args[0] == state) {
        const wt_op& gop = b->ops[j];
        if (gop.args[3] != WT_KV_POS_AUTO || gop.args[4] != B * nh || gop.args[5] != B * kvh || gop.args[6] != hd) return false;
        if (gop.args[1]) kT = gop.args[1];
        if (gop.args[2]) vv = gop.args[2];
        ops.push_back(j++);
    }
    if (!kT || !vv || j + 5 > b->n_ops) return false;
    const wt_op &sc = b->ops[j], &bi = b->ops[j + 1], &ad = b->ops[j + 2], &sm = b->ops[j + 3], &pv = b->ops[j + 4];
    if (sc.opcode != OP_MATMUL_F16 || bi.opcode != OP_BINARY_F16 || ad.opcode != OP_ADD_F16 ||
        sm.opcode != OP_SOFTMAX_F16 || pv.opcode != OP_MATMUL_F16) return false;
    uint32_t H = B * nh, nslots = sc.args[5];
    if (sc.args[1] != kT || sc.args[3] != 1 || sc.args[4] != hd || (sc.args[6] & 7u) != 4u || (sc.args[6] >> 16) != H) return false;
    if (bi.args[0] != sc.args[2] || (bi.args[4] != 2 && bi.args[4] != 3) || bi.args[3] != H * nslots) return false;
    if (ad.args[0] != bi.args[2] || ad.args[3] != H * nslots) return false;
    if (sm.args[0] != ad.args[2] || sm.args[2] != H || sm.args[3] != nslots) return false;
    if (pv.args[0] != sm.args[1] || pv.args[1] != vv || pv.args[3] != 1 || pv.args[4] != nslots || pv.args[5] != hd ||
        (pv.args[6] & 7u) != 4u || (pv.args[6] >> 16) != H) return false;
    float scale;
    if (!const_scalar(G, G.producer_of_arg[1][j + 1], scale)) return false;
    // q: rotary over SPLIT index 0 of the same qkv
    Rope rq = match_rope(G, G.producer_of_arg[0][j]);
    if (!rq.ok || rq.hd != hd || rq.rows != H || rq.src_op < 0) return false;
    const wt_op& qs = b->ops[rq.src_op];
    if (qs.opcode != OP_SPLIT_F16 || qs.args[0] != ks.args[0] || qs.args[15] != 0 || qs.args[10] != 3 || qs.args[11] != s0) return false;
    // the ring must be the one the geometry implies
    uint32_t si = state & 0x1FFFu;
    if ((state & 0xE000u) != WT_REF_STATE_FLAG || si >= g.n_states || !g.kv[si].ready || g.kv[si].nslots != nslots ||
        g.kv[si].slot_bytes != B * kvh * hd * 4u) return false;
    if (nh / kvh > 16 || (hd != 128 && hd != 64)) return false;
    // mask operand: a temp or slot of H*nslots elements laid out [H][nslots]
    for (uint32_t o : rq.ops) ops.push_back(o);
    for (uint32_t o : rk.ops) ops.push_back(o);
    ops.push_back((uint32_t)rq.src_op); ops.push_back((uint32_t)rk.src_op); ops.push_back((uint32_t)vsplit);
    ops.push_back(ia);
    for (uint32_t k = 0; k < 5; k++) ops.push_back(j + k);
    uint32_t first;
    if (!contiguous(ops, first)) return false;
    if (!closed(G, ops, {j + 4})) return false;
    sp.kind = 0; sp.first = first; sp.count = (uint32_t)ops.size(); sp.ops = ops;
    {
        const int lp = G.producer_of_arg[0][rk.src_op];
        sp.qkv_lin = -1;
        if (lp >= 0 && (uint32_t)lp + 1 == first && b->ops[lp].opcode == OP_MATMUL_W4A16 && b->ops[lp].args[2] == ks.args[0]) {
            bool only_chain = true;
            for (uint32_t u : G.users[lp]) only_chain = only_chain && std::binary_search(ops.begin(), ops.end(), u);
            if (only_chain) sp.qkv_lin = lp;
        }
    }
    sp.qkv = ks.args[0]; sp.cos_q = rq.cos_b; sp.sin_q = rq.sin_b; sp.cos_k = rk.cos_b; sp.sin_k = rk.sin_b;
    sp.q_out = b->ops[rq.out_op].args[2]; sp.mask = ad.args[1]; sp.ctx = pv.args[2]; sp.state = si;
    sp.B = B; sp.nh = nh; sp.kvh = kvh; sp.hd = hd; sp.nslots = nslots; sp.pos = ap.args[3];
    sp.scale = scale; sp.scale_div = bi.args[4] == 3;
    return true;
}

// Standalone rotary chain ending in the ADD at `add_op`.
bool match_rope_span(const Graph& G, uint32_t add_op, Span& sp) {
    Rope r = match_rope(G, (int)add_op);
    if (!r.ok || (r.hd & 3u)) return false;
    std::vector<uint32_t> ops = r.ops;
    uint32_t first;
    if (!contiguous(ops, first) || ops.back() != add_op || !closed(G, ops, {add_op})) return false;
    sp.kind = 3; sp.first = first; sp.count = (uint32_t)ops.size(); sp.ops = ops;
    sp.a_ref = r.x; sp.cos_q = r.cos_b; sp.sin_q = r.sin_b; sp.y = G.b->ops[add_op].args[2]; sp.M = r.rows; sp.hd = r.hd;
    return true;
}

// Prefill attention chain around the SOFTMAX at `ism`:
//   TRANSPOSE_GEN q [S,nh,hd]->[nh,S,hd], k [Sk,kvh,hd]->[kvh,hd,Sk], v [Sk,kvh,hd]->[kvh,Sk,hd],
//   MATMUL_F16 batched over kvh (rows = rep*S), BINARY scale by a broadcast constant, ADD mask,
//   SOFTMAX, MATMUL_F16 batched with V, TRANSPOSE_GEN [nh,S,hd]->[S,nh,hd].
bool match_prefill_attention(const Graph& G, uint32_t ism, Span& sp) {
    const wt_blob* b = G.b;
    if (ism < 3 || ism + 2 >= b->n_ops) return false;
    const uint32_t j = ism - 3;
    const wt_op &sc = b->ops[j], &bi = b->ops[j + 1], &ad = b->ops[j + 2], &sm = b->ops[j + 3], &pv = b->ops[j + 4], &ot = b->ops[j + 5];
    if (sc.opcode != OP_MATMUL_F16 || bi.opcode != OP_BINARY_F16 || ad.opcode != OP_ADD_F16 || sm.opcode != OP_SOFTMAX_F16 ||
        pv.opcode != OP_MATMUL_F16 || ot.opcode != OP_TRANSPOSE_GEN_F16) return false;
    if ((sc.args[6] & 7u) != 4u || (pv.args[6] & 7u) != 4u) return false;
    const uint32_t kvh = sc.args[6] >> 16, rows = sc.args[3], hd = sc.args[4], seq_k = sc.args[5];
    if (!kvh || (pv.args[6] >> 16) != kvh || pv.args[3] != rows || pv.args[4] != seq_k || pv.args[5] != hd) return false;
    if (hd != 128 && hd != 64) return false;
    const int tq = G.producer_of_arg[0][j], tk = G.producer_of_arg[1][j], tv = G.producer_of_arg[1][j + 4];
    if (tq < 0 || tk < 0 || tv < 0) return false;
    const wt_op &oq = b->ops[tq], &ok = b->ops[tk], &ov = b->ops[tv];
    auto tr = [](const wt_op& o, uint32_t d0, uint32_t d1, uint32_t d2, uint32_t perm) {
        return o.opcode == OP_TRANSPOSE_GEN_F16 && o.args[2] == 3 && o.args[3] == d0 && o.args[4] == d1 && o.args[5] == d2 &&
               (o.args[7] & 0xFFFFFFu) == perm;
    };
    if (oq.opcode != OP_TRANSPOSE_GEN_F16 || oq.args[2] != 3 || oq.args[5] != hd) return false;
    const uint32_t seq_q = oq.args[3], nh = oq.args[4];
    if (!seq_q || !nh || nh % kvh || (nh / kvh) * seq_q != rows) return false;
    if (!tr(oq, seq_q, nh, hd, 1u | 0u << 8 | 2u << 16) || !tr(ok, seq_k, kvh, hd, 1u | 2u << 8 | 0u << 16) ||
        !tr(ov, seq_k, kvh, hd, 1u | 0u << 8 | 2u << 16) || !tr(ot, nh, seq_q, hd, 1u | 0u << 8 | 2u << 16)) return false;
    const uint64_t n_sc = (uint64_t)nh * seq_q * seq_k;
    if (n_sc > 0xFFFFFFFFull) return false;
    if (bi.args[0] != sc.args[2] || (bi.args[4] != 2 && bi.args[4] != 3) || bi.args[3] != (uint32_t)n_sc) return false;
    if (ad.args[0] != bi.args[2] || ad.args[3] != (uint32_t)n_sc) return false;
    if (sm.args[0] != ad.args[2] || sm.args[2] != nh * seq_q || sm.args[3] != seq_k) return false;
    if (pv.args[0] != sm.args[1] || ot.args[0] != pv.args[2]) return false;
    float scale;
    if (!const_scalar(G, G.producer_of_arg[1][j + 1], scale)) return false;
    // the mask operand: a [nh][S][Sk] tensor, or the broadcast over heads of a constant [S][Sk] slot
    sp.mask_is_slot = false;
    const int mb = G.producer_of_arg[1][j + 2];
    if (mb >= 0 && b->ops[mb].opcode == OP_BROADCAST_F16) {
        const wt_op& bo = b->ops[mb];
        const uint32_t src = bo.args[0];
        if ((src & 0x8000u) && (src & 0x7FFFu) < b->n_slots) {
            const wt_slot& sl = b->slots[src & 0x7FFFu];
            // in dims (1,1,S,Sk) -> out dims (1,nh,S,Sk)
            if (sl.addr == 0 && sl.len == (uint64_t)seq_q * seq_k * 2u && bo.args[4] == 1 && bo.args[5] == 1 && bo.args[6] == seq_q &&
                bo.args[7] == seq_k && bo.args[8] == 1 && bo.args[9] == nh && bo.args[10] == seq_q && bo.args[11] == seq_k) {
                sp.mask_is_slot = true;
                sp.mask_slot = src & 0x7FFFu;
            }
        }
    }
    std::vector<uint32_t> ops = {(uint32_t)tq, (uint32_t)tk, (uint32_t)tv, j, j + 1, j + 2, j + 3, j + 4, j + 5};
    uint32_t first;
    if (!contiguous(ops, first) || !closed(G, ops, {j + 5})) return false;
    sp.kind = 4; sp.first = first; sp.count = (uint32_t)ops.size(); sp.ops = ops;
    sp.pq = oq.args[0]; sp.pk = ok.args[0]; sp.pv = ov.args[0]; sp.mask = ad.args[1]; sp.ctx = ot.args[1];
    sp.M = seq_q; sp.N = seq_k; sp.nh = nh; sp.kvh = kvh; sp.hd = hd; sp.scale = scale; sp.scale_div = bi.args[4] == 3;
    return true;
}

bool match_swiglu(const Graph& G, uint32_t ip, Span& sp) {
    const wt_blob* b = G.b;
    const wt_op& pr = b->ops[ip];
    if (pr.opcode != OP_BINARY_F16 || pr.args[4] != 2) return false;
    int act = G.producer_of_arg[0][ip], up = G.producer_of_arg[1][ip];
    if (act < 0 || up < 0 || b->ops[act].opcode != OP_BINARY_F16 || b->ops[act].args[4] != 2 || b->ops[up].opcode != OP_MATMUL_W4A16) return false;
    int gate = G.producer_of_arg[0][act], sig = G.producer_of_arg[1][act];
    if (gate < 0 || sig < 0 || b->ops[gate].opcode != OP_MATMUL_W4A16 || b->ops[sig].opcode != OP_UNARY_F16 || b->ops[sig].args[3] != 8) return false;
    if (G.producer_of_arg[0][sig] != gate) return false;
    const wt_op &gt = b->ops[gate], &u = b->ops[up];
    if (gt.args[0] != u.args[0] || gt.args[3] != u.args[3] || gt.args[4] != u.args[4] || gt.args[5] != u.args[5]) return false;
    uint32_t M = gt.args[3], n = M * gt.args[5];
    if (M > 64 || M >= w4_gemm_min_rows() || pr.args[3] != n || b->ops[act].args[3] != n || b->ops[sig].args[2] != n) return false;
    std::vector<uint32_t> ops = {(uint32_t)gate, (uint32_t)sig, (uint32_t)act, (uint32_t)up, ip};
    uint32_t first;
    if (!contiguous(ops, first) || !closed(G, ops, {ip})) return false;
    sp.kind = 1; sp.first = first; sp.count = 5; sp.ops = ops;
    sp.a_ref = gt.args[0]; sp.wg = gt.args[1]; sp.wu = u.args[1]; sp.y = pr.args[2];
    sp.M = M; sp.K = gt.args[4]; sp.N = gt.args[5];
    return true;
}

// SPLIT(qkv, 0) -> rotary chain, SPLIT(qkv, 1) -> rotary chain, SPLIT(qkv, 2): the 17 consecutive
// ops between the q|k|v projection and the attention chain of a prefill block. `i` is the first SPLIT.
bool match_qkv_split_rope(const Graph& G, const std::vector<PlanOp>& meas, uint32_t i, Span& sp) {
    const wt_blob* b = G.b;
    if (i + 17 > b->n_ops) return false;
    const wt_op &s0 = b->ops[i], &s1 = b->ops[i + 8], &s2 = b->ops[i + 16];
    auto split_ok = [&](const wt_op& s, uint32_t idx) {
        return s.opcode == OP_SPLIT_F16 && s.args[0] == s0.args[0] && s.args[10] == 3 && s.args[15] == idx &&
               s.args[11] == s0.args[11] && s.args[12] == s0.args[12] && s.args[13] == s0.args[13];
    };
    if (!split_ok(s0, 0) || !split_ok(s1, 1) || !split_ok(s2, 2) || !is_temp_ref(s0.args[0])) return false;
    Rope ra = match_rope(G, (int)i + 7), rb = match_rope(G, (int)i + 15);
    if (!ra.ok || !rb.ok || ra.hd != rb.hd || (ra.hd & 3u)) return false;
    const uint32_t hd = ra.hd, wq = s0.args[11], wk = s0.args[12];
    if (s0.args[13] != wk || wq % hd || wk % hd || !wk || !wq) return false;
    if (ra.x != s0.args[1] || rb.x != s1.args[1] || ra.src_op != (int)i || rb.src_op != (int)i + 8) return false;
    if (meas[i].out_bytes[0] % (wq * 2u)) return false;
    const uint32_t tokens = meas[i].out_bytes[0] / (wq * 2u);
    if (!tokens || ra.rows != tokens * (wq / hd) || rb.rows != tokens * (wk / hd) ||
        meas[i + 8].out_bytes[0] != tokens * wk * 2u || meas[i + 16].out_bytes[0] != tokens * wk * 2u) return false;
    std::vector<uint32_t> ops = {i, i + 8, i + 16};
    ops.insert(ops.end(), ra.ops.begin(), ra.ops.end());
    ops.insert(ops.end(), rb.ops.begin(), rb.ops.end());
    uint32_t first;
    if (!contiguous(ops, first) || ops.size() != 17 || first != i || !closed(G, ops, {i + 7, i + 15, i + 16})) return false;
    sp.kind = 5; sp.first = i; sp.count = 17; sp.ops = ops; sp.keep = {i + 7, i + 15};
    sp.qkv = s0.args[0]; sp.cos_q = ra.cos_b; sp.sin_q = ra.sin_b; sp.cos_k = rb.cos_b; sp.sin_k = rb.sin_b;
    sp.q_out = b->ops[i + 7].args[2]; sp.k_out = b->ops[i + 15].args[2]; sp.v_out = s2.args[1];
    sp.B = tokens; sp.nh = wq / hd; sp.kvh = wk / hd; sp.hd = hd;
    return true;
}

// The SwiGLU chain of match_swiglu with more rows than the fused GEMV form takes: the two
// projections keep their own launches (GEMMs) and the three elementwise ops become one kernel.
bool match_swiglu_tail(const Graph& G, uint32_t ip, Span& sp) {
    const wt_blob* b = G.b;
    const wt_op& pr = b->ops[ip];
    if (pr.opcode != OP_BINARY_F16 || pr.args[4] != 2) return false;
    int act = G.producer_of_arg[0][ip], up = G.producer_of_arg[1][ip];
    if (act < 0 || up < 0 || b->ops[act].opcode != OP_BINARY_F16 || b->ops[act].args[4] != 2 || b->ops[up].opcode != OP_MATMUL_W4A16) return false;
    int gate = G.producer_of_arg[0][act], sig = G.producer_of_arg[1][act];
    if (gate < 0 || sig < 0 || b->ops[gate].opcode != OP_MATMUL_W4A16 || b->ops[sig].opcode != OP_UNARY_F16 || b->ops[sig].args[3] != 8) return false;
    if (G.producer_of_arg[0][sig] != gate) return false;
    const wt_op &gt = b->ops[gate], &u = b->ops[up];
    if (gt.args[3] != u.args[3] || gt.args[5] != u.args[5]) return false;
    const uint64_t n64 = (uint64_t)gt.args[3] * gt.args[5];
    const uint32_t n = (uint32_t)n64;
    if (n64 > 0xFFFFFFFFull || (gt.args[3] <= 64 && gt.args[3] < w4_gemm_min_rows()) || pr.args[3] != n || b->ops[act].args[3] != n || b->ops[sig].args[2] != n) return false;
    if (!is_temp_ref(gt.args[2]) || !is_temp_ref(u.args[2]) || !is_temp_ref(pr.args[2])) return false;
    std::vector<uint32_t> ops = {(uint32_t)gate, (uint32_t)sig, (uint32_t)act, (uint32_t)up, ip};
    uint32_t first;
    if (!contiguous(ops, first) || !closed(G, ops, {ip})) return false;
    sp.kind = 6; sp.first = first; sp.count = 5; sp.ops = ops; sp.keep = {(uint32_t)gate, (uint32_t)up};
    sp.gate_op = (uint32_t)gate; sp.up_op = (uint32_t)up; sp.gate_t = gt.args[2]; sp.up_t = u.args[2];
    sp.a_ref = gt.args[0]; sp.y = pr.args[2]; sp.n = n;
    // one input and one K: the pair can also run as the gate | up GEMM
    sp.M = gt.args[3]; sp.N = gt.args[5]; sp.K = (gt.args[0] == u.args[0] && gt.args[4] == u.args[4]) ? gt.args[4] : 0;
    sp.wg = gt.args[1]; sp.wu = u.args[1];
    return true;
}

// TRANSPOSE_GEN of a [heads][rows][d] tensor to [rows][heads * d] whose only reader is the W4A16 GEMM right behind it
// (the output of a per-head kernel on its way into a projection): the GEMM reads the untransposed tensor through a
// three-dimensional tensor map. `i` is the transposition.
bool match_transpose_gemm(const Graph& G, uint32_t i, Span& sp) {
    const wt_blob* b = G.b;
    if (i + 1 >= b->n_ops) return false;
    const wt_op &tr = b->ops[i], &mm = b->ops[i + 1];
    if (tr.opcode != OP_TRANSPOSE_GEN_F16 || mm.opcode != OP_MATMUL_W4A16) return false;
    if (tr.args[2] != 3 || (tr.args[7] & 0xFFFFFFu) != (1u | 0u << 8 | 2u << 16)) return false;
    const uint32_t heads = tr.args[3], rows = tr.args[4], d = tr.args[5];
    if (!heads || !rows || !d || d % 64u || rows < w4_gemm_min_rows()) return false;
    if (!is_temp_ref(tr.args[1]) || mm.args[0] != tr.args[1] || mm.args[3] != rows || mm.args[4] != heads * d || mm.args[5] % 128u) return false;
    std::vector<uint32_t> ops = {i, i + 1};
    if (!closed(G, ops, {i + 1})) return false;
    sp.kind = 7; sp.first = i; sp.count = 2; sp.ops = ops; sp.keep = {i};
    sp.a_ref = tr.args[0]; sp.M = rows; sp.K = heads * d; sp.N = mm.args[5]; sp.hd = d;
    return true;
}

// Greedy sampling of a batch as the op list spells it: for every row r of the logits [rows][n] a SLICE of that row and
// an ARGMAX of the slice, the int32 results joined in row order by a tree of CONCAT ops (up to four inputs each).
// `root` is the CONCAT at the top of such a tree. One launch finds all the maxima and writes them where the root's
// output lies.
bool match_argmax_rows(const Graph& G, uint32_t root, Span& sp) {
    const wt_blob* b = G.b;
    std::vector<uint32_t> ops, leaves;
    // depth-first, inputs in order: the leaves come out in the order their values lie in the root's output
    std::vector<std::pair<uint32_t, uint32_t>> stack;     // (concat op, next input)
    if (b->ops[root].opcode != OP_CONCAT_F16) return false;
    stack.push_back({root, 0});
    std::vector<uint32_t> width(b->n_ops, 0);              // fp16 units an op contributes
    while (!stack.empty()) {
        const uint32_t c = stack.back().first, k = stack.back().second;
        const wt_op& co = b->ops[c];
        const uint32_t n_seg = co.args[10];
        if (n_seg < 1 || n_seg > 4 || ops.size() > 4096) return false;
        if (k == n_seg) {
            uint32_t total = 0;
            for (uint32_t s = 0; s < n_seg; s++) total += co.args[12 + s];
            if (co.args[11] != total || total != width[c]) return false;      // one outer row, sizes add up to what came in
            ops.push_back(c);
            stack.pop_back();
            if (!stack.empty()) width[stack.back().first] += total;
            continue;
        }
        stack.back().second++;
        const int p = G.producer_of_arg[k][c];
        if (p < 0) return false;
        if (b->ops[p].opcode == OP_CONCAT_F16) {
            if (co.args[12 + k] == 0) return false;
            stack.push_back({(uint32_t)p, 0});
        } else if (b->ops[p].opcode == OP_ARGMAX_F16) {
            if (co.args[12 + k] != 2) return false;                            // an int32 = two fp16-sized units
            leaves.push_back((uint32_t)p);
            ops.push_back((uint32_t)p);
            width[c] += 2;
        } else {
            return false;
        }
    }
    if (leaves.size() < 2 || leaves.size() > kArgmaxMaxRows) return false;
    uint32_t src = 0, n = 0;
    for (size_t r = 0; r < leaves.size(); r++) {
        const wt_op& am = b->ops[leaves[r]];
        const int sl = G.producer_of_arg[0][leaves[r]];
        if (sl < 0 || b->ops[sl].opcode != OP_STRIDED_SLICE_F16) return false;
        const wt_op& s = b->ops[sl];
        if (r == 0) { src = s.args[0]; n = am.args[2]; }
        // rank 2, rows [r, r+1) x columns [0, n) of a [rows][n] tensor, unit strides
        if (s.args[0] != src || am.args[2] != n || s.args[2] != n || s.args[3] != 2 || s.args[4] != r || s.args[5] != 0 ||
            s.args[7] != r + 1 || s.args[8] != n || s.args[10] > 1 || s.args[11] > 1 || s.args[13] < leaves.size() || s.args[14] != n)
            return false;
        ops.push_back((uint32_t)sl);
    }
    uint32_t first;
    if (!contiguous(ops, first) || !closed(G, ops, {root})) return false;
    sp.kind = 8; sp.first = first; sp.count = (uint32_t)ops.size(); sp.ops = ops;
    sp.a_ref = src; sp.y = b->ops[root].args[8]; sp.M = (uint32_t)leaves.size(); sp.N = n;
    return true;
}

bool match_add_norm(const Graph& G, uint32_t i, Span& sp) {
    const wt_blob* b = G.b;
    if (i + 1 >= b->n_ops) return false;
    const wt_op &ad = b->ops[i], &nm = b->ops[i + 1];
    if (ad.opcode != OP_ADD_F16 || nm.opcode != OP_RMSNORM2_F16) return false;
    if (nm.args[0] != ad.args[2] || nm.args[4] != ad.args[3] || !is_temp_ref(ad.args[2])) return false;
    sp.kind = 2; sp.first = i; sp.count = 2; sp.ops = {i, i + 1};
    sp.add_a = ad.args[0]; sp.add_b = ad.args[1]; sp.sum_t = ad.args[2];
    sp.gamma_s = nm.args[1] & 0x7FFFu; sp.beta_s = nm.args[2] & 0x7FFFu; sp.norm_y = nm.args[3]; sp.n = ad.args[3];
    return true;
}

std::vector<Span> g_spans;
float* g_attn_scratch = nullptr;
std::map<std::pair<uint32_t, uint64_t>, uint8_t*> g_skip_maps;   // (mask slot, S<<32|Sk) -> device tile-skip bitmap

const uint8_t* resolve(const wt_blob* b, uint32_t arg) {
    if (arg & 0x8000u) {
        uint32_t s = arg & 0x7FFFu;
        if (s >= b->n_slots) return nullptr;
        auto it = g.d_ext.find(s);
        if (it != g.d_ext.end()) return it->second;
        return g.d_weights + b->slots[s].offset;
    }
    if (!is_temp_ref(arg)) return nullptr;
    return g.temp_dev[arg];
}

}  // namespace

// Finds the chains. `internal[t]` is set for temp ids written only inside
// fused chains (and not among a chain's outputs): they need no memory.
void fuse_analyze(const wt_blob* b, const std::vector<PlanOp>& meas, std::vector<uint8_t>& internal, std::vector<uint8_t>& dead) {
    g_spans.clear();
    internal.assign(kMaxTemps, 0);
    dead.assign(b->n_ops, 0);
    Graph G;
    build_graph(b, meas, G);
    std::vector<uint8_t> taken(b->n_ops, 0);
    auto claim = [&](Span& sp) {
        for (uint32_t o : sp.ops) if (taken[o] || meas[o].rc) return false;
        // an op whose output is all-reduced over the ranks keeps its own launch (the reduction hangs on it)
        if (g.tp_world > 1)
            for (uint32_t o : sp.ops) if (o < g_allreduce_after.size() && g_allreduce_after[o]) return false;
        for (uint32_t o : sp.ops) taken[o] = 1;
        g_spans.push_back(sp);
        return true;
    };
    for (uint32_t i = 0; i < b->n_ops; i++) {
        Span sp{};
        if (b->ops[i].opcode == OP_KV_APPEND_F16 && match_attention(G, i, sp)) claim(sp);
    }
    for (uint32_t i = 0; i < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && b->ops[i].opcode == OP_SOFTMAX_F16 && match_prefill_attention(G, i, sp)) claim(sp);
    }
    for (uint32_t i = 0; i < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && b->ops[i].opcode == OP_SPLIT_F16 && match_qkv_split_rope(G, meas, i, sp)) claim(sp);
    }
    for (uint32_t i = 0; i < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && b->ops[i].opcode == OP_ADD_F16 && match_rope_span(G, i, sp)) claim(sp);
    }
    for (uint32_t i = 0; i < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && b->ops[i].opcode == OP_BINARY_F16 && (match_swiglu(G, i, sp) || match_swiglu_tail(G, i, sp))) claim(sp);
    }
    for (uint32_t i = 0; i + 1 < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && !taken[i + 1] && match_transpose_gemm(G, i, sp)) claim(sp);
    }
    for (uint32_t i = b->n_ops; i-- > 0;) {      // from the back: the root of a CONCAT tree comes after its branches
        Span sp{};
        if (!taken[i] && b->ops[i].opcode == OP_CONCAT_F16 && match_argmax_rows(G, i, sp)) claim(sp);
    }
    for (uint32_t i = 0; i + 1 < b->n_ops; i++) {
        Span sp{};
        if (!taken[i] && !taken[i + 1] && match_add_norm(G, i, sp)) claim(sp);
    }
    // temps written only by interior ops of chains
    std::vector<int> writes_in(kMaxTemps, 0), writes_out(kMaxTemps, 0);
    std::vector<uint8_t> interior(b->n_ops, 0);
    for (const Span& sp : g_spans) {
        if (sp.kind == 2) continue;
        for (uint32_t o : sp.ops) interior[o] = 1;
        interior[sp.ops.back()] = 0;                       // the chain's result
        if (sp.kind == 0)                                   // the rotated q is kept as the attention kernel's input
            for (uint32_t o : sp.ops)
                if (meas[o].out_id[0] == sp.q_out) interior[o] = 0;
        for (uint32_t o : sp.keep) interior[o] = 0;
    }
    for (uint32_t i = 0; i < b->n_ops; i++)
        for (int k = 0; k < 2; k++) {
            uint32_t id = meas[i].out_id[k];
            if (id == kNoOff) continue;
            (interior[i] ? writes_in : writes_out)[id]++;
        }
    for (uint32_t t = 0; t < kMaxTemps; t++) internal[t] = writes_in[t] > 0 && writes_out[t] == 0;

    // Ops outside the chains whose results only the replaced ops read (the broadcast of
    // the scale constant, a mask expanded over heads that the kernel takes unexpanded):
    // dead when every chain runs fused.
    std::vector<int> span_of(b->n_ops, -1);
    for (size_t si = 0; si < g_spans.size(); si++)
        for (uint32_t o : g_spans[si].ops) span_of[o] = (int)si;
    auto span_reads = [&](const Span& sp, uint32_t t) {
        switch (sp.kind) {
        case 0: return t == sp.qkv || t == sp.cos_q || t == sp.sin_q || t == sp.cos_k || t == sp.sin_k || t == sp.mask;
        case 1: return t == sp.a_ref;
        case 2: return t == sp.add_a || t == sp.add_b;
        case 3: return t == sp.a_ref || t == sp.cos_q || t == sp.sin_q;
        case 4: return t == sp.pq || t == sp.pk || t == sp.pv || (!sp.mask_is_slot && t == sp.mask);
        case 5: return t == sp.qkv || t == sp.cos_q || t == sp.sin_q || t == sp.cos_k || t == sp.sin_k;
        case 6: return t == sp.a_ref;
        case 7: return t == sp.a_ref;
        case 8: return t == sp.a_ref;
        }
        return true;
    };
    for (uint32_t i = 0; i < b->n_ops; i++) {
        if (span_of[i] >= 0 || G.users[i].empty() || meas[i].rc) continue;
        const uint32_t opc = b->ops[i].opcode;
        if (opc != OP_BROADCAST_F16) continue;          // pure functions of their inputs only
        const uint32_t t = meas[i].out_id[0];
        if (t == kNoOff || meas[i].out_id[1] != kNoOff) continue;
        bool all_dead = true;
        for (uint32_t u : G.users[i])
            if (span_of[u] < 0 || span_reads(g_spans[span_of[u]], t)) { all_dead = false; break; }
        if (all_dead) dead[i] = 1;
    }
}

// Bakes the fused launches into the plan (after addresses are known).
void fuse_materialize(const wt_blob* b) {
    size_t scratch_floats = 0;
    for (const Span& sp : g_spans)
        if (sp.kind == 0) {
            uint32_t ns = attn_decode_nsplit(sp.B * sp.kvh, sp.nslots, sp.nh / sp.kvh, sp.hd, 0);
            size_t f = attn_decode_scratch_floats(sp.B * sp.kvh, sp.nh / sp.kvh, sp.hd, ns);
            if (f > scratch_floats) scratch_floats = f;
        }
    if (scratch_floats) {
        if (cudaMalloc(&g_attn_scratch, scratch_floats * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return; }
    }
    g.fused_ops = 0;
    for (const Span& sp : g_spans) {
        PlanOp& head = g.plan[sp.first];
        if (sp.kind == 0) {
            const uint16_t* qkv = (const uint16_t*)resolve(b, sp.qkv);
            const uint16_t *cq = (const uint16_t*)resolve(b, sp.cos_q), *sq = (const uint16_t*)resolve(b, sp.sin_q);
            const uint16_t *ck = (const uint16_t*)resolve(b, sp.cos_k), *sk = (const uint16_t*)resolve(b, sp.sin_k);
            uint16_t* q_out = (uint16_t*)resolve(b, sp.q_out);
            const uint16_t* mask = (const uint16_t*)resolve(b, sp.mask);
            uint16_t* ctx = (uint16_t*)resolve(b, sp.ctx);
            if (!qkv || !cq || !sq || !ck || !sk || !q_out || !mask || !ctx) continue;
            uint32_t si = sp.state;
            uint16_t* ring = (uint16_t*)g.st_buf[si];
            uint32_t* posmap = g.kv[si].posmap;
            uint32_t* ctr = g.d_st_count + si;
            uint32_t B = sp.B, nh = sp.nh, kvh = sp.kvh, hd = sp.hd, nslots = sp.nslots, pos = sp.pos;
            AttnDecodeArgs a{};
            a.status = g.d_status;
            a.q = q_out; a.ring = ring; a.counter = ctr; a.n_kv = 0; a.n_kv_add = 1; a.bump_counter = ctr;
            a.mask = mask; a.mask_seq_stride = nh * nslots; a.kvh_per_seq = kvh;
            a.scale = sp.scale; a.scale_div = sp.scale_div; a.rep = nh / kvh; a.kv_heads = B * kvh; a.nslots = nslots;
            a.nsplit = attn_decode_nsplit(B * kvh, nslots, nh / kvh, hd, 0);
            a.part_o = g_attn_scratch;
            a.part_ml = g_attn_scratch + (size_t)B * kvh * a.nsplit * a.rep * hd;
            head.fused = [=](cudaStream_t st) {
                k_rope_kv_append(st, qkv, cq, sq, ck, sk, q_out, ring, posmap, ctr, B, nh, kvh, hd, nslots, pos);
                k_attn_decode(st, a, hd, ctx, B * kvh);
            };
            // The q|k|v projection right before the chain takes the rotary embedding and the append into
            // its epilogue (one launch less per layer); the projection op becomes the head of the span.
            if (sp.qkv_lin >= 0 && hd == 128 && B <= 8) {
                PlanOp& lin = g.plan[sp.qkv_lin];
                const wt_op& lo = b->ops[sp.qkv_lin];
                const uint32_t K = lo.args[4], N = lo.args[5];
                const bool reduced = g.tp_world > 1 && (uint32_t)sp.qkv_lin < g_allreduce_after.size() && g_allreduce_after[sp.qkv_lin];
                uint64_t key = (uint64_t)(lo.args[1] & 0x7FFFu) | ((uint64_t)K << 16) | ((uint64_t)N << 40);
                auto it = g.w4.find(key);
                const uint16_t* act = (const uint16_t*)resolve(b, lo.args[0]);
                if (it != g.w4.end() && act && !lin.fused && !lin.rc && lin.launch && !lin.uses_internal && !reduced &&
                    lo.args[3] == B && N == (nh + 2 * kvh) * hd && K % 512 == 0 && K / 512 <= 10 &&
                    N / 32 >= 148) {     // one CTA per pair of strips: worth it only while every SM still gets one
                    W4Epilogue ep;
                    ep.mode = 2;
                    ep.cos_q = cq; ep.sin_q = sq; ep.cos_k = ck; ep.sin_k = sk; ep.q_out = q_out; ep.ring = ring;
                    ep.posmap = posmap; ep.counter = ctr; ep.nh = nh; ep.kvh = kvh; ep.nslots = nslots; ep.pos_const = pos;
                    const uint32_t* pk = it->second.packed;
                    const uint16_t* sc = it->second.scales;
                    lin.fused = [=](cudaStream_t st) {
                        k_w4a16_skinny_qkv_rope(st, act, pk, sc, B, K, N, ep);
                        k_attn_decode(st, a, hd, ctx, B * kvh);
                    };
                    lin.span = 1 + sp.count;
                    g.fused_ops += 1;
                }
            }
        } else if (sp.kind == 1) {
            const uint16_t* act = (const uint16_t*)resolve(b, sp.a_ref);
            uint16_t* y = (uint16_t*)resolve(b, sp.y);
            auto find = [&](uint32_t wref) -> const W4Packed* {
                uint64_t key = (uint64_t)(wref & 0x7FFFu) | ((uint64_t)sp.K << 16) | ((uint64_t)sp.N << 40);
                auto it = g.w4.find(key);
                return it == g.w4.end() ? nullptr : &it->second;
            };
            const W4Packed *wg = find(sp.wg), *wu = find(sp.wu);
            if (!act || !y || !wg || !wu) continue;
            const uint32_t *pg = wg->packed, *pu = wu->packed;
            const uint16_t *sg = wg->scales, *su = wu->scales;
            uint32_t M = sp.M, K = sp.K, N = sp.N;
            head.fused = [=](cudaStream_t st) { k_w4a16_skinny_swiglu(st, act, pg, sg, pu, su, y, M, K, N); };
        } else if (sp.kind == 3) {
            const uint16_t *x = (const uint16_t*)resolve(b, sp.a_ref), *ct = (const uint16_t*)resolve(b, sp.cos_q),
                           *stb = (const uint16_t*)resolve(b, sp.sin_q);
            uint16_t* y = (uint16_t*)resolve(b, sp.y);
            if (!x || !ct || !stb || !y || ((((uintptr_t)x) | ((uintptr_t)ct) | ((uintptr_t)stb) | ((uintptr_t)y)) & 3u)) continue;
            uint32_t rows = sp.M, hd = sp.hd;
            head.fused = [=](cudaStream_t st) { k_rope(st, x, ct, stb, y, rows, hd); };
        } else if (sp.kind == 5) {
            const uint16_t* qkv = (const uint16_t*)resolve(b, sp.qkv);
            const uint16_t *cq = (const uint16_t*)resolve(b, sp.cos_q), *sq = (const uint16_t*)resolve(b, sp.sin_q);
            const uint16_t *ck = (const uint16_t*)resolve(b, sp.cos_k), *sk = (const uint16_t*)resolve(b, sp.sin_k);
            uint16_t *qo = (uint16_t*)resolve(b, sp.q_out), *ko = (uint16_t*)resolve(b, sp.k_out), *vo = (uint16_t*)resolve(b, sp.v_out);
            if (!qkv || !cq || !sq || !ck || !sk || !qo || !ko || !vo) continue;
            if ((((uintptr_t)qkv) | ((uintptr_t)cq) | ((uintptr_t)sq) | ((uintptr_t)ck) | ((uintptr_t)sk) | ((uintptr_t)qo) |
                 ((uintptr_t)ko) | ((uintptr_t)vo)) & 3u) continue;
            uint32_t tokens = sp.B, nh = sp.nh, kvh = sp.kvh, hd = sp.hd;
            head.fused = [=](cudaStream_t st) { k_qkv_split_rope(st, qkv, cq, sq, ck, sk, qo, ko, vo, tokens, nh, kvh, hd); };
        } else if (sp.kind == 8) {
            const uint16_t* x = (const uint16_t*)resolve(b, sp.a_ref);
            int32_t* y = (int32_t*)resolve(b, sp.y);
            if (!x || !y || (((uintptr_t)y) & 3u)) continue;
            const uint32_t rows = sp.M, n = sp.N;
            // the ops of the tree, in list order, for the case that the one launch is refused
            std::vector<std::function<void(cudaStream_t)>> each;
            bool whole = true;
            for (uint32_t o : sp.ops) {
                if (g.plan[o].rc || !g.plan[o].launch || g.plan[o].uses_internal) { whole = false; break; }
                each.push_back(g.plan[o].launch);
            }
            head.fused = [=](cudaStream_t st) {
                if (k_argmax_rows(st, x, y, rows, n)) return;
                if (whole) for (const auto& f : each) f(st);
            };
        } else if (sp.kind == 7) {
            const PlanOp &tr = g.plan[sp.first], &mm = g.plan[sp.first + 1];
            const uint16_t* src = (const uint16_t*)resolve(b, sp.a_ref);
            if (!tr.launch || !mm.launch || !mm.launch_w4_gemm || tr.rc || mm.rc || !src || (((uintptr_t)src) & 15u) || g.exact_ops) continue;
            auto transpose = tr.launch, plain = mm.launch;
            auto gemm = mm.launch_w4_gemm;
            const uint32_t d = sp.hd;
            unsigned int* status = g.d_status;
            head.fused = [=](cudaStream_t st) {
                W4Epilogue ep;
                ep.status = status;
                if (gemm(st, ep, src, d)) return;
                transpose(st);
                plain(st);
            };
        } else if (sp.kind == 6) {
            const PlanOp &pg = g.plan[sp.gate_op], &pu = g.plan[sp.up_op];
            const uint16_t *gt = (const uint16_t*)resolve(b, sp.gate_t), *up = (const uint16_t*)resolve(b, sp.up_t);
            uint16_t* y = (uint16_t*)resolve(b, sp.y);
            if (!pg.launch || !pu.launch || pg.rc || pu.rc || !gt || !up || !y) continue;
            if ((((uintptr_t)gt) | ((uintptr_t)up) | ((uintptr_t)y)) & 15u) continue;
            auto lg = pg.launch, lu = pu.launch;
            size_t n = sp.n;
            // both projections and the elementwise tail on one tcgen05 kernel when they share input and shape
            const uint16_t* act = sp.K ? (const uint16_t*)resolve(b, sp.a_ref) : nullptr;
            auto find = [&](uint32_t wref) -> const W4Packed* {
                uint64_t key = (uint64_t)(wref & 0x7FFFu) | ((uint64_t)sp.K << 16) | ((uint64_t)sp.N << 40);
                auto it = g.w4.find(key);
                return it == g.w4.end() ? nullptr : &it->second;
            };
            const W4Packed *wg = act ? find(sp.wg) : nullptr, *wu = act ? find(sp.wu) : nullptr;
            if (wg && wu && !g.exact_ops && w4a16_gemm_sm100_swiglu_takes(sp.M, sp.K, sp.N) && !(((uintptr_t)act) & 15u)) {
                const uint32_t *qg = wg->packed, *qu = wu->packed;
                const uint16_t *sg = wg->scales, *su = wu->scales;
                const uint32_t M = sp.M, K = sp.K, N = sp.N;
                unsigned int* status = g.d_status;
                head.fused = [=](cudaStream_t st) {
                    if (k_w4a16_gemm_sm100_swiglu(st, act, qg, sg, qu, su, y, M, K, N, status)) return;
                    lg(st); lu(st); k_swiglu_tail(st, gt, up, y, n);
                };
            } else {
                head.fused = [=](cudaStream_t st) { lg(st); lu(st); k_swiglu_tail(st, gt, up, y, n); };
            }
        } else if (sp.kind == 4) {
            const uint16_t *q = (const uint16_t*)resolve(b, sp.pq), *k = (const uint16_t*)resolve(b, sp.pk),
                           *v = (const uint16_t*)resolve(b, sp.pv);
            uint16_t* out = (uint16_t*)resolve(b, sp.ctx);
            const uint16_t* mask = (const uint16_t*)resolve(b, sp.mask_is_slot ? (0x8000u | sp.mask_slot) : sp.mask);
            if (!q || !k || !v || !out || !mask) continue;
            uint32_t sq = sp.M, sk = sp.N, nh = sp.nh, kvh = sp.kvh, hd = sp.hd;
            size_t mstride = sp.mask_is_slot ? 0 : (size_t)sq * sk;
            const uint8_t *skip = nullptr, *zero = nullptr;
            if (sp.mask_is_slot) {
                // tiles of the constant mask that are -inf everywhere are never computed
                const uint32_t T = attn_prefill_tile(), nq = (sq + T - 1) / T, nk = (sk + T - 1) / T;
                auto key = std::make_pair(sp.mask_slot, (uint64_t)sq << 32 | sk);
                auto it = g_skip_maps.find(key);
                if (it == g_skip_maps.end()) {
                    const uint16_t* hm = (const uint16_t*)(b->weight_base + b->slots[sp.mask_slot].offset);
                    // first nq * nk bytes: 1 = the tile is -inf everywhere; next nq * nk bytes: 1 = +0 everywhere
                    std::vector<uint8_t> bm((size_t)2 * nq * nk, 1);
                    for (uint32_t r = 0; r < sq; r++)
                        for (uint32_t c = 0; c < sk; c++) {
                            const uint16_t mv = hm[(size_t)r * sk + c];
                            if (mv != 0xFC00u) bm[(size_t)(r / T) * nk + c / T] = 0;
                            if (mv != 0x0000u) bm[(size_t)nq * nk + (size_t)(r / T) * nk + c / T] = 0;
                        }
                    uint8_t* d = nullptr;
                    if (cudaMalloc(&d, bm.size()) == cudaSuccess) {
                        cudaMemcpyAsync(d, bm.data(), bm.size(), cudaMemcpyHostToDevice, g.stream);
                        cudaStreamSynchronize(g.stream);
                        it = g_skip_maps.emplace(key, d).first;
                    } else cudaGetLastError();
                }
                if (it != g_skip_maps.end()) { skip = it->second; zero = skip + (size_t)nq * nk; }
            }
            float scale = sp.scale; int sdiv = sp.scale_div;
            if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v)) & 15u) continue;
            unsigned int* status = g.d_status;
            static const int sm100_on = [] { const char* e = std::getenv("GEHTP_CUDA_PREFILL_SM100"); return e ? std::atoi(e) : 1; }();
            head.fused = [=](cudaStream_t st) {
                // head_dim 128: tcgen05 / TMEM form; anything it does not take goes to the mma.sync form
                if (sm100_on && k_attn_prefill_sm100(st, q, k, v, mask, mstride, skip, zero, scale, sdiv, sq, sk, nh, kvh, hd, out, status)) return;
                k_attn_prefill(st, q, k, v, mask, mstride, skip, scale, sdiv, sq, sk, nh, kvh, hd, out);
            };
        } else {
            const uint16_t *aa = (const uint16_t*)resolve(b, sp.add_a), *ab = (const uint16_t*)resolve(b, sp.add_b);
            uint16_t *sum = (uint16_t*)resolve(b, sp.sum_t), *y = (uint16_t*)resolve(b, sp.norm_y);
            const uint16_t* gam = (const uint16_t*)resolve(b, 0x8000u | sp.gamma_s);
            const uint16_t* bet = (const uint16_t*)resolve(b, 0x8000u | sp.beta_s);
            if (!aa || !ab || !sum || !y || !gam) continue;
            uint32_t rw = b->slots[sp.gamma_s].len / 2u;
            if (!rw || sp.n % rw) continue;
            uint32_t rows = sp.n / rw;
            head.fused = [=](cudaStream_t st) { k_add_rmsnorm(st, aa, ab, gam, bet, sum, y, rows, rw); };
            // One GPU: when the addend is the output of the W4A16 GEMM right before the ADD, the three ops run as the
            // GEMM with the add and the norm in its epilogue (with K split into runs: in the kernel that adds the runs).
            if (g.tp_world <= 1 && sp.first > 0 && !g.exact_ops && rw > 512) {
                PlanOp& lin = g.plan[sp.first - 1];
                const bool b_is_out = is_temp_ref(sp.add_b) && lin.out_id[0] == sp.add_b;
                const bool a_is_out = is_temp_ref(sp.add_a) && lin.out_id[0] == sp.add_a;
                if (lin.launch_w4_gemm && lin.launch && !lin.fused && !lin.rc && !lin.uses_internal && (a_is_out != b_is_out) &&
                    lin.out_bytes[0] == sp.n * 2u && lin.w4_m == rows && sum && gam) {
                    auto gemm = lin.launch_w4_gemm;
                    auto plain = lin.launch;
                    const uint16_t* res = b_is_out ? aa : ab;
                    unsigned int* status = g.d_status;
                    lin.fused = [=](cudaStream_t st) {
                        W4Epilogue ep;
                        ep.mode = 3; ep.status = status; ep.res = res; ep.gamma = gam; ep.beta = bet; ep.sum_out = sum; ep.norm_out = y;
                        if (gemm(st, ep, nullptr, 0)) return;
                        plain(st);
                        k_add_rmsnorm(st, aa, ab, gam, bet, sum, y, rows, rw);
                    };
                    lin.span = 3;
                    g.fused_ops += 1;
                }
            }
            // Tensor parallel: when the addend is the partial sum of the row-parallel
            // projection right before the ADD, projection + all-reduce + add + norm run
            // as two launches: the projection, then one kernel that exchanges the rows
            // with the peers, adds them and normalises.
            if (g.tp_world > 1 && tp_p2p_ready() && sp.first > 0) {
                PlanOp& lin = g.plan[sp.first - 1];
                const bool b_is_partial = is_temp_ref(sp.add_b) && lin.out_id[0] == sp.add_b;
                const bool a_is_partial = is_temp_ref(sp.add_a) && lin.out_id[0] == sp.add_a;
                if (lin.launch_local && !lin.fused && !lin.rc && !lin.uses_internal && (a_is_partial != b_is_partial) &&
                    lin.out_bytes[0] == sp.n * 2u) {
                    auto local = lin.launch_local;
                    const uint16_t* res = b_is_partial ? aa : ab;
                    uint16_t* part = (uint16_t*)(b_is_partial ? ab : aa);
                    lin.fused = [=](cudaStream_t st) {
                        local(st);
                        if (!tp_p2p_add_rmsnorm(st, res, part, gam, bet, sum, y, rows, rw)) {
                            tp_allreduce_f16(st, part, (size_t)rows * rw);
                            k_add_rmsnorm(st, aa, ab, gam, bet, sum, y, rows, rw);
                        }
                    };
                    lin.span = 3;
                    g.fused_ops += 1;
                }
            }
        }
        head.span = sp.count;
        g.fused_ops += sp.count;
    }
}

// Constant results. Compiled runlists slice, transpose and broadcast tables that live in weight slots (rotary tables,
// masks, per-chunk windows of a constant tensor) with one op per ONNX node; such an op gives the same bytes on every
// run. It is marked when: it only moves data; every tensor it reads is a weight slot with data in the blob or the
// result of a marked op; it is the only writer of its output temp; that temp's memory overlaps no other temp's; and the
// runlist has none of the memory-planner ops (SPILL, FILL, DMA: they write slots and parts of temps) and no static
// temp table (aliased temps). The first eager run that reaches a marked op executes it, later runs - and the
// captured graph - skip it.
void fold_constants(const wt_blob* b, uint8_t* const* addr, const uint64_t* maxb) {
    g.const_ops = 0;
    for (uint32_t i = 0; i < b->n_ops; i++) {
        const uint32_t oc = b->ops[i].opcode;
        if (oc == OP_SPILL || oc == OP_FILL || oc == OP_DMA) return;
    }
    for (uint32_t s = 0; s < b->n_slots; s++)
        if (b->slots[s].addr == WT_SLOT_TEMPOFF) return;
    std::vector<int> writers(kMaxTemps, 0);
    std::vector<uint8_t> in_span(b->n_ops, 0), const_temp(kMaxTemps, 0);
    for (uint32_t i = 0; i < b->n_ops; i++) {
        const PlanOp& p = g.plan[i];
        for (int k = 0; k < 2; k++)
            if (p.out_id[k] != kNoOff && p.out_id[k] < kMaxTemps) writers[p.out_id[k]]++;
        if (p.fused && p.span)
            for (uint32_t k = 0; k < p.span && i + k < b->n_ops; k++) in_span[i + k] = 1;
    }
    auto plain_slot = [&](uint32_t s) {
        if (s >= b->n_slots || !b->slots[s].len) return false;
        const uint64_t a = b->slots[s].addr;
        return a != WT_SLOT_EXT_IN && a != WT_SLOT_EXT_OUT && a != WT_SLOT_TEMPOFF && a != WT_SLOT_EXT_WGT && a != WT_SLOT_STATE;
    };
    for (uint32_t i = 0; i < b->n_ops; i++) {
        PlanOp& p = g.plan[i];
        const wt_op& op = b->ops[i];
        if (p.rc || !p.launch || in_span[i] || p.uses_internal) continue;
        switch (op.opcode) {
        case OP_STRIDED_SLICE_F16: case OP_TRANSPOSE_GEN_F16: case OP_TRANSPOSE_F16: case OP_BROADCAST_F16: case OP_CONCAT_F16:
        case OP_SPLIT_F16: case OP_PAD_F16:
            break;
        default:
            continue;
        }
        int ia[8];
        const int n = input_args(op, ia);
        bool ok = n > 0;
        for (int k = 0; k < n && ok; k++) {
            const uint32_t a = op.args[ia[k]];
            if ((a & 0xC000u) == 0x8000u) ok = plain_slot(a & 0x7FFFu);
            else ok = is_temp_ref(a) && const_temp[a];
        }
        int outs = 0;
        for (int k = 0; k < 2 && ok; k++) {
            const uint32_t id = p.out_id[k];
            if (id == kNoOff) continue;
            outs++;
            if (id >= kMaxTemps || writers[id] != 1 || !addr[id] || !maxb[id]) { ok = false; break; }
            const uint8_t *lo = addr[id], *hi = lo + maxb[id];
            for (uint32_t t = 0; t < kMaxTemps && ok; t++)
                if (t != id && addr[t] && maxb[t] && addr[t] < hi && lo < addr[t] + maxb[t]) ok = false;
        }
        if (!ok || !outs) continue;
        p.const_fold = true;
        p.const_done = false;
        for (int k = 0; k < 2; k++)
            if (p.out_id[k] != kNoOff) const_temp[p.out_id[k]] = 1;
        g.const_ops++;
    }
}

bool fuse_all_materialized() {
    for (const Span& sp : g_spans)
        if (!g.plan[sp.first].fused || g.plan[sp.first].span != sp.count) return false;
    return true;
}

void fuse_release() {
    if (g_attn_scratch) { cudaFree(g_attn_scratch); g_attn_scratch = nullptr; }
    for (auto& kv : g_skip_maps) cudaFree(kv.second);
    g_skip_maps.clear();
    g_spans.clear();
}

}  // namespace gehtp
