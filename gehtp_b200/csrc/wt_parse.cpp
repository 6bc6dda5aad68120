// WTOP blob parser: header, slot table, op table, weight-area bounds.
// Same checks, in the same order, as the reference parser
// (kernels/src/runtime/oplist_parse.c:86-169), so a malformed blob is refused
// with the same WT_ERR_* code.
#include <cstring>
#include <initializer_list>
#include "wtop_format.h"

namespace {

struct OpInfo {
    int16_t arity;      // -1 = opcode does not exist
    uint16_t ref_mask;  // bit i set = args[i] may be a slot reference
};

constexpr uint16_t bits(std::initializer_list<int> idx) {
    uint16_t m = 0;
    for (int i : idx) m |= (uint16_t)(1u << i);
    return m;
}

// Which argument positions can carry a 0x8000|slot reference follows
// arg_is_slot (oplist_parse.c:51-84).
const OpInfo* op_info(uint16_t opcode) {
    static OpInfo tab[36];
    static bool init = false;
    if (!init) {
        for (auto& t : tab) t = {-1, 0};
        tab[OP_NOP] = {WT_ARITY_NOP, 0};
        tab[OP_MATMUL_W4A16] = {WT_ARITY_MATMUL, bits({0, 1})};
        tab[OP_RMSNORM_F16] = {WT_ARITY_RMSNORM, bits({1})};
        tab[OP_PIN] = {WT_ARITY_PIN, bits({0})};
        tab[OP_SILU_F16] = {WT_ARITY_SILU, 0};
        tab[OP_IM2COL] = {WT_ARITY_IM2COL, 0};
        tab[OP_CONV2D_F16] = {WT_ARITY_CONV2D_F16, bits({1, 2})};
        tab[OP_ADD_F16] = {WT_ARITY_ADD_F16, 0};
        tab[OP_SPILL] = {WT_ARITY_SPILL, bits({1})};
        tab[OP_FILL] = {WT_ARITY_FILL, bits({0})};
        tab[OP_TRANSPOSE_F16] = {WT_ARITY_TRANSPOSE_F16, 0};
        tab[OP_UNARY_F16] = {WT_ARITY_UNARY_F16, bits({0})};
        tab[OP_BINARY_F16] = {WT_ARITY_BINARY_F16, bits({0, 1})};
        tab[OP_SOFTMAX_F16] = {WT_ARITY_SOFTMAX_F16, bits({0})};
        tab[OP_CONCAT_F16] = {WT_ARITY_CONCAT_F16, bits({0, 1, 2, 3, 4, 5, 6, 7})};
        tab[OP_STRIDED_SLICE_F16] = {WT_ARITY_STRIDED_SLICE_F16, bits({0})};
        tab[OP_SPLIT_F16] = {WT_ARITY_SPLIT_F16, bits({0})};
        tab[OP_REDUCE_F16] = {WT_ARITY_REDUCE_F16, bits({0})};
        tab[OP_CUMSUM_F32] = {WT_ARITY_CUMSUM_F32, bits({0})};
        tab[OP_CONV1D_SSM_F16] = {WT_ARITY_CONV1D_SSM_F16, bits({0, 1})};
        tab[OP_GATHER_F16] = {WT_ARITY_GATHER_F16, bits({0, 1})};
        tab[OP_ARGMAX_F16] = {WT_ARITY_ARGMAX_F16, bits({0})};
        tab[OP_KV_APPEND_F16] = {WT_ARITY_KV_APPEND_F16, bits({0, 1, 2})};
        tab[OP_KV_GATHER_F16] = {WT_ARITY_KV_GATHER_F16, bits({0, 1})};
        tab[OP_MATMUL_F16] = {WT_ARITY_MATMUL_F16, bits({0, 1})};
        tab[OP_RMSNORM2_F16] = {WT_ARITY_RMSNORM2_F16, bits({1, 2})};
        tab[OP_BROADCAST_F16] = {WT_ARITY_BROADCAST_F16, bits({0})};
        tab[OP_TRANSPOSE_GEN_F16] = {WT_ARITY_TRANSPOSE_GEN_F16, bits({0})};
        tab[OP_SCATTER_ND_F16] = {WT_ARITY_SCATTER_ND_F16, bits({0, 1, 2})};
        tab[OP_CONV1D_SSM_STEP_F16] = {WT_ARITY_CONV1D_SSM_STEP_F16, bits({0, 1})};
        tab[OP_DELTA_CHUNK_F16] = {WT_ARITY_DELTA_CHUNK_F16, bits({0, 1, 2, 3, 4})};
        tab[OP_DMA] = {WT_ARITY_DMA, bits({0, 1})};
        tab[OP_PAD_F16] = {WT_ARITY_PAD_F16, bits({0})};
        tab[OP_MATMUL_F16_SPLIT] = {WT_ARITY_MATMUL_F16_SPLIT, bits({0, 1})};
        init = true;
    }
    if (opcode >= sizeof(tab) / sizeof(tab[0]) || tab[opcode].arity < 0) return nullptr;
    return &tab[opcode];
}

}  // namespace

extern "C" int wt_parse(const uint8_t* buf, size_t size, struct wt_blob* out) {
    if (!buf || !out || size < 16) return WT_ERR_SHORT;
    if (std::memcmp(buf, "WTOP", 4) != 0) return WT_ERR_MAGIC;
    out->ver = wt_rd_u16(buf + 4);
    const bool v2 = out->ver == WT_BLOB_VER_2;
    if (out->ver != WT_BLOB_VER && !v2) return WT_ERR_VER;
    if (wt_rd_u16(buf + 6) != WT_ENDIAN_CHK) return WT_ERR_ENDIAN;
    out->n_slots = wt_rd_u32(buf + 8);
    out->n_ops = wt_rd_u32(buf + 12);
    if (out->n_slots == 0 || out->n_slots > WT_MAX_SLOTS) return WT_ERR_NSLOTS;
    if (out->n_ops == 0 || out->n_ops > WT_MAX_OPS) return WT_ERR_NOPS;

    const size_t rec = v2 ? WT_SLOT_SIZE_V2 : WT_SLOT_SIZE;
    size_t pos = 16 + (size_t)out->n_slots * rec;
    if (size < pos) return WT_ERR_SLOTS_OVERRUN;
    for (uint32_t i = 0; i < out->n_slots; i++) {
        const uint8_t* r = buf + 16 + (size_t)i * rec;
        wt_slot& s = out->slots[i];
        s.len = wt_rd_u32(r);
        s.count = wt_rd_u32(r + 4);
        s.offset = wt_rd_u32(r + 8);
        if (v2) {
            s.offset |= (uint64_t)wt_rd_u32(r + 12) << 32;
            s.addr = wt_rd_u32(r + 16);
        } else {
            s.addr = wt_rd_u32(r + 12);
        }
        if (s.len == 0) return WT_ERR_WEIGHT_OVERRUN;
        if (s.offset % WT_WEIGHT_ALIGN) return WT_ERR_ALIGN;
        if (!v2 && s.offset + s.len > 0xFFFFFFFFull) return WT_ERR_WEIGHT_OVERRUN;
    }

    for (uint32_t i = 0; i < out->n_ops; i++) {
        if (size < pos + 4) return WT_ERR_OP_TRUNC;
        const uint16_t opcode = wt_rd_u16(buf + pos);
        const uint16_t n_args = wt_rd_u16(buf + pos + 2);
        const OpInfo* info = op_info(opcode);
        if (!info) return WT_ERR_OPCODE;
        if (n_args != (uint16_t)info->arity) return WT_ERR_ARITY;
        if (size < pos + 4 + (size_t)n_args * 4) return WT_ERR_OP_TRUNC;
        wt_op& op = out->ops[i];
        op.opcode = opcode;
        op.n_args = n_args;
        for (uint16_t a = 0; a < n_args; a++) op.args[a] = wt_rd_u32(buf + pos + 4 + (size_t)a * 4);
        pos += 4 + (size_t)n_args * 4;
    }

    // The reference rounds the op-table end up in 32 bits.
    const uint32_t p32 = (uint32_t)pos;
    out->weight_off = WT_WEIGHT_ALIGN * ((p32 + WT_WEIGHT_ALIGN - 1u) / WT_WEIGHT_ALIGN);
    if ((size_t)out->weight_off > size) return WT_ERR_WEIGHT_OVERRUN;
    out->weight_base = buf + out->weight_off;
    out->weight_bytes = size - out->weight_off;

    for (uint32_t i = 0; i < out->n_slots; i++) {
        const wt_slot& s = out->slots[i];
        if (s.addr == WT_SLOT_EXT_WGT) continue;  // offset is into the external weight file
        if (s.offset + s.len > out->weight_bytes) return WT_ERR_WEIGHT_OVERRUN;
    }
    for (uint32_t i = 0; i < out->n_ops; i++) {
        const wt_op& op = out->ops[i];
        const uint16_t mask = op_info(op.opcode)->ref_mask;
        for (uint16_t a = 0; a < op.n_args; a++) {
            if (!(mask >> a & 1u)) continue;
            const uint32_t v = op.args[a];
            if (op.opcode == OP_DMA && (v & 0xC000u) == 0xC000u) continue;  // engine face
            // only 0x8000-flagged values point into slot space; bare values are temp ids
            if ((v & 0x8000u) && (v & 0x7FFFu) >= out->n_slots) return WT_ERR_BAD_REF;
        }
    }
    return WT_OK;
}

extern "C" const char* wt_err_str(int rc) {
    switch (rc) {
    case WT_OK: return "OK";
    case WT_ERR_SHORT: return "buffer shorter than header";
    case WT_ERR_MAGIC: return "bad magic";
    case WT_ERR_VER: return "unsupported version";
    case WT_ERR_ENDIAN: return "endian check failed";
    case WT_ERR_NSLOTS: return "n_slots out of range";
    case WT_ERR_NOPS: return "n_ops out of range";
    case WT_ERR_SLOTS_OVERRUN: return "slot table overruns buffer";
    case WT_ERR_WEIGHT_OVERRUN: return "slot offset+len overruns weight region";
    case WT_ERR_OP_TRUNC: return "op table truncated";
    case WT_ERR_OPCODE: return "unknown opcode";
    case WT_ERR_ARITY: return "n_args mismatch for opcode";
    case WT_ERR_BAD_REF: return "op arg references missing slot";
    case WT_ERR_ALIGN: return "slot offset not 128B aligned";
    default: return "unknown";
    }
}
