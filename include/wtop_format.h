/* WTOP runlist blob: wire format and in-memory form.
 *
 * This is the ABI shared with the GEHTP toolchain (kernels/include/oplist_parse.h:1-312
 * in the reference): a blob produced by its `wtop_emit` parses with wt_parse()
 * below into the same struct layout, and the numeric values of every constant
 * here are the reference's. Names are kept so that callers written against the
 * reference header compile unchanged.
 *
 * Wire layout, little endian:
 *   0   "WTOP"
 *   4   u16 version (1 or 2)        6   u16 0x1234 byte-order probe
 *   8   u32 n_slots                 12  u32 n_ops
 *   16  slot records: v1 = 16 B {len, count, offset32, addr}
 *                     v2 = 24 B {len, count, offset_lo, offset_hi, addr, reserved}
 *   ..  op records: {u16 opcode, u16 n_args, u32 args[n_args]}
 *   ..  weight area, starting at the next multiple of 128 after the op table;
 *       slot offsets are relative to it and 128-byte aligned.
 *
 * An op argument that names a tensor is a "ref":
 *   bare value          temp id
 *   0x8000 | slot       constant / input slot
 *   0x4000 | temp       temp resident in on-chip scratch (VTCM on Hexagon; an
 *                       ordinary arena temp on a GPU)
 *   0x6000 | state      persistent state buffer (KV ring, conv window, delta S)
 *   0xC000 | face       engine face, OP_DMA only
 */
#ifndef GEHTP_B200_WTOP_FORMAT_H
#define GEHTP_B200_WTOP_FORMAT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WT_BLOB_VER        1u
#define WT_BLOB_VER_2      2u
#define WT_ENDIAN_CHK      0x1234u
#define WT_SLOT_SIZE       16u
#define WT_SLOT_SIZE_V2    24u
#define WT_WEIGHT_ALIGN    128u
#define WT_MAX_SLOTS       4096u
#define WT_MAX_OPS         65536u
#define WT_MAX_ARGS        16u
#define WT_MAX_STATES      64u
#define WT_EXEC_MAX_TEMPS  4096

/* slot.addr markers (oplist_parse.h:62-88) */
#define WT_SLOT_EXT_IN     0xFFFFFFFFu  /* data comes from run_io's in_ptr        */
#define WT_SLOT_EXT_OUT    0xFFFFFFFEu
#define WT_SLOT_TEMPOFF    0xFFFFFFFDu  /* static temp offset table               */
#define WT_SLOT_EXT_WGT    0xFFFFFFFCu  /* data in the external weight file       */
#define WT_SLOT_STATE      0xFFFFFFFBu  /* persistent state size table            */
#define WT_KV_POS_AUTO     0xFFFFFFFAu  /* KV pos / n_kv taken from state counter */

#define WT_REF_SLOT_FLAG   0x8000u
#define WT_REF_VTCM_FLAG   0x4000u
#define WT_REF_STATE_FLAG  0x6000u
#define WT_REF_ENG_FLAG    0xC000u
#define WT_ENG_ACT  0u
#define WT_ENG_OUT  1u
#define WT_ENG_WT   2u
#define WT_ENG_BIAS 3u
#define WT_DMA_FENCE_NONE  0xFFu

/* Opcodes (oplist_parse.h:103-215). Argument lists are given beside the
 * executor entry that implements each one, in gehtp_b200/csrc/. */
enum {
    OP_NOP = 0, OP_MATMUL_W4A16 = 1, OP_RMSNORM_F16 = 2, OP_PIN = 3, OP_SILU_F16 = 4,
    OP_IM2COL = 5, OP_CONV2D_F16 = 6, OP_ADD_F16 = 7, OP_SPILL = 8, OP_FILL = 9,
    OP_TRANSPOSE_F16 = 10, OP_UNARY_F16 = 11, OP_BINARY_F16 = 12, OP_SOFTMAX_F16 = 13,
    OP_CONCAT_F16 = 14, OP_STRIDED_SLICE_F16 = 15, OP_SPLIT_F16 = 16, OP_REDUCE_F16 = 17,
    OP_CUMSUM_F32 = 18, OP_CONV1D_SSM_F16 = 19, OP_GATHER_F16 = 20, OP_ARGMAX_F16 = 21,
    OP_KV_APPEND_F16 = 22, OP_KV_GATHER_F16 = 23, OP_MATMUL_F16 = 24, OP_RMSNORM2_F16 = 25,
    OP_BROADCAST_F16 = 26, OP_TRANSPOSE_GEN_F16 = 27, OP_SCATTER_ND_F16 = 28,
    OP_CONV1D_SSM_STEP_F16 = 29, OP_DELTA_CHUNK_F16 = 30,
    OP_DMA = 33, OP_PAD_F16 = 34, OP_MATMUL_F16_SPLIT = 35
};

/* Fixed argument count per opcode (oplist_parse.h:218-251). */
#define WT_ARITY_NOP 0
#define WT_ARITY_MATMUL 6
#define WT_ARITY_RMSNORM 4
#define WT_ARITY_PIN 1
#define WT_ARITY_SILU 3
#define WT_ARITY_IM2COL 15
#define WT_ARITY_CONV2D_F16 13
#define WT_ARITY_ADD_F16 4
#define WT_ARITY_SPILL 4
#define WT_ARITY_FILL 4
#define WT_ARITY_TRANSPOSE_F16 6
#define WT_ARITY_UNARY_F16 4
#define WT_ARITY_BINARY_F16 5
#define WT_ARITY_SOFTMAX_F16 4
#define WT_ARITY_CONCAT_F16 16
#define WT_ARITY_STRIDED_SLICE_F16 16
#define WT_ARITY_SPLIT_F16 16
#define WT_ARITY_REDUCE_F16 9
#define WT_ARITY_CUMSUM_F32 7
#define WT_ARITY_CONV1D_SSM_F16 6
#define WT_ARITY_GATHER_F16 15
#define WT_ARITY_ARGMAX_F16 3
#define WT_ARITY_KV_APPEND_F16 4
#define WT_ARITY_KV_GATHER_F16 7
#define WT_ARITY_MATMUL_F16 7
#define WT_ARITY_RMSNORM2_F16 5
#define WT_ARITY_BROADCAST_F16 12
#define WT_ARITY_TRANSPOSE_GEN_F16 8
#define WT_ARITY_SCATTER_ND_F16 14
#define WT_ARITY_DMA 8
#define WT_ARITY_PAD_F16 7
#define WT_ARITY_MATMUL_F16_SPLIT 9
#define WT_ARITY_CONV1D_SSM_STEP_F16 6
#define WT_ARITY_DELTA_CHUNK_F16 12

struct wt_slot {
    uint32_t len;     /* bytes */
    uint32_t count;   /* elements (f16 unless the consuming op says otherwise) */
    uint64_t offset;  /* bytes from weight_base (or from the external weight base) */
    uint32_t addr;    /* 0 or one of WT_SLOT_* */
};

struct wt_op {
    uint16_t opcode;
    uint16_t n_args;
    uint32_t args[WT_MAX_ARGS];
};

/* About 4.5 MB: callers allocate it on the heap. */
struct wt_blob {
    uint16_t ver;
    uint32_t n_slots;
    uint32_t n_ops;
    uint32_t weight_off;         /* absolute offset of the weight area in the blob */
    struct wt_slot slots[WT_MAX_SLOTS];
    struct wt_op ops[WT_MAX_OPS];
    const uint8_t* weight_base;  /* points into the caller's blob buffer */
    size_t weight_bytes;
};

/* wt_parse() results (oplist_parse.h:277-292). */
enum {
    WT_OK = 0,
    WT_ERR_SHORT = -1, WT_ERR_MAGIC = -2, WT_ERR_VER = -3, WT_ERR_ENDIAN = -4,
    WT_ERR_NSLOTS = -5, WT_ERR_NOPS = -6, WT_ERR_SLOTS_OVERRUN = -7,
    WT_ERR_WEIGHT_OVERRUN = -8, WT_ERR_OP_TRUNC = -9, WT_ERR_OPCODE = -10,
    WT_ERR_ARITY = -11, WT_ERR_BAD_REF = -12, WT_ERR_ALIGN = -13
};

/* Parses and bounds-checks a blob. `out` is valid only when WT_OK is returned;
 * it keeps pointers into `buf`, which must outlive it.
 * Replaces wt_parse (kernels/src/runtime/oplist_parse.c:86-169). */
int wt_parse(const uint8_t* buf, size_t size, struct wt_blob* out);

/* Short English text for a wt_parse() result (oplist_parse.c:171-189). */
const char* wt_err_str(int rc);

static inline uint32_t wt_rd_u32(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline uint16_t wt_rd_u16(const uint8_t* p) {
    return (uint16_t)(p[0] | (p[1] << 8));
}

#ifdef __cplusplus
}
#endif
#endif
