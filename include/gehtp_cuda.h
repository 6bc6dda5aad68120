/* libgehtp_cuda.so — CUDA (sm_100a) executor for WTOP runlists.
 *
 * The wt_exec_* entry points below are the ones the GEHTP runners bind
 * (kernels/include/oplist_exec.h:31-114 in the reference), with the same
 * argument meaning, return codes and lifetime rules. The op list, the slot
 * table and the TEMPOFF / STATE tables are consumed as they are; temps live in
 * one device arena, slots are uploaded once, states stay resident across runs.
 *
 * Return convention of the run calls: 0 = every op succeeded; >0 = 1-based
 * index of the op that failed; -1 = range / TEMPOFF / STATE table error.
 * `err` (may be NULL) receives a short reason. One engine per process, one
 * caller thread (the reference has the same rule).
 *
 * The library never computes on the CPU: without a usable CUDA device every
 * run call fails with "no CUDA device".
 */
#ifndef GEHTP_B200_GEHTP_CUDA_H
#define GEHTP_B200_GEHTP_CUDA_H

#include <stddef.h>
#include <stdint.h>
#include "wtop_format.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- engine */

/* oplist_exec.h:31 — run every op of `b`. */
int wt_exec_run(const struct wt_blob* b, uint32_t* engine_m,
                int64_t* op_us, char* err, size_t errn);

/* oplist_exec.h:66 — run ops [first, first+count). Running the list in
 * pieces leaves the same bytes in every temp as one whole run. */
int wt_exec_run_range(const struct wt_blob* b, uint32_t first, uint32_t count,
                      uint32_t* engine_m, int64_t* op_us, char* err, size_t errn);

/* oplist_exec.h:75 — as wt_exec_run, with the EXT_IN slot read from host
 * memory `in_ptr` and temp `out_temp` copied to host memory `out_ptr` after
 * the run (its last written size). Either pointer may be NULL. */
int wt_exec_run_io(const struct wt_blob* b, const void* in_ptr, void* out_ptr,
                   uint32_t out_temp, uint32_t* engine_m, int64_t* op_us,
                   char* err, size_t errn);

/* oplist_exec.h:35-38 — host view of a temp. The pointer is a pinned host
 * mirror refreshed from the device by this call; it stays valid until
 * wt_exec_shutdown() or the next wt_exec_temp() of the same id. */
uint8_t* wt_exec_temp(uint32_t id);
uint32_t wt_exec_temp_bytes(uint32_t id);
uint32_t wt_exec_temp_last_bytes(uint32_t id);

/* oplist_exec.h:43 — drops the plan, the temp arena and uploaded slots.
 * Persistent states survive (decode semantics); call on PASS and FAIL paths. */
void wt_exec_shutdown(void);

/* oplist_exec.h:48 — zero every persistent state and its position counter. */
void wt_exec_state_reset(void);

/* oplist_exec.h:56 — static temp pool supplied by the caller. On the GPU the
 * pool memory itself is device memory owned by the engine, so `base` is only
 * tested for NULL; `offsets[id]` (0xFFFFFFFF = not in table) and the two
 * capacities are honoured. NULL/NULL restores the default. */
void wt_exec_pool_init(uint8_t* base, uint32_t total_cap, uint32_t static_cap,
                       const uint32_t* offsets);

/* oplist_exec.h:62-68 */
struct wt_exec_stats {
    uint32_t ops, nop, matmul, rmsnorm, silu, pin, pin_skipped;
    uint32_t im2col, conv2d, add, spill, fill, transpose;
};
void wt_exec_get_stats(struct wt_exec_stats* st);

/* oplist_exec.h:81 — base of the external weight file image (host memory)
 * for slots marked WT_SLOT_EXT_WGT. Borrowed for the life of the process. */
void wt_exec_set_ext_weights(const void* wgt_ptr);

/* oplist_exec.h:87-95 — per-op timestamps. Tensor-core ops report
 * WT_ENG_HMX, other GPU kernels WT_ENG_HVX, host-only bookkeeping ops
 * WT_ENG_SCALAR. Registering a buffer (or passing op_us) makes the engine
 * synchronise after every op; without either, ops are queued back to back. */
enum wt_engine { WT_ENG_SCALAR = 0, WT_ENG_HVX = 1, WT_ENG_HMX = 2 };
struct wt_op_ts {
    uint32_t start_us, dur_us, dma_us, dma_bytes, engine;
};
void wt_exec_set_ts(struct wt_op_ts* buf, uint32_t cap);

/* oplist_exec.h:101 — per-op trace lines (to $GEHTP_TRACE_FILE or
 * /tmp/gehtp_optrace.txt). Off by default here. */
void wt_exec_set_trace(int on);

/* oplist_exec.h:108 — "opidx:temp,opidx:temp": after op `opidx` of a range
 * succeeds, temp `temp` is written to /tmp/hook_<idx>_<temp>.f16.raw.
 * Falls back to $GEHTP_HOOK when never set. */
void wt_exec_set_hook(const char* spec);

/* oplist_exec.h:112 — one JSON line per slot and op through `emit`. */
void wt_w3_report(const char* blob_name, const uint8_t* buf, size_t size,
                  const struct wt_blob* w,
                  void (*emit)(const char* line, void* ud), void* ud);

/* ------------------------------------------------ CUDA-side configuration
 * None of these has a counterpart in the reference; they select how the same
 * op list is run on GPUs. */

/* Device ordinal used by the engine (default: $GEHTP_CUDA_DEVICE or 0).
 * Call before the first run. Returns 0, or -1 with no such device. */
int gehtp_cuda_set_device(int ordinal);

/* 1 = recognise op chains at plan time and run each as one kernel (attention
 * over the KV ring, rotary embedding, SwiGLU, norm+matmul prologues).
 * 0 = one kernel per op (every temp materialised; used for op-by-op parity).
 * Default 1, or $GEHTP_CUDA_FUSE. */
void gehtp_cuda_set_fusion(int on);

/* 1 = after a first eager run of a blob, replay whole runs as one CUDA graph.
 * Default 1, or $GEHTP_CUDA_GRAPH. Timing (op_us / set_ts), hooks and traces
 * force eager execution for that run. */
void gehtp_cuda_set_graph(int on);

/* Tensor parallelism inside one node: this process is `rank` of `world`.
 * `nccl_unique_id` is the 128-byte id made by rank 0 and sent to the others by
 * the caller (the engine does no rendezvous of its own). Column- and
 * row-parallel matmuls are found from the op list's dataflow. Returns 0 or -1. */
int gehtp_cuda_tp_init(int rank, int world, const void* nccl_unique_id, size_t id_bytes);
int gehtp_cuda_tp_unique_id(void* out_id, size_t id_bytes);
void gehtp_cuda_tp_shutdown(void);
/* Ops whose first output is a partial sum over the ranks (the outputs of
 * row-parallel projections): the engine all-reduces it in place right after
 * the op. Indices come from the blob's sideband manifest. */
int gehtp_cuda_tp_allreduce_after(const uint32_t* op_idx, uint32_t n);
/* Optional fast path for the small all-reduces of a decode step: a one-kernel
 * all-reduce over NVLink peer memory (each rank pushes its partial sums into a
 * mailbox in every rank's HBM, waits for the peers' flags with a bounded poll,
 * and adds the slots in rank order). After gehtp_cuda_tp_init, every rank
 * calls _export (64-byte CUDA IPC handle of its mailbox), the caller gathers
 * the handles of all ranks in rank order (`handle_stride` bytes apart) and
 * every rank calls _import — every rank, also one whose _export failed: _import ends with an
 * agreement over the communicator of tp_init (minimum of the ranks' success flags), so that either
 * all ranks use the mailboxes (0) or none does (-1 on every rank; all-reduces then go through NCCL).
 * Vectors above 1 MiB keep using NCCL. A peer that never arrives makes the run return an error
 * instead of hanging. */
int gehtp_cuda_tp_p2p_export(void* handle_out, size_t handle_bytes);
int gehtp_cuda_tp_p2p_import(const void* handles, size_t handle_stride, int world);
/* Back to NCCL for every all-reduce (call it on every rank or on none). */
void gehtp_cuda_tp_p2p_disable(void);
/* Number of polls a device-side wait of the peer-memory exchange makes before it gives up,
 * leaves a code in the engine's status word and lets the run return "all-reduce timed out"
 * (0 = the default, a few seconds). Every such wait is bounded; this only moves the bound. */
void gehtp_cuda_set_wait_limit(uint32_t polls);
/* Bring-up aid for the peer-memory exchange on ONE GPU: this process becomes rank 0 of
 * `world`, and the other ranks' mailboxes are private buffers on the same GPU that nobody
 * ever writes. Every exchange therefore runs into its wait limit and the run reports the
 * timeout: the way to see the failure path of a lost peer without losing one. Undone by
 * gehtp_cuda_tp_shutdown. Returns 0 or -1. */
int gehtp_cuda_tp_p2p_loopback(int world);

/* Kernels launched by the engine since the process started. */
uint64_t gehtp_cuda_launch_count(void);
/* Number of ops of the current plan replaced by fused launches. */
uint32_t gehtp_cuda_fused_ops(void);
/* Number of ops of the current plan whose result is a constant of the blob (data movement over weight slots:
 * slices, transposes, broadcasts of tables): executed by the first run that reaches them, skipped afterwards. */
uint32_t gehtp_cuda_const_ops(void);
/* Number of TEMPOFF entries of the current plan that were moved out of the
 * static pool because their byte ranges overlap another entry's while both
 * tensors are live (the emitter binds plan offsets to recycled temp ids,
 * compiler/tools/wtop_ops/wtop_ops.hpp:143-167). 0 for a sound table. */
uint32_t gehtp_cuda_demoted_temps(void);
/* Device pointer / stream the engine uses (so a host that owns device memory,
 * e.g. a bench, can time on the right stream). */
void* gehtp_cuda_stream(void);
void* gehtp_cuda_temp_dev(uint32_t id);
/* Wait for every queued op. Returns 0 or the CUDA error code. */
int gehtp_cuda_sync(void);
const char* gehtp_cuda_last_error(void);
/* How a run reports the word a kernel leaves when it cannot finish: the message that
 * wt_exec_run* puts into `err` and the value it returns for device status `code` (a 1-based op
 * index for a KV gather that found another position in its ring slot; -1 with its own message
 * for each bounded wait that ran out: peer-memory all-reduce 0x80000001, decode-attention tile
 * copy 0x80000002, tcgen05 GEMM pipeline barrier 0x80000003). Pure host function. */
int gehtp_cuda_status_message(uint32_t code, char* msg, size_t msg_bytes);

/* Device-resident I/O for hosts that keep buffers on the GPU: like
 * wt_exec_run_io but `in_dev` / `out_dev` are device pointers and nothing is
 * synchronised before return. */
int gehtp_cuda_run_dev(const struct wt_blob* b, const void* in_dev, void* out_dev,
                       uint32_t out_temp, char* err, size_t errn);

/* Eager run with a CUDA event pair (on the engine stream) around every launch
 * unit: op_ms[i] = device milliseconds of the unit that starts at op i, 0 for
 * ops absorbed into a fused unit. `in_ptr` is host memory as in wt_exec_run_io. */
int gehtp_cuda_run_profiled(const struct wt_blob* b, const void* in_ptr, uint32_t out_temp,
                            float* op_ms, uint32_t cap, char* err, size_t errn);
/* Device time (summed, ms) and launch count of the decode attention kernel alone in the last
 * gehtp_cuda_run_profiled: its launch unit also holds the rotary/append and merge kernels. */
void gehtp_cuda_profiled_attn(float* total_ms, uint32_t* launches);

/* Persistent-state image exchange (the reference keeps states inside its
 * engine and can only fill them by running append ops; its host golden saves
 * and restores them through a file, compiler/src/ops/host_decode_state.cpp:14-62).
 * load: copy `bytes` from host (or device) memory into state `idx`; with
 * kv_elems != 0 the state is a KV ring of kv_elems K values per position, ring
 * slots [0, n_positions) are marked as holding positions 0.. and the state's
 * position counter becomes n_positions. `b` (may be NULL once a blob has run)
 * makes sure the blob's state table is resident first. */
int gehtp_cuda_state_load(const struct wt_blob* b, uint32_t idx, const void* src, size_t bytes,
                          int src_is_device, uint32_t kv_elems, uint32_t n_positions,
                          char* err, size_t errn);
int gehtp_cuda_state_set_count(uint32_t idx, uint32_t n_positions);
int gehtp_cuda_state_read(uint32_t idx, void* dst, size_t bytes);

/* State file in the layout of the reference's host golden (magic "HDS1";
 * host_decode_state_save / _load, compiler/src/ops/host_decode_state.cpp:14-62):
 *   "HDS1", u32 n = 42, u32 kv_count[6], f32 kv_k[6][64][512], f32 kv_v[6][64][512],
 *   f32 conv_win[18][3*6144], f32 delta_s[18][16*128*128]
 * (compiler/include/hnnx/host_decode_state.hpp:17-27). The blob's state table must be the
 * 42-state decode table: KV rings 0..5 with 512 values per face, conv windows 6..23, delta
 * states 24..41 (decode_state_gid, compiler/tools/wtop_ops/wtop_ops.hpp:478-492). KV faces
 * are fp16 on the device and fp32 in the file; positions 0..count-1 are exchanged.
 * save: 0 or -1. load: 0 loaded, 1 no such file, -1 bad file or table (checked before anything is written),
 * the return values of host_decode_state_load. */
int gehtp_cuda_state_save_hds1(const struct wt_blob* b, const char* path, char* err, size_t errn);
int gehtp_cuda_state_load_hds1(const struct wt_blob* b, const char* path, char* err, size_t errn);

/* ------------------------------------------------------- W4A16 group-64
 * Weight slot form accepted by opcode 1 on this executor (the reference's
 * opcode 1 is an HMX-specific integer contract found by slot size,
 * oplist_exec.c:438-529; it selects W4A16 when the weight slot holds K*N/2
 * bytes, wtop_ops/op_matmul.cpp:40-44):
 *
 *   slot = nibbles[K][N/2] then scales[K/64][N], len = K*N/2 + 2*(K/64)*N
 *   byte[k][j] = q[k][2j] | q[k][2j+1] << 4      (low nibble = even column;
 *                nibble order of kernels/host/vendor/weight_pack.cc:114)
 *   w[k][n] = fp16( (q[k][n] - 8) * scale[k/64][n] ),  y = fp16( sum_k a*w ) with
 *   fp32 accumulation. K % 64 == 0, N % 16 == 0.
 *
 * Op args: [a_ref, w_ref, out_temp, M, K, N]; a_ref / w_ref decode like every
 * other ref. A weight slot of exactly K*N/2 bytes (the legacy side-band form)
 * is rejected with "legacy W4A16 slot form unsupported on CUDA". */
#define GEHTP_W4_GROUP 64u
size_t gehtp_w4a16_slot_bytes(uint32_t K, uint32_t N);

/* Host-pointer kernel entry points: each copies its operands to the device,
 * runs the same kernel the engine uses, and copies the result back. For
 * tests and small tools; 0 on success, -1 otherwise (see gehtp_cuda_last_error).
 *
 * gehtp_w4a16_matmul: `w_slot` in the slot form above. `path`: 0 = engine's
 * choice by M, 1 = streaming GEMV (mma.sync), 2 = tcgen05 GEMM with the tile
 * chosen from the shape, 3 / 4 / 5 = tcgen05 GEMM with 128x128 / 256x128 /
 * 256x256 tiles (256-wide tiles need N % 256 == 0). */
int gehtp_w4a16_matmul(const uint16_t* a_f16, const uint8_t* w_slot, uint16_t* y_f16,
                       uint32_t M, uint32_t K, uint32_t N, int path);
/* Integer q-8 of every weight, read back out of the device-side packed
 * layout: out_i8[k*N + n]. Proves the repack is lossless. */
int gehtp_w4a16_unpack(const uint8_t* w_slot, int8_t* out_i8, uint32_t K, uint32_t N);
/* y = x / sqrt(mean(x^2) + 1e-6) * gamma (+ beta); rows x width (opcode 25,
 * oplist_exec.c:1817-1872). beta may be NULL. */
int gehtp_rmsnorm(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta,
                  uint16_t* y, uint32_t rows, uint32_t width);
/* Decode attention straight off a KV ring (layout of kvcache.h:19-47:
 * slot = [K face kv_heads*hd][V face kv_heads*hd], position p in slot
 * p % nslots): out[h] = softmax(q[h]·K^T * scale + mask) · V for n_kv
 * positions; head h reads KV head h / (n_heads/kv_heads). mask (n_kv f16,
 * additive) may be NULL. */
int gehtp_attn_decode(const uint16_t* q, const uint16_t* kv_ring, const uint16_t* mask,
                      uint16_t* out, uint32_t n_heads, uint32_t kv_heads, uint32_t head_dim,
                      uint32_t n_kv, uint32_t nslots, float scale);

/* Device-pointer forms of the kernels above: every buffer is device memory of
 * the caller, work is queued on the engine stream (gehtp_cuda_stream) and not
 * waited for. `packed_dev` is the strip-major layout made by gehtp_dev_w4_repack
 * from the nibble part of a weight slot (K*N/2 bytes in, K*N/2 bytes out);
 * `scales_dev` is the fp16 [K/64][N] part of the slot. gehtp_dev_w4a16_swiglu
 * computes silu-gated gate/up projections in one pass (M <= 16: the streaming
 * kernel; M >= 64 with N a multiple of 128: the tcgen05 GEMM with both
 * accumulators in TMEM; -1 for shapes neither form takes);
 * gehtp_dev_rmsnorm normalises f16(x + res) when res_dev is given (and stores
 * that sum to sum_dev when not NULL). */
int gehtp_dev_w4_repack(const uint8_t* slot_dev, uint32_t* packed_dev, uint32_t K, uint32_t N);
int gehtp_dev_w4a16_matmul(const uint16_t* a_dev, const uint32_t* packed_dev, const uint16_t* scales_dev,
                           uint16_t* y_dev, uint32_t M, uint32_t K, uint32_t N, int path);
int gehtp_dev_matmul_f16_nk(const uint16_t* a_dev, const uint16_t* w_dev, uint16_t* y_dev, uint32_t M, uint32_t K, uint32_t N);
int gehtp_dev_w4a16_swiglu(const uint16_t* a_dev, const uint32_t* pg, const uint16_t* sg,
                           const uint32_t* pu, const uint16_t* su, uint16_t* y_dev,
                           uint32_t M, uint32_t K, uint32_t N);
int gehtp_dev_rmsnorm(const uint16_t* x_dev, const uint16_t* res_dev, const uint16_t* gamma_dev,
                      const uint16_t* beta_dev, uint16_t* sum_dev, uint16_t* y_dev,
                      uint32_t rows, uint32_t width);

/* Timing aid: everything queued on the engine stream between begin and end is
 * captured into one CUDA graph, replayed `reps` times, and the mean device time
 * of a replay is returned in milliseconds. */
int gehtp_cuda_capture_begin(void);
int gehtp_cuda_capture_end_replay(int reps, float* ms_per_replay);

/* No counterpart in the reference. The same decode attention as
 * gehtp_attn_decode, for callers that are not allowed to allocate device memory
 * (a serving loop living inside a pre-carved memory pool, a latency-critical
 * thread that must not take the driver's allocation lock, a process with a fixed
 * device-memory budget). All four buffers are DEVICE pointers owned by the caller
 * (q and out: n_heads*head_dim fp16; ring: nslots*2*kv_heads*head_dim fp16; mask:
 * n_kv fp16 or NULL). The kernel's scratch is a fixed array inside the library's
 * device image: GEHTP_NOALLOC_SCRATCH_BYTES on every GPU that loads the library,
 * held until the process exits. The call allocates and frees nothing, only
 * queues work on `stream` (a cudaStream_t, NULL = default stream) of the current
 * device, and does not wait for it.
 * Limit: the context is cut into as many slices as keep every SM busy, fewer
 * when the partial results (n_heads * slices * (head_dim+2) * 4 bytes) would not
 * fit; unsliced, n_heads * (head_dim+2) * 4 bytes must fit in the array; larger problems return -1 with a message in
 * gehtp_cuda_last_error(). The first call on each device looks up the array's
 * device address; make that first call before starting any stream capture.
 * All calls share the one array and it keeps whatever the last call left in it:
 * calls that overlap on the GPU race and must be serialised by the caller. */
#define GEHTP_NOALLOC_SCRATCH_BYTES (5u * 1024u * 1024u)
int gehtp_attn_decode_noalloc(const uint16_t* q_dev, const uint16_t* ring_dev, const uint16_t* mask_dev,
                              uint16_t* out_dev, uint32_t n_heads, uint32_t kv_heads, uint32_t head_dim,
                              uint32_t n_kv, uint32_t nslots, float scale, void* stream);
/* No counterpart in the reference. The kernel behind gehtp_attn_decode_noalloc waits for
 * its K/V tile copies with a bounded poll; a wait that runs out leaves a code in a status
 * word that also lives in the library's device image. This reads and clears that word for
 * the current device (one 4-byte device-to-host copy, no allocation): 0 = every call since
 * the last query completed, > 0 = a wait ran out and that call's output is incomplete,
 * -1 = the copy failed. Call it after synchronising the stream the calls were queued on. */
int gehtp_attn_decode_noalloc_status(void);

#ifdef __cplusplus
}
#endif
#endif
