/* CPU restatement of the GEHTP LLM hot-path ops. TEST INFRASTRUCTURE: only
 * tests, the smoke check and the bench's CPU-baseline legs may load this; the
 * product never calls it.
 *
 * Every function follows the reference routine cited beside it (paths under
 * the reference's kernels/ directory). Parity status: all functions except the
 * W4A16 group-64 pair are pinned against the reference executor compiled for
 * the host (oracle/_ref, built by the Makefile) by tests/test_oracle_pins.py and
 * against the golden vectors under tests/golden/. orc_w4_dequant /
 * orc_w4a16_matmul restate a weight format the reference does not define
 * (group-64 fp16 scales over a [K][N/2] nibble matrix): PARITY UNPINNED for the
 * format itself; its nibble order follows kernels/host/vendor/weight_pack.cc:114
 * and its matmul is the pinned orc_matmul_f16 run on the dequantised weights. */
#ifndef GEHTP_ORACLE_H
#define GEHTP_ORACLE_H
#include <stdint.h>
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

float orc_f16_to_f32(uint16_t h);            /* src/runtime/oplist_exec.c:371-393 */
uint16_t orc_f32_to_f16(float f);            /* src/runtime/oplist_exec.c:395-418 */

/* int4 -> q-8 (int8) and -> fp16((q-8)*scale[k/64][n]) */
void orc_w4_unpack_i8(const uint8_t* nib, int8_t* out, uint32_t K, uint32_t N);
void orc_w4_dequant(const uint8_t* slot, uint16_t* w_f16, uint32_t K, uint32_t N);
void orc_w4a16_matmul(const uint16_t* a, const uint8_t* slot, uint16_t* y, uint32_t M, uint32_t K, uint32_t N);

/* src/runtime/oplist_exec.c:1786-1812 (scalar path of exec_matmul_f16) */
void orc_matmul_f16(const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K,
                    uint32_t N, uint32_t n0, uint32_t N_full, int t0, int t1, int batched, uint32_t Bn);
/* src/runtime/oplist_exec.c:1858-1870 */
void orc_rmsnorm2(const uint16_t* x, const uint16_t* g, const uint16_t* b, uint16_t* y, uint32_t rows, uint32_t width);
/* src/runtime/oplist_exec.c:1172-1192 + src/hvx/hvx_softmax.c:83-95 */
void orc_softmax(const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n);
/* src/runtime/oplist_exec.c:1146-1159 (scalar) / src/hvx/hvx_binary.c host loops (n >= 32) */
void orc_binary(const uint16_t* a, const uint16_t* b, uint16_t* y, uint32_t n, uint32_t subtype);
/* src/runtime/oplist_exec.c:1048-1077 */
int orc_unary(const uint16_t* x, uint16_t* y, uint32_t n, uint32_t subtype);

/* KV ring: src/runtime/kvcache.c:17-76; gather: src/runtime/oplist_exec.c:2208-2229 */
void orc_kv_append(uint16_t* ring, uint32_t* posmap, uint32_t nslots, uint32_t kv_elems,
                   const uint16_t* k, const uint16_t* v, uint32_t pos);
int orc_kv_gather(const uint16_t* ring, const uint32_t* posmap, uint32_t nslots, uint32_t n_kv,
                  uint32_t pstride, uint32_t n_heads, uint32_t kv_heads, uint32_t hd, uint16_t* kT, uint16_t* vo);
/* the attention op chain as the runlist carries it: gather, q.K^T (batched
 * matmul), scale (mul or div), + mask, softmax, .V — fp16 after every op.
 * out [n_heads][hd]; mask may be NULL (then no mask op). */
int orc_attn_decode_chain(const uint16_t* q, const uint16_t* ring, const uint32_t* posmap,
                          uint32_t nslots, uint32_t n_kv, uint32_t n_heads, uint32_t kv_heads,
                          uint32_t hd, float scale, int scale_div, const uint16_t* mask, uint16_t* out);
/* same math in double, no intermediate rounding: out_f64 [n_heads][hd] */
void orc_attn_decode_f64(const uint16_t* q, const uint16_t* ring, uint32_t nslots, uint32_t n_kv,
                         uint32_t n_heads, uint32_t kv_heads, uint32_t hd, double scale,
                         const uint16_t* mask, double* out);

/* src/runtime/oplist_exec.c:1363-1374 */
void orc_conv1d_ssm(const uint16_t* x, const uint16_t* w, uint16_t* y, uint32_t seq, uint32_t C, uint32_t k);
/* src/hvx/gdn_kern.c:14-38 */
void orc_conv1d_step(const uint16_t* x, const uint16_t* w, uint16_t* y, float* win, uint32_t C, uint32_t dc);
/* src/hvx/gdn_kern.c:54-167 */
int orc_delta_chunk(const uint16_t* k, const uint16_t* v, const uint16_t* q, const uint16_t* beta,
                    const uint16_t* g, uint16_t* y, float* S, int c, int ntok, int H, int D, int q_raw);
/* src/hvx/gdn_ref.c:93-112, per-token recurrence in fp32 */
void orc_delta_token(float* S, int D, const float* k, const float* v, const float* q, float beta, float g, float* y);

#ifdef __cplusplus
}
#endif
#endif
