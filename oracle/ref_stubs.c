/* Host stand-ins for the Hexagon-only plumbing the reference executor links
 * against (VTCM cache, UserDMA, HMX engine). Test infrastructure only: with
 * these the reference's oplist_exec.c runs its own scalar CPU code paths.
 * DMA becomes memcpy; the HMX W4A16 engine and the VTCM cache report failure,
 * so legacy opcode 1 is unavailable in this build (its golden surfaces are
 * not in the reference checkout either). */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include "dc_parts.h"
#include "wtcache.h"

void dc_arena_init(struct dc_arena* a, uint8_t* base, uint32_t size) {
    a->base = base; a->size = size; a->off = 0;
}
void dc_clean_ddr(const void* p, uint32_t bytes) { (void)p; (void)bytes; }
int dc_dma_init(struct dc_dma* d, uint8_t* src, uint8_t* dst, uint32_t bytes, dc_mutex_t* mu) {
    d->src = src; d->dst = dst; d->bytes = bytes; d->mu = mu; d->desc = NULL;
    d->src_bypass = 1; d->dst_bypass = 0;
    return 0;
}
void dc_dma_destroy(struct dc_dma* d) { (void)d; }
int dc_dma_once(struct dc_dma* d) { memcpy(d->dst, d->src, d->bytes); return 0; }
int dc_dma_once_ex(struct dc_dma* d, int sb, int db) { (void)sb; (void)db; return dc_dma_once(d); }
void dc_dma_reset(void) {}
void dc_dma_get(int64_t* us, int64_t* bytes) { if (us) *us = 0; if (bytes) *bytes = 0; }
void dc_mutex_init(dc_mutex_t* m) { if (m) *m = 0; }
int dc_w4_carve(struct dc_w4* e, struct dc_arena* a, uint32_t m, uint32_t k, uint32_t n,
                const uint8_t* atbl, const uint8_t* otbl) {
    (void)e; (void)a; (void)m; (void)k; (void)n; (void)atbl; (void)otbl; return 1;
}
int dc_w4_invoke(struct dc_w4* e) { (void)e; return 1; }
void* hmx_runtime_get_vtcm_base(void) { return NULL; }
void hmx_runtime_teardown(void) {}
int wtcache_open(struct wtcache_ctx** out, uint32_t pin_cap_bytes) {
    (void)out; (void)pin_cap_bytes; return -1;
}
int wtcache_close(struct wtcache_ctx* ctx) { (void)ctx; return 0; }
void wtcache_layout(const struct wtcache_ctx* ctx, void** vb, uint32_t* vs, void** pb, uint32_t* pc) {
    (void)ctx; if (vb) *vb = NULL; if (vs) *vs = 0; if (pb) *pb = NULL; if (pc) *pc = 0;
}
