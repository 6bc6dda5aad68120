// Fused decode attention over the KV ring (ops_attn_decode.cu).
#pragma once
#include "launchers.h"

namespace gehtp {

struct AttnDecodeArgs {
    const uint16_t* q;         // [kv_heads_total * rep][hd], rotary already applied
    const uint16_t* ring;      // KV ring of kvcache.h layout
    const uint32_t* counter;   // device position counter (AUTO) or NULL
    uint32_t n_kv;             // positions to attend when counter == NULL
    uint32_t n_kv_add;         // added to *counter (1 when the append of this step has not bumped it yet)
    uint32_t* bump_counter;    // when set, the merge kernel advances this counter by one
    const uint16_t* mask;      // additive fp16 mask per position, or NULL
    uint32_t mask_seq_stride;  // elements between the masks of two sequences (0 = shared)
    uint32_t kvh_per_seq;      // KV heads of one sequence (batch folds into the head dim)
    float scale;               // score * scale, or score / scale when scale_div
    int scale_div;
    uint32_t rep;              // query heads per KV head (<= 16)
    uint32_t kv_heads;         // KV heads per ring slot (= kv_heads_total)
    uint32_t nslots;
    uint32_t nsplit;           // context slices per KV head (= slots per head in the scratch buffers)
    float* part_o;             // scratch [kv_heads_total][nsplit][rep][hd]
    float* part_ml;            // scratch [kv_heads_total][nsplit][rep][2]
    unsigned int* status;      // engine status word (bounded waits report here), or NULL
    int no_cache;              // 1: keep no host-side record of this ring (its tensor map is built per call)
};

// Timing probe for profiled runs: between begin and end every launch of the grouped attention kernel
// is bracketed by a CUDA event pair on its stream; end waits for nothing (the caller has synchronised)
// and returns the summed kernel time and the number of launches.
void attn_prof_begin();
void attn_prof_end(float* total_ms, uint32_t* launches);

uint32_t attn_decode_nsplit(uint32_t kv_heads_total, uint32_t max_positions, uint32_t rep, uint32_t hd, size_t max_floats);
size_t attn_decode_scratch_floats(uint32_t kv_heads_total, uint32_t rep, uint32_t hd, uint32_t nsplit);
// false: shape not handled (rep > 16 or head_dim not 64/128); nothing launched
bool k_attn_decode(cudaStream_t st, const AttnDecodeArgs& a, uint32_t hd, uint16_t* out,
                   uint32_t kv_heads_total);

// split + rotary + KV append in one launch (ops_fused.cu)
void k_rope_kv_append(cudaStream_t st, const uint16_t* qkv, const uint16_t* cos_q, const uint16_t* sin_q,
                      const uint16_t* cos_k, const uint16_t* sin_k, uint16_t* q_out, uint16_t* ring,
                      uint32_t* posmap, const uint32_t* counter, uint32_t B, uint32_t nh, uint32_t kvh,
                      uint32_t hd, uint32_t nslots, uint32_t pos_const);

// Prefill attention over token-major q [seq_q][nh][hd], k / v [seq_k][kvh][hd] -> out [seq_q][nh*hd]
// (ops_attn_prefill.cu). `skip` marks (64-row query tile, 64-position key tile) pairs whose mask is -inf
// everywhere, [ceil(seq_q/64)][ceil(seq_k/64)] bytes, or NULL. false: shape not handled, nothing launched.
bool k_attn_prefill(cudaStream_t st, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask,
                    size_t mask_head_stride, const uint8_t* skip, float scale, int scale_div, uint32_t seq_q,
                    uint32_t seq_k, uint32_t nh, uint32_t kvh, uint32_t hd, uint16_t* out);
uint32_t attn_prefill_tile();
// The same on tcgen05 / TMEM for head_dim 128 (attn_prefill_sm100.cu): 128 x 128 tiles, two passes (row statistics,
// then P V). `skip` has the 64 x 64 granularity of k_attn_prefill; `zero` (same shape, may be NULL) marks tiles whose
// mask is +0 everywhere. false: shape not taken, nothing launched.
bool k_attn_prefill_sm100(cudaStream_t st, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask,
                          size_t mask_head_stride, const uint8_t* skip, const uint8_t* zero, float scale, int scale_div,
                          uint32_t seq_q, uint32_t seq_k, uint32_t nh, uint32_t kvh, uint32_t hd, uint16_t* out,
                          unsigned int* status);
// rotary embedding, split-half form, with the op chain's roundings: out = f16(f16(x*cos) + f16(rot(x)*sin))
void k_rope(cudaStream_t st, const uint16_t* x, const uint16_t* cos_t, const uint16_t* sin_t, uint16_t* out,
            uint32_t rows, uint32_t hd);

// SPLIT q / rotary / SPLIT k / rotary / SPLIT v of a prefill block in one pass: qkv is [tokens][q | k | v],
// the tables are [tokens * heads][hd]; q_out [tokens][nh*hd], k_out and v_out [tokens][kvh*hd].
void k_qkv_split_rope(cudaStream_t st, const uint16_t* qkv, const uint16_t* cos_q, const uint16_t* sin_q,
                      const uint16_t* cos_k, const uint16_t* sin_k, uint16_t* q_out, uint16_t* k_out, uint16_t* v_out,
                      uint32_t tokens, uint32_t nh, uint32_t kvh, uint32_t hd);
// y = fp16(fp16(gate * fp16(sigmoid(gate))) * up), elementwise over n values (16-byte aligned operands).
void k_swiglu_tail(cudaStream_t st, const uint16_t* gate, const uint16_t* up, uint16_t* y, size_t n);


}  // namespace gehtp
