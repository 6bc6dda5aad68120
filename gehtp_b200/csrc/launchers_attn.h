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

}  // namespace gehtp
