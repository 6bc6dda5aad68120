// Host-callable launchers of every kernel in the library. All pointers are
// device pointers; every launcher only enqueues work on `st`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gehtp {

extern unsigned long long g_launches;  // kernels launched by this library

// ---- elementwise / data movement (ops_elem.cu) ----
void k_unary(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t subtype);
void k_binary(cudaStream_t st, const uint16_t* a, const uint16_t* b, uint16_t* y, uint32_t n,
              uint32_t subtype, bool guard_div);
void k_select(cudaStream_t st, const uint16_t* c, uint32_t cn, const uint16_t* t, uint32_t tn,
              const uint16_t* f, uint32_t fn, uint16_t* y, uint32_t n);
void k_copy_bytes(cudaStream_t st, const void* src, void* dst, size_t bytes);
void k_fill16(cudaStream_t st, uint16_t* dst, size_t n, uint16_t v);
void k_concat_seg(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t seg,
                  uint32_t total_axis, uint32_t start);
void k_split_seg(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t seg,
                 uint32_t total_axis, uint32_t off);
void k_slice(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n_out, uint32_t rk,
             const uint32_t* b3, const uint32_t* s3, const uint32_t* istr3, const uint32_t* ostr3);
void k_broadcast(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t r,
                 uint32_t lead, const uint32_t* in_d4, const uint32_t* istr4, const uint32_t* ostr4);
void k_transpose_gen(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t rk,
                     const uint32_t* si4, const uint32_t* so4, const uint32_t* perm4);
void k_reduce(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t L,
              uint32_t inner, uint32_t subtype);
void k_pad(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t in_inner,
           uint32_t out_inner, uint32_t pad_before, uint16_t pv);
void k_cumsum(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n,
              uint32_t exclusive, uint32_t reverse);
void k_gather(cudaStream_t st, const uint16_t* tbl, const int32_t* idx, uint16_t* y, uint32_t n,
              uint32_t axis, uint32_t xrank, uint32_t irank, const uint32_t* td5,
              const uint32_t* xd5);
void k_scatter_nd(cudaStream_t st, const int32_t* idx, const uint16_t* upd, uint16_t* y,
                  uint32_t n, uint32_t K, uint32_t n_idx, uint32_t block, const uint32_t* od5);
void k_argmax(cudaStream_t st, const uint16_t* x, int32_t* y, uint32_t n);
// y[r] = argmax of row r of x [rows][n] (rows <= kArgmaxMaxRows): one launch for a batch of rows. false: too many rows.
constexpr uint32_t kArgmaxMaxRows = 256;
bool k_argmax_rows(cudaStream_t st, const uint16_t* x, int32_t* y, uint32_t rows, uint32_t n);
void k_im2col(cudaStream_t st, const uint16_t* a, uint16_t* cols, const uint32_t* args15);
void k_conv2d(cudaStream_t st, const uint16_t* A, const uint16_t* W, const uint16_t* Bv,
              uint16_t* out, uint32_t M, uint32_t K, uint32_t N, uint32_t oy0, uint32_t ox0,
              uint32_t out_W, uint32_t co0, uint32_t co_n);
void k_transpose_hwc(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t H, uint32_t W,
                     uint32_t C, uint32_t perm);

// ---- norms, softmax, KV ring, attention (ops_attn.cu) ----
void k_rmsnorm(cudaStream_t st, const uint16_t* x, const uint16_t* g, const uint16_t* b,
               uint16_t* y, uint32_t rows, uint32_t width);
// y = rmsnorm(a + r) * g, and sum_out = f16(a + r) when sum_out != NULL
void k_add_rmsnorm(cudaStream_t st, const uint16_t* a, const uint16_t* r, const uint16_t* g,
                   const uint16_t* b, uint16_t* sum_out, uint16_t* y, uint32_t rows, uint32_t width);
void k_softmax(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n);
// pos_const == 0xFFFFFFFA: position = *counter, and the counter is advanced.
void k_kv_append(cudaStream_t st, const uint16_t* k, const uint16_t* v, uint16_t* ring,
                 uint32_t* posmap, uint32_t* counter, uint32_t kv_elems, uint32_t nslots,
                 uint32_t pos_const);
void k_kv_gather(cudaStream_t st, const uint16_t* ring, const uint32_t* posmap,
                 const uint32_t* counter, uint16_t* kT, uint16_t* vo, uint32_t n_kv_const,
                 uint32_t pstride, uint32_t n_heads, uint32_t kv_heads, uint32_t hd,
                 uint32_t nslots, unsigned int* status, unsigned int op_code);

// ---- matmuls (ops_matmul.cu, ops_w4a16.cu) ----
void k_matmul_f16(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M,
                  uint32_t K, uint32_t N, uint32_t n0, uint32_t N_full, int t0, int t1,
                  uint32_t Bn);

// W stored [N, K] on the tensor cores (M >= 128: TMA-fed tcgen05 GEMM) or as a streaming GEMV (M < 32),
// f16_gemm_sm100.cu; y rows are ldy elements apart. false: shape not taken, nothing launched.
bool k_matmul_f16_nk(cudaStream_t st, const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M,
                     uint32_t K, uint32_t N, uint32_t ldy, unsigned int* status);

// ---- gated delta net (ops_gdn.cu) ----
void k_conv1d_ssm(cudaStream_t st, const uint16_t* x, const uint16_t* w, uint16_t* y, uint32_t seq,
                  uint32_t C, uint32_t k);
void k_conv1d_step(cudaStream_t st, const uint16_t* x, const uint16_t* w, uint16_t* y, float* win,
                   uint32_t C, uint32_t dc);
// Tensor-core form of the chunked delta rule (gdn_delta_mma.cu): head dim 64 or 128. false: shape not taken.
bool k_delta_chunk_mma(cudaStream_t st, const uint16_t* k, const uint16_t* v, const uint16_t* q, const uint16_t* beta,
                       const uint16_t* g, uint16_t* y, float* S, uint32_t c, uint32_t ntok, uint32_t H, uint32_t D, uint32_t q_raw);
void k_delta_chunk(cudaStream_t st, const uint16_t* k, const uint16_t* v, const uint16_t* q,
                   const uint16_t* beta, const uint16_t* g, uint16_t* y, float* S, uint32_t c,
                   uint32_t ntok, uint32_t H, uint32_t D, uint32_t q_raw);

}  // namespace gehtp
