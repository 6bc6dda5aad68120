// Host-pointer entry points around single kernels (tests, small tools): each
// stages its operands on the device, runs the kernel the engine uses, and
// copies the result back.
#include <cstdio>
#include <vector>
#include "engine.h"
#include "launchers_attn.h"

using namespace gehtp;

namespace {
struct DevBuf {
    void* p = nullptr;
    explicit DevBuf(size_t n) { if (cudaMalloc(&p, n ? n : 16) != cudaSuccess) p = nullptr; }
    ~DevBuf() { if (p) cudaFree(p); }
    template <class T> T* as() { return (T*)p; }
};
int fail(const char* m) { g.last_error = m; return -1; }
int finish(const char* what) {
    cudaError_t e = cudaStreamSynchronize(g.stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { g.last_error = std::string(what) + ": " + cudaGetErrorString(e); return -1; }
    return 0;
}
}  // namespace

extern "C" {

int gehtp_w4a16_matmul(const uint16_t* a_f16, const uint8_t* w_slot, uint16_t* y_f16, uint32_t M,
                       uint32_t K, uint32_t N, int path) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!M || !K || !N || K % 64 || N % 16) return fail("w4a16 shape");
    size_t nb = (size_t)K * N / 2, sb = gehtp_w4a16_slot_bytes(K, N);
    DevBuf da((size_t)M * K * 2), dslot(sb), dpk(nb), dy((size_t)M * N * 2);
    if (!da.p || !dslot.p || !dpk.p || !dy.p) return fail("device alloc");
    cudaMemcpyAsync(da.p, a_f16, (size_t)M * K * 2, cudaMemcpyHostToDevice, g.stream);
    cudaMemcpyAsync(dslot.p, w_slot, sb, cudaMemcpyHostToDevice, g.stream);
    k_w4_repack(g.stream, dslot.as<uint8_t>(), dpk.as<uint32_t>(), K, N);
    const uint16_t* sc = (const uint16_t*)(dslot.as<uint8_t>() + nb);
    W4Epilogue ep;
    ep.status = g.d_status;
    bool done = false;
    if (path >= 2 || (path == 0 && M >= 128)) {   // 2: tile by shape; 3, 4, 5: 128x128, 256x128, 256x256 tiles
        done = k_w4a16_gemm_sm100(g.stream, da.as<uint16_t>(), dpk.as<uint32_t>(), sc, dy.as<uint16_t>(), M, K, N, ep, path >= 3 ? path - 2 : 0);
        if (!done && path >= 2) return fail("tcgen05 GEMM does not take this shape");
    }
    if (!done) k_w4a16_skinny(g.stream, da.as<uint16_t>(), dpk.as<uint32_t>(), sc, dy.as<uint16_t>(), M, K, N, ep);
    cudaMemcpyAsync(y_f16, dy.p, (size_t)M * N * 2, cudaMemcpyDeviceToHost, g.stream);
    if (finish("w4a16 matmul")) return -1;
    return read_status(nullptr, 0) ? -1 : 0;
}

int gehtp_w4a16_unpack(const uint8_t* w_slot, int8_t* out_i8, uint32_t K, uint32_t N) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!K || !N || K % 64 || N % 16) return fail("w4a16 shape");
    size_t nb = (size_t)K * N / 2;
    DevBuf dslot(nb), dpk(nb), dout((size_t)K * N);
    if (!dslot.p || !dpk.p || !dout.p) return fail("device alloc");
    cudaMemcpyAsync(dslot.p, w_slot, nb, cudaMemcpyHostToDevice, g.stream);
    k_w4_repack(g.stream, dslot.as<uint8_t>(), dpk.as<uint32_t>(), K, N);
    k_w4_unpack_i8(g.stream, dpk.as<uint32_t>(), dout.as<int8_t>(), K, N);
    cudaMemcpyAsync(out_i8, dout.p, (size_t)K * N, cudaMemcpyDeviceToHost, g.stream);
    return finish("w4a16 unpack");
}

int gehtp_rmsnorm(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, uint16_t* y,
                  uint32_t rows, uint32_t width) {
    if (!ensure_device(nullptr, 0)) return -1;
    size_t n = (size_t)rows * width * 2;
    DevBuf dx(n), dg((size_t)width * 2), db((size_t)width * 2), dy(n);
    if (!dx.p || !dg.p || !db.p || !dy.p) return fail("device alloc");
    cudaMemcpyAsync(dx.p, x, n, cudaMemcpyHostToDevice, g.stream);
    cudaMemcpyAsync(dg.p, gamma, (size_t)width * 2, cudaMemcpyHostToDevice, g.stream);
    if (beta) cudaMemcpyAsync(db.p, beta, (size_t)width * 2, cudaMemcpyHostToDevice, g.stream);
    k_rmsnorm(g.stream, dx.as<uint16_t>(), dg.as<uint16_t>(), beta ? db.as<uint16_t>() : nullptr, dy.as<uint16_t>(), rows, width);
    cudaMemcpyAsync(y, dy.p, n, cudaMemcpyDeviceToHost, g.stream);
    return finish("rmsnorm");
}

int gehtp_attn_decode(const uint16_t* q, const uint16_t* kv_ring, const uint16_t* mask, uint16_t* out,
                      uint32_t n_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t n_kv,
                      uint32_t nslots, float scale) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!n_heads || !kv_heads || n_heads % kv_heads || !nslots || n_kv > nslots) return fail("attn shape");
    uint32_t rep = n_heads / kv_heads;
    size_t ring_b = (size_t)nslots * kv_heads * head_dim * 4, q_b = (size_t)n_heads * head_dim * 2;
    uint32_t nsplit = attn_decode_nsplit(kv_heads, n_kv, rep, head_dim, 0);
    size_t scr = attn_decode_scratch_floats(kv_heads, rep, head_dim, nsplit);
    DevBuf dq(q_b), dr(ring_b), dm((size_t)n_kv * 2), dout(q_b), dscr(scr * 4);
    if (!dq.p || !dr.p || !dm.p || !dout.p || !dscr.p) return fail("device alloc");
    cudaMemcpyAsync(dq.p, q, q_b, cudaMemcpyHostToDevice, g.stream);
    cudaMemcpyAsync(dr.p, kv_ring, ring_b, cudaMemcpyHostToDevice, g.stream);
    if (mask) cudaMemcpyAsync(dm.p, mask, (size_t)n_kv * 2, cudaMemcpyHostToDevice, g.stream);
    AttnDecodeArgs a{};
    a.status = g.d_status;
    a.q = dq.as<uint16_t>(); a.ring = dr.as<uint16_t>(); a.counter = nullptr; a.n_kv = n_kv; a.n_kv_add = 0; a.bump_counter = nullptr;
    a.mask = mask ? dm.as<uint16_t>() : nullptr; a.mask_seq_stride = 0; a.kvh_per_seq = kv_heads;
    a.scale = scale; a.scale_div = 0; a.rep = rep; a.kv_heads = kv_heads; a.nslots = nslots; a.nsplit = nsplit;
    a.part_o = dscr.as<float>();
    a.part_ml = a.part_o + (size_t)kv_heads * nsplit * rep * head_dim;
    if (!k_attn_decode(g.stream, a, head_dim, dout.as<uint16_t>(), kv_heads)) return fail("attn shape not handled by the fused kernel");
    cudaMemcpyAsync(out, dout.p, q_b, cudaMemcpyDeviceToHost, g.stream);
    if (finish("attn decode")) return -1;
    return read_status(nullptr, 0) ? -1 : 0;
}

}  // extern "C"

// ---- device-pointer entry points: the caller owns every buffer (device
// memory) and the work is queued on the engine stream without waiting. Used by
// the bench to time single kernels with inputs resident in HBM.
extern "C" {

int gehtp_dev_w4_repack(const uint8_t* slot_dev, uint32_t* packed_dev, uint32_t K, uint32_t N) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!K || !N || K % 64 || N % 16) return fail("w4a16 shape");
    k_w4_repack(g.stream, slot_dev, packed_dev, K, N);
    return 0;
}

// path: 0 = engine's choice by M, 1 = streaming kernel, 2 = tcgen05 GEMM (tile by shape), 3 / 4 / 5 = tcgen05 GEMM
// with 128x128 / 256x128 / 256x256 tiles
int gehtp_dev_w4a16_matmul(const uint16_t* a_dev, const uint32_t* packed_dev, const uint16_t* scales_dev,
                           uint16_t* y_dev, uint32_t M, uint32_t K, uint32_t N, int path) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!M || !K || !N || K % 64 || N % 16) return fail("w4a16 shape");
    W4Epilogue ep;
    ep.status = g.d_status;
    if (path >= 2 || (path == 0 && M >= 128)) {
        if (k_w4a16_gemm_sm100(g.stream, a_dev, packed_dev, scales_dev, y_dev, M, K, N, ep, path >= 3 ? path - 2 : 0)) return 0;
        if (path >= 2) return fail("tcgen05 GEMM does not take this shape");
    }
    k_w4a16_skinny(g.stream, a_dev, packed_dev, scales_dev, y_dev, M, K, N, ep);
    return 0;
}

// y[M, N] = a[M, K] . w^T with w stored [N, K] (fp16): tcgen05 GEMM for M >= 128, streaming GEMV for M < 32
int gehtp_dev_matmul_f16_nk(const uint16_t* a_dev, const uint16_t* w_dev, uint16_t* y_dev, uint32_t M, uint32_t K, uint32_t N) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!k_matmul_f16_nk(g.stream, a_dev, w_dev, y_dev, M, K, N, N, g.d_status)) return fail("matmul_f16 [N,K]: shape not taken by the tensor-core forms");
    return 0;
}

int gehtp_dev_w4a16_swiglu(const uint16_t* a_dev, const uint32_t* pg, const uint16_t* sg, const uint32_t* pu,
                           const uint16_t* su, uint16_t* y_dev, uint32_t M, uint32_t K, uint32_t N) {
    if (!ensure_device(nullptr, 0)) return -1;
    if (!M || !K || !N || K % 64 || N % 16) return fail("w4a16 shape");
    if (M >= w4_gemm_min_rows()) {       // the engine's rule: the tcgen05 gate | up GEMM from this many rows
        if (k_w4a16_gemm_sm100_swiglu(g.stream, a_dev, pg, sg, pu, su, y_dev, M, K, N, g.d_status)) return 0;
        return fail("w4a16 swiglu: shape not taken by the tcgen05 form");
    }
    if (M > 16) return fail("w4a16 swiglu: more than 16 rows below the GEMM's row count");
    k_w4a16_skinny_swiglu(g.stream, a_dev, pg, sg, pu, su, y_dev, M, K, N);
    return 0;
}

int gehtp_dev_rmsnorm(const uint16_t* x_dev, const uint16_t* res_dev, const uint16_t* gamma_dev, const uint16_t* beta_dev,
                      uint16_t* sum_dev, uint16_t* y_dev, uint32_t rows, uint32_t width) {
    if (!ensure_device(nullptr, 0)) return -1;
    k_add_rmsnorm(g.stream, x_dev, res_dev, gamma_dev, beta_dev, sum_dev, y_dev, rows, width);
    return 0;
}

}  // extern "C"
