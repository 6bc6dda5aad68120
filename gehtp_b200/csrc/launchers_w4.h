// W4A16 launchers and the epilogue descriptor shared by the W4A16 kernels.
#pragma once
#include <cuda_fp16.h>
#include "launchers.h"

namespace gehtp {

// What happens to an fp32 accumulator on its way to memory.
//   mode 0: y = f16(acc)
//   mode 1: y = f16( f16(acc) + res )          (matmul followed by a residual ADD op;
//           both fp16 roundings of the two-op form are kept)
//   mode 2: the matmul is the fused q|k|v projection of a decode step (head_dim 128): the rotary
//           embedding is applied to the q and k heads with the rounding points of the op chain
//           (matmul output -> fp16, x*cos -> fp16, rot(x)*sin -> fp16, sum -> fp16), q goes to
//           q_out, k and v go straight into the KV ring slot of the position (SPLIT x3 + rotary
//           chain x2 + KV_APPEND of the runlist). Streaming kernel only, M <= 8.
//   mode 3: the matmul is followed by a residual ADD and an RMSNORM2 (tcgen05 GEMM only): y = f16(acc) as in
//           mode 0, sum_out = f16(y + res), norm_out = rmsnorm(sum_out) * gamma + beta with the roundings of the
//           two ops. With K split into runs the kernel that adds the runs also adds the residual and normalises
//           (one CTA per row); otherwise the add + norm kernel is launched behind the GEMM.
struct W4Epilogue {
    int mode = 0;
    const uint16_t* res = nullptr;
    // mode 3
    const uint16_t *gamma = nullptr, *beta = nullptr;
    uint16_t *sum_out = nullptr, *norm_out = nullptr;
    unsigned int* status = nullptr;   // engine status word: the tcgen05 GEMM reports a barrier wait that ran out here
    // mode 2
    const uint16_t *cos_q = nullptr, *sin_q = nullptr, *cos_k = nullptr, *sin_k = nullptr;   // [M*heads][hd]
    uint16_t *q_out = nullptr, *ring = nullptr;
    uint32_t* posmap = nullptr;
    const uint32_t* counter = nullptr;
    uint32_t nh = 0, kvh = 0, nslots = 0, pos_const = 0;
};

#ifdef __CUDACC__
__device__ __forceinline__ void w4_store(const W4Epilogue& ep, uint16_t* y, uint32_t m, uint32_t n,
                                         uint32_t N, float acc) {
    const size_t o = (size_t)m * N + n;
    uint16_t h = __half_as_ushort(__float2half_rn(acc));
    if (acc != acc) h = (uint16_t)(((__float_as_uint(acc) >> 16) & 0x8000u) | 0x7c00u);
    if (ep.mode == 1) {
        float s = __fadd_rn(__half2float(__ushort_as_half(h)),
                            __half2float(__ushort_as_half(ep.res[o])));
        h = __half_as_ushort(__float2half_rn(s));
        if (s != s) h = (uint16_t)(((__float_as_uint(s) >> 16) & 0x8000u) | 0x7c00u);
    }
    y[o] = h;
}
#endif

// nib: slot nibbles [K][N/2]; packed: K*N/2 bytes in the strip-major layout.
void k_w4_repack(cudaStream_t st, const uint8_t* nib, uint32_t* packed, uint32_t K, uint32_t N);
void k_w4_unpack_i8(cudaStream_t st, const uint32_t* packed, int8_t* out, uint32_t K, uint32_t N);
// Streaming form, any M (intended for M <= 16; larger M re-reads the weights
// from L2 once per 16 rows).
void k_w4a16_skinny(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                    uint16_t* y, uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep);
// The q|k|v projection with rotary embedding and KV append in the epilogue (ep.mode == 2, head_dim 128).
// false: shape not handled (M > 8, K not a multiple of 512 or above 5120, N != (nh + 2 kvh) * 128).
bool k_w4a16_skinny_qkv_rope(cudaStream_t st, const uint16_t* a, const uint32_t* packed, const uint16_t* sc,
                             uint32_t M, uint32_t K, uint32_t N, const W4Epilogue& ep);
// Gate and up projections with the SwiGLU product in the epilogue (one pass over both matrices).
void k_w4a16_skinny_swiglu(cudaStream_t st, const uint16_t* a, const uint32_t* pg, const uint16_t* sg,
                           const uint32_t* pu, const uint16_t* su, uint16_t* y, uint32_t M, uint32_t K,
                           uint32_t N);
// tcgen05 / TMEM form for M >= 128 (w4a16_gemm_sm100.cu). Returns false when
// the shape is outside what it handles (the caller then uses the skinny form).
// `tile`: 0 = chosen from the shape, 1 = 128x128, 2 = 256x128, 3 = 256x256 (N % 256 == 0).
// `a_d` != 0: the activations are stored [K / a_d][M][a_d] (a_d a multiple of 64 that divides K) - the output of a
// per-head kernel, read through a three-dimensional tensor map without the transposition to [M][K].
bool k_w4a16_gemm_sm100(cudaStream_t st, const uint16_t* a, const uint32_t* packed,
                        const uint16_t* sc, uint16_t* y, uint32_t M, uint32_t K, uint32_t N,
                        const W4Epilogue& ep, int tile = 0, uint32_t a_d = 0);
// Gate and up projections of a gated FFN plus its three elementwise ops on the same kernel: y[M, N] =
// fp16(fp16(g * fp16(sigmoid(g))) * u), g = a . Wg, u = a . Wu (both [K, N]), neither g nor u written to memory.
// `takes`: the shape test alone (N a multiple of 128, K of 64); the launcher also wants
// 16-byte aligned operands. false: nothing launched.
bool w4a16_gemm_sm100_swiglu_takes(uint32_t M, uint32_t K, uint32_t N);
bool k_w4a16_gemm_sm100_swiglu(cudaStream_t st, const uint16_t* a, const uint32_t* pg, const uint16_t* sg, const uint32_t* pu,
                               const uint16_t* su, uint16_t* y, uint32_t M, uint32_t K, uint32_t N, unsigned int* status);

}  // namespace gehtp
