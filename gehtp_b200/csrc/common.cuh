// Shared device helpers: fp16 <-> fp32 with the reference's rounding rules.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gehtp {

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// fp32 -> fp16, round to nearest even including subnormals. NaN becomes a
// signed infinity, as the reference's converter does (oplist_exec.c:395-418).
__device__ __forceinline__ uint16_t f2h(float f) {
    if (f != f) return (uint16_t)(((__float_as_uint(f) >> 16) & 0x8000u) | 0x7c00u);
    return __half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Device status word: first failing op (1-based) wins.
__device__ __forceinline__ void raise_status(unsigned int* status, unsigned int code) {
    if (status) atomicCAS(status, 0u, code);
}

}  // namespace gehtp
