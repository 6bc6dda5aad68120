// Shared device helpers: fp16 <-> fp32 with the reference's rounding rules.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdlib>

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

// Codes a kernel leaves in the engine's status word when one of its bounded waits
// runs out (bit 31 set); any other non-zero value is the 1-based index of an op
// whose KV gather found a ring slot that holds another position. The host turns
// the word into the run's error return (status_message, executor.cu).
constexpr unsigned int kStatusAllReduceTimeout = 0x80000001u;   // peer-memory all-reduce: a rank never wrote
constexpr unsigned int kStatusAttnTimeout = 0x80000002u;        // decode attention: a K/V tile copy never arrived
constexpr unsigned int kStatusGemmTimeout = 0x80000003u;        // tcgen05 GEMM: a pipeline barrier never completed

// Device status word: first failing op (1-based) wins.
__device__ __forceinline__ void raise_status(unsigned int* status, unsigned int code) {
    if (status) atomicCAS(status, 0u, code);
}

// cudaFuncSetAttribute is per device: remembers, per device ordinal, the largest
// dynamic shared-memory size a kernel has been opted into, and raises it when needed.
template <typename K>
inline bool ensure_dyn_smem(K kernel, size_t bytes, int (&have)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if ((size_t)have[dev] >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    have[dev] = (int)bytes;
    return true;
}

// Launch with programmatic dependent launch allowed: the grid may start while
// its predecessor in the stream is still running; the kernel orders itself
// after the predecessor with griddepcontrol.wait before it touches anything the
// predecessor wrote (and writes nothing before that point).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    // $GEHTP_CUDA_PDL=0 makes every launch wait for the whole previous kernel (for bisecting ordering faults)
    static const int pdl = [] { const char* e = std::getenv("GEHTP_CUDA_PDL"); return e ? std::atoi(e) : 1; }();
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace gehtp
