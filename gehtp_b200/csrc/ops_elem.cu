// Elementwise and data-movement ops of the runlist: fp16 faces in, fp32 math,
// one fp16 rounding at each op's output. Compiled with --fmad=false so that
// multiply-then-add keeps the two roundings the reference's scalar code has.
// Every kernel cites the reference routine whose results it reproduces
// (all in kernels/src/runtime/oplist_exec.c).
#include "common.cuh"
#include "launchers.h"

namespace gehtp {

unsigned long long g_launches = 0;

static inline unsigned grid_for(size_t n, unsigned block, unsigned cap = 148u * 16u) {
    size_t g = (n + block - 1) / block;
    if (g < 1) g = 1;
    return (unsigned)(g > cap ? cap : g);
}

// ---------------------------------------------------------------- unary
// exec_unary, oplist_exec.c:1013-1079 (subtype table at oplist_parse.h:117).
__device__ __forceinline__ float unary_apply(float v, uint32_t subtype) {
    switch (subtype) {
    case 0: return -v;
    case 1: return expf(v);
    case 2: return (v >= 0) ? sqrtf(v) : 0.0f;
    case 3: return (v > 0) ? 1.0f / sqrtf(v) : 0.0f;
    case 4: return (v > 0) ? logf(v) : 0.0f;
    case 5: return fabsf(v);
    case 6: return sinf(v);
    case 7: return cosf(v);
    case 8: return 1.0f / (1.0f + expf(-v));
    case 9: return tanhf(v);
    case 10: return 0.5f * v * (1.0f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v)));
    case 11: return fmaxf(0.0f, v);
    case 12: return v / (1.0f + expf(-v));
    case 13: return (v > 30.0f) ? v : (v < -30.0f ? expf(v) : log1pf(expf(v)));
    case 15: return (v != v) ? 1.0f : 0.0f;
    case 16: return (v == v && (v > 3.4e38f || v < -3.4e38f)) ? 1.0f : 0.0f;
    default: return v;  // 14 = copy
    }
}

__global__ void unary_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, uint32_t n,
                             uint32_t subtype) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        y[i] = f2h(unary_apply(h2f(x[i]), subtype));
}

void k_unary(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t subtype) {
    if (!n) return;
    launch_pdl(unary_kernel, dim3(grid_for(n, 256)), dim3(256), 0, st, x, y, n, subtype);
    g_launches++;
}

// ---------------------------------------------------------------- binary
// exec_binary / exec_add, oplist_exec.c:807-829, 1081-1161. guard_div selects
// the scalar form of DIV (x/0 -> 0) that the reference uses for n < 32.
__global__ void binary_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                              uint16_t* __restrict__ y, uint32_t n, uint32_t subtype,
                              int guard_div) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float x0 = h2f(a[i]), x1 = h2f(b[i]), r = x0;
        switch (subtype) {
        case 0: r = x0 + x1; break;
        case 1: r = x0 - x1; break;
        case 2: r = x0 * x1; break;
        case 3: r = guard_div ? ((x1 != 0) ? x0 / x1 : 0.0f) : x0 / x1; break;
        case 4: r = (x0 == x1) ? 1.0f : 0.0f; break;
        case 5: r = ((uint32_t)x0 & (uint32_t)x1) ? 1.0f : 0.0f; break;
        default: break;
        }
        y[i] = f2h(r);
    }
}

void k_binary(cudaStream_t st, const uint16_t* a, const uint16_t* b, uint16_t* y, uint32_t n,
              uint32_t subtype, bool guard_div) {
    if (!n) return;
    launch_pdl(binary_kernel, dim3(grid_for(n, 256)), dim3(256), 0, st, a, b, y, n, subtype, guard_div ? 1 : 0);
    g_launches++;
}

// SELECT form of opcode 12 (oplist_exec.c:1085-1111): each source is a scalar,
// a tile repeated modulo its length, or full size.
__global__ void select_kernel(const uint16_t* __restrict__ c, uint32_t cn,
                              const uint16_t* __restrict__ t, uint32_t tn,
                              const uint16_t* __restrict__ f, uint32_t fn,
                              uint16_t* __restrict__ y, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float cv = h2f(c[cn <= 1u ? 0 : (cn < n ? i % cn : i)]);
        float r = (cv != 0.0f) ? h2f(t[tn <= 1u ? 0 : (tn < n ? i % tn : i)])
                               : h2f(f[fn <= 1u ? 0 : (fn < n ? i % fn : i)]);
        y[i] = f2h(r);
    }
}

void k_select(cudaStream_t st, const uint16_t* c, uint32_t cn, const uint16_t* t, uint32_t tn,
              const uint16_t* f, uint32_t fn, uint16_t* y, uint32_t n) {
    select_kernel<<<grid_for(n, 256), 256, 0, st>>>(c, cn, t, tn, f, fn, y, n);
    g_launches++;
}

// ---------------------------------------------------------------- byte moves
__global__ void copy16_kernel(const uint4* __restrict__ s, uint4* __restrict__ d, size_t n16) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
         i += (size_t)gridDim.x * blockDim.x)
        d[i] = s[i];
}
__global__ void copy1_kernel(const uint8_t* __restrict__ s, uint8_t* __restrict__ d, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        d[i] = s[i];
}

void k_copy_bytes(cudaStream_t st, const void* src, void* dst, size_t bytes) {
    if (!bytes || src == dst) return;
    if ((((uintptr_t)src | (uintptr_t)dst | bytes) & 15u) == 0)
        launch_pdl(copy16_kernel, dim3(grid_for(bytes / 16, 256)), dim3(256), 0, st, (const uint4*)src, (uint4*)dst,
                                                                bytes / 16);
    else
        copy1_kernel<<<grid_for(bytes, 256), 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst,
                                                          bytes);
    g_launches++;
}

__global__ void fill16_kernel(uint16_t* d, size_t n, uint16_t v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        d[i] = v;
}
void k_fill16(cudaStream_t st, uint16_t* dst, size_t n, uint16_t v) {
    if (!n) return;
    fill16_kernel<<<grid_for(n, 256), 256, 0, st>>>(dst, n, v);
    g_launches++;
}

// Concat along the flattened "axis" (oplist_exec.c:1196-1220): segment rows of
// width `seg` go to columns [start, start+seg) of rows of width total_axis.
__global__ void rows_move_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                 uint32_t outer, uint32_t seg, uint32_t xs, uint32_t xo,
                                 uint32_t ys, uint32_t yo) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    size_t total = (size_t)outer * seg;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        uint32_t o = (uint32_t)(i / seg), j = (uint32_t)(i % seg);
        y[(size_t)o * ys + yo + j] = x[(size_t)o * xs + xo + j];
    }
}
void k_concat_seg(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t seg,
                  uint32_t total_axis, uint32_t start) {
    if (!outer || !seg) return;
    launch_pdl(rows_move_kernel, dim3(grid_for((size_t)outer * seg, 256)), dim3(256), 0, st, x, y, outer, seg, seg, 0,
                                                                       total_axis, start);
    g_launches++;
}
// Split = the inverse (oplist_exec.c:1222-1256).
void k_split_seg(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t seg,
                 uint32_t total_axis, uint32_t off) {
    if (!outer || !seg) return;
    launch_pdl(rows_move_kernel, dim3(grid_for((size_t)outer * seg, 256)), dim3(256), 0, st, x, y, outer, seg,
                                                                       total_axis, off, seg, 0);
    g_launches++;
}

struct U4 { uint32_t v[4]; };
struct U5 { uint32_t v[5]; };

// Strided slice, rank <= 3 (oplist_exec.c:1950-1988).
__global__ void slice_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                             uint32_t n_out, uint32_t rk, U4 b, U4 s, U4 istr, U4 ostr) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_out;
         i += gridDim.x * blockDim.x) {
        uint32_t rem = i, in_lin = 0;
        for (uint32_t ax = 0; ax < rk; ax++) {
            uint32_t c = rem / ostr.v[ax];
            rem %= ostr.v[ax];
            in_lin += (b.v[ax] + c * s.v[ax]) * istr.v[ax];
        }
        y[i] = x[in_lin];
    }
}
void k_slice(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n_out, uint32_t rk,
             const uint32_t* b3, const uint32_t* s3, const uint32_t* istr3, const uint32_t* ostr3) {
    if (!n_out) return;
    U4 b{}, s{}, is{}, os{};
    for (uint32_t i = 0; i < 3; i++) { b.v[i] = b3[i]; s.v[i] = s3[i]; is.v[i] = istr3[i]; os.v[i] = ostr3[i]; }
    launch_pdl(slice_kernel, dim3(grid_for(n_out, 256)), dim3(256), 0, st, x, y, n_out, rk, b, s, is, os);
    g_launches++;
}

// numpy-style broadcast, right aligned (oplist_exec.c:1876-1907).
__global__ void broadcast_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                 uint32_t n, uint32_t r, uint32_t lead, U4 in_d, U4 istr, U4 ostr) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t rem = i, in_lin = 0;
        for (uint32_t d = 0; d < r; d++) {
            uint32_t c = rem / ostr.v[d];
            rem %= ostr.v[d];
            if (d < lead) continue;
            uint32_t idim = in_d.v[d - lead];
            if (idim > 1) in_lin += (c % idim) * istr.v[d - lead];
        }
        y[i] = x[in_lin];
    }
}
void k_broadcast(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t r,
                 uint32_t lead, const uint32_t* in_d4, const uint32_t* istr4, const uint32_t* ostr4) {
    if (!n) return;
    U4 d{}, is{}, os{};
    for (uint32_t i = 0; i < 4; i++) { d.v[i] = in_d4[i]; is.v[i] = istr4[i]; os.v[i] = ostr4[i]; }
    launch_pdl(broadcast_kernel, dim3(grid_for(n, 256)), dim3(256), 0, st, x, y, n, r, lead, d, is, os);
    g_launches++;
}

// General N-D transpose, rank 2..4 (oplist_exec.c:1910-1948).
__global__ void transpose_gen_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                     uint32_t n, uint32_t rk, U4 si, U4 so, U4 p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
        uint32_t rem = t, ic[4] = {0, 0, 0, 0};
        for (uint32_t i = 0; i < rk; i++) { ic[i] = rem / si.v[i]; rem %= si.v[i]; }
        uint32_t ot = 0;
        for (uint32_t ax = 0; ax < rk; ax++) ot += ic[p.v[ax] & 3u] * so.v[ax];
        y[ot] = x[t];
    }
}
void k_transpose_gen(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t n, uint32_t rk,
                     const uint32_t* si4, const uint32_t* so4, const uint32_t* perm4) {
    if (!n) return;
    U4 si{}, so{}, p{};
    for (uint32_t i = 0; i < 4; i++) { si.v[i] = si4[i]; so.v[i] = so4[i]; p.v[i] = perm4[i]; }
    launch_pdl(transpose_gen_kernel, dim3(grid_for(n, 256)), dim3(256), 0, st, x, y, n, rk, si, so, p);
    g_launches++;
}

// Legacy 4-D transpose with N = 1 (oplist_exec.c:983-1009): output-major walk.
__global__ void transpose_hwc_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                     uint32_t H, uint32_t W, uint32_t C, U4 p) {
    uint32_t dims[4] = {1, H, W, C};
    uint32_t sin[4] = {H * W * C, W * C, C, 1};
    uint32_t od[4] = {dims[p.v[0]], dims[p.v[1]], dims[p.v[2]], dims[p.v[3]]};
    uint32_t n = H * W * C;
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < n; o += gridDim.x * blockDim.x) {
        uint32_t rem = o, oc[4];
        oc[3] = rem % od[3]; rem /= od[3];
        oc[2] = rem % od[2]; rem /= od[2];
        oc[1] = rem % od[1]; rem /= od[1];
        oc[0] = rem;
        uint32_t src = 0;
        for (int ax = 0; ax < 4; ax++) src += oc[ax] * sin[p.v[ax]];
        y[o] = x[src];
    }
}
void k_transpose_hwc(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t H, uint32_t W,
                     uint32_t C, uint32_t perm) {
    U4 p{{perm & 3u, (perm >> 8) & 3u, (perm >> 16) & 3u, (perm >> 24) & 3u}};
    transpose_hwc_kernel<<<grid_for((size_t)H * W * C, 256), 256, 0, st>>>(x, y, H, W, C, p);
    g_launches++;
}

// Single-axis reduce (oplist_exec.c:1258-1299): sequential fp32 accumulation
// along the axis per output element, so sums match the reference bit for bit.
__global__ void reduce_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                              uint32_t outer, uint32_t L, uint32_t inner, uint32_t subtype) {
    size_t total = (size_t)outer * inner;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        uint32_t o = (uint32_t)(e / inner), i = (uint32_t)(e % inner);
        const uint16_t* base = x + ((size_t)o * L) * inner + i;
        float acc = (subtype == 2) ? -3.0e38f : (subtype == 3) ? 3.0e38f : 0.0f;
        for (uint32_t l = 0; l < L; l++) {
            float v = h2f(base[(size_t)l * inner]);
            if (subtype == 2) acc = v > acc ? v : acc;
            else if (subtype == 3) acc = v < acc ? v : acc;
            else acc += v;
        }
        if (subtype == 1) acc /= (float)L;
        y[e] = f2h(acc);
    }
}
// Max / min over a long contiguous axis (inner == 1): one CTA per output. The
// sequential scan keeps the first of equal candidates (it matters for +0 / -0),
// so candidates carry their position and ties go to the smaller one.
__global__ void __launch_bounds__(256)
reduce_minmax_row_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, uint32_t L, int is_max) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    const uint16_t* row = x + (size_t)blockIdx.x * L;
    float best = is_max ? -3.0e38f : 3.0e38f;
    uint32_t bi = 0xffffffffu;
    auto take = [&](uint16_t h, uint32_t l) {
        const float v = h2f(h);
        if (is_max ? v > best : v < best) { best = v; bi = l; }
    };
    // unaligned head, 16-byte body (ascending positions per thread), tail
    uint32_t head = (uint32_t)((16 - ((uintptr_t)row & 15)) & 15) / 2;
    if (head > L) head = L;
    const uint32_t nvec = (L - head) / 8;
    if (threadIdx.x < head) take(row[threadIdx.x], threadIdx.x);
    const uint4* rv = (const uint4*)(row + head);
    for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 q = __ldg(rv + v);
        const uint16_t* h = (const uint16_t*)&q;
#pragma unroll
        for (int i = 0; i < 8; i++) take(h[i], head + v * 8 + i);
    }
    for (uint32_t l = head + nvec * 8 + threadIdx.x; l < L; l += blockDim.x) take(row[l], l);
    auto better = [&](float v, uint32_t i, float w, uint32_t j) {   // is (v,i) ahead of (w,j)?
        return (is_max ? v > w : v < w) || (v == w && i < j);
    };
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(v, i, best, bi)) { best = v; bi = i; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (better(sv[w], si[w], best, bi)) { best = sv[w]; bi = si[w]; }
        y[blockIdx.x] = f2h(best);
    }
}

void k_reduce(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t L,
              uint32_t inner, uint32_t subtype) {
    if (inner == 1 && L >= 1024 && (subtype == 2 || subtype == 3)) {
        reduce_minmax_row_kernel<<<outer, 256, 0, st>>>(x, y, L, subtype == 2);
        g_launches++;
        return;
    }
    reduce_kernel<<<grid_for((size_t)outer * inner, 128), 128, 0, st>>>(x, y, outer, L, inner,
                                                                      subtype);
    g_launches++;
}

// Constant pad of the innermost flattened dim (oplist_exec.c:1301-1318).
__global__ void pad_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                           uint32_t outer, uint32_t in_inner, uint32_t out_inner,
                           uint32_t pad_before, uint16_t pv) {
    size_t total = (size_t)outer * out_inner;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        uint32_t o = (uint32_t)(e / out_inner), j = (uint32_t)(e % out_inner);
        y[e] = (j >= pad_before && j < pad_before + in_inner)
                   ? x[(size_t)o * in_inner + (j - pad_before)] : pv;
    }
}
void k_pad(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t outer, uint32_t in_inner,
           uint32_t out_inner, uint32_t pad_before, uint16_t pv) {
    if (!outer || !out_inner) return;
    pad_kernel<<<grid_for((size_t)outer * out_inner, 256), 256, 0, st>>>(x, y, outer, in_inner,
                                                                       out_inner, pad_before, pv);
    g_launches++;
}

// Row cumsum (oplist_exec.c:1320-1347): one thread per row, sequential, so
// every partial sum rounds as in the reference.
__global__ void cumsum_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                              uint32_t rows, uint32_t n, uint32_t exclusive, uint32_t reverse) {
    uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float acc = 0.0f;
    for (uint32_t s = 0; s < n; s++) {
        uint32_t i = reverse ? (n - 1 - s) : s;
        size_t idx = (size_t)r * n + i;
        float v = h2f(x[idx]);
        y[idx] = f2h(exclusive ? acc : acc + v);
        acc += v;
    }
}
void k_cumsum(cudaStream_t st, const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n,
              uint32_t exclusive, uint32_t reverse) {
    if (!rows || !n) return;
    cumsum_kernel<<<(rows + 63) / 64, 64, 0, st>>>(x, y, rows, n, exclusive, reverse);
    g_launches++;
}

// Gather along one axis with an index tensor of rank xrank (oplist_exec.c:1378-1432).
__global__ void gather_kernel(const uint16_t* __restrict__ tbl, const int32_t* __restrict__ idx,
                              uint16_t* __restrict__ y, uint32_t n, uint32_t axis, uint32_t xrank,
                              uint32_t irank, U5 td, U5 xd, U5 os, U5 ts, U5 xs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t rem = i, oc[5];
        for (int d = 0; d < 5; d++) { oc[d] = rem / os.v[d]; rem %= os.v[d]; }
        uint32_t il = 0;
        for (uint32_t k = 0; k < xrank && k < 5 && axis + k < 5; k++) il += (oc[axis + k] % xd.v[k]) * xs.v[k];
        int32_t r = idx[il];
        if (r < 0) r += (int32_t)td.v[axis];
        if (r < 0 || r >= (int32_t)td.v[axis]) { y[i] = 0; continue; }
        size_t src = 0;
        for (uint32_t d = 0; d < axis && d < 5; d++) src += (size_t)oc[d] * ts.v[d];
        src += (size_t)r * ts.v[axis];
        for (uint32_t d = axis + 1; d < irank && d < 5; d++) {
            uint32_t ocd = d + xrank - 1;
            src += (size_t)(ocd < 5 ? oc[ocd] : 0) * ts.v[d];
        }
        y[i] = tbl[src];
    }
}
void k_gather(cudaStream_t st, const uint16_t* tbl, const int32_t* idx, uint16_t* y, uint32_t n,
              uint32_t axis, uint32_t xrank, uint32_t irank, const uint32_t* td5,
              const uint32_t* xd5) {
    if (!n) return;
    U5 td, xd, od, os, ts, xs;
    for (int i = 0; i < 5; i++) { td.v[i] = td5[i]; xd.v[i] = xd5[i]; od.v[i] = 1; }
    for (uint32_t d = 0; d < axis && d < 5; d++) od.v[d] = td.v[d];
    for (uint32_t k = 0; k < xrank && axis + k < 5; k++) od.v[axis + k] = xd.v[k];
    for (uint32_t d = axis + 1; d < irank && d < 5; d++) {
        uint32_t ocd = d + xrank - 1;
        if (ocd < 5) od.v[ocd] = td.v[d];
    }
    os.v[4] = ts.v[4] = xs.v[4] = 1;
    for (int d = 3; d >= 0; d--) {
        os.v[d] = os.v[d + 1] * od.v[d + 1];
        ts.v[d] = ts.v[d + 1] * td.v[d + 1];
        xs.v[d] = xs.v[d + 1] * xd.v[d + 1];
    }
    for (int d = 0; d < 5; d++) { if (!os.v[d]) os.v[d] = 1; if (!xd.v[d]) xd.v[d] = 1; }
    launch_pdl(gather_kernel, dim3(grid_for(n, 256)), dim3(256), 0, st, tbl, idx, y, n, axis, xrank, irank, td, xd, os,
                                                   ts, xs);
    g_launches++;
}

// ScatterNd update pass (oplist_exec.c:1438-1470); the data copy runs first as
// a separate launch. Index groups are applied in order by one block, so a
// later group overwrites an earlier one as in the reference.
__global__ void scatter_nd_kernel(const int32_t* __restrict__ idx, const uint16_t* __restrict__ upd,
                                  uint16_t* __restrict__ y, uint32_t n, uint32_t K, uint32_t n_idx,
                                  uint32_t block, U5 od, U5 ostr) {
    for (uint32_t e = 0; e < n_idx; e++) {
        size_t base = 0;
        bool bad = false;
        for (uint32_t k = 0; k < K; k++) {
            int32_t c = idx[(size_t)e * K + k];
            if (c < 0 || c >= (int32_t)od.v[k]) { bad = true; break; }
            base += (size_t)c * ostr.v[k];
        }
        if (bad || base + block > n) continue;
        for (uint32_t j = threadIdx.x; j < block; j += blockDim.x) y[base + j] = upd[(size_t)e * block + j];
        __syncthreads();
    }
}
void k_scatter_nd(cudaStream_t st, const int32_t* idx, const uint16_t* upd, uint16_t* y,
                  uint32_t n, uint32_t K, uint32_t n_idx, uint32_t block, const uint32_t* od5) {
    U5 od, os;
    for (int i = 0; i < 5; i++) od.v[i] = od5[i];
    os.v[4] = 1;
    for (int d = 3; d >= 0; d--) os.v[d] = os.v[d + 1] * od.v[d + 1];
    scatter_nd_kernel<<<1, 256, 0, st>>>(idx, upd, y, n, K, n_idx, block, od, os);
    g_launches++;
}

// Argmax, first maximum wins, start value -1e30 (oplist_exec.c:1990-2004).
// Up to 128 CTAs scan contiguous ranges with 16-byte loads; the last CTA to
// finish merges the per-CTA winners (lower index wins ties), so one launch
// covers a vocabulary-sized row in a few microseconds.
__device__ float g_argmax_val[128];
__device__ int g_argmax_idx[128];
__device__ unsigned int g_argmax_done = 0;

__device__ __forceinline__ void argmax_take(float v, int i, float& bv, int& bi) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void __launch_bounds__(256) argmax_kernel(const uint16_t* __restrict__ x, int32_t* __restrict__ y, uint32_t n) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool s_last;
    const uint32_t per = ((n + gridDim.x - 1) / gridDim.x + 7u) & ~7u;
    const uint32_t lo = blockIdx.x * per, hi = (lo + per < n) ? lo + per : n;
    float bv = -1e30f;
    int bi = 0x7fffffff;
    if (lo < hi) {
        if ((((uintptr_t)x) & 15u) == 0) {
            for (uint32_t i = lo + threadIdx.x * 8; i < hi; i += blockDim.x * 8) {
                if (i + 8 <= hi) {
                    uint4 q = *(const uint4*)(x + i);
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        float a = h2f((uint16_t)(w[k] & 0xffffu)), b = h2f((uint16_t)(w[k] >> 16));
                        if (a > bv) { bv = a; bi = (int)(i + 2 * k); }
                        if (b > bv) { bv = b; bi = (int)(i + 2 * k + 1); }
                    }
                } else {
                    for (uint32_t k = i; k < hi; k++) { float a = h2f(x[k]); if (a > bv) { bv = a; bi = (int)k; } }
                }
            }
        } else {
            for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) { float a = h2f(x[i]); if (a > bv) { bv = a; bi = (int)i; } }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(ov, oi, bv, bi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) argmax_take(sv[w], si[w], bv, bi);
        g_argmax_val[blockIdx.x] = bv;
        g_argmax_idx[blockIdx.x] = bi;
        __threadfence();
        s_last = atomicAdd(&g_argmax_done, 1u) + 1 == gridDim.x;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        float fv = -1e30f;
        int fi = 0x7fffffff;
        for (uint32_t b = 0; b < gridDim.x; b++) argmax_take(g_argmax_val[b], g_argmax_idx[b], fv, fi);
        y[0] = (fi == 0x7fffffff) ? 0 : fi;
        g_argmax_done = 0;
    }
}
void k_argmax(cudaStream_t st, const uint16_t* x, int32_t* y, uint32_t n) {
    unsigned grid = (n + 4095) / 4096;
    if (grid < 1) grid = 1;
    if (grid > 128) grid = 128;
    argmax_kernel<<<grid, 256, 0, st>>>(x, y, n);
    g_launches++;
}

// The same for a batch of rows in one launch (grid.y = row): greedy sampling of a decode step over B sequences is
// B argmax ops on the rows of the logits matrix; per-row winners and counters, the last CTA of a row merges it.
__device__ float g_argmax_rows_val[kArgmaxMaxRows][128];
__device__ int g_argmax_rows_idx[kArgmaxMaxRows][128];
__device__ unsigned int g_argmax_rows_done[kArgmaxMaxRows];

__global__ void __launch_bounds__(256) argmax_rows_kernel(const uint16_t* x, int32_t* __restrict__ y, uint32_t n) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.y;
    const uint16_t* xr = x + (size_t)row * n;
    const uint32_t per = ((n + gridDim.x - 1) / gridDim.x + 7u) & ~7u;
    const uint32_t lo = blockIdx.x * per, hi = (lo + per < n) ? lo + per : n;
    float bv = -1e30f;
    int bi = 0x7fffffff;
    if (lo < hi) {
        if ((((uintptr_t)xr) & 15u) == 0) {
            for (uint32_t i = lo + threadIdx.x * 8; i < hi; i += blockDim.x * 8) {
                if (i + 8 <= hi) {
                    const uint4 q = __ldcg((const uint4*)(xr + i));
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float a = h2f((uint16_t)(w[k] & 0xffffu)), b = h2f((uint16_t)(w[k] >> 16));
                        if (a > bv) { bv = a; bi = (int)(i + 2 * k); }
                        if (b > bv) { bv = b; bi = (int)(i + 2 * k + 1); }
                    }
                } else {
                    for (uint32_t k = i; k < hi; k++) { const float a = h2f(__ldcg(xr + k)); if (a > bv) { bv = a; bi = (int)k; } }
                }
            }
        } else {
            for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) { const float a = h2f(__ldcg(xr + i)); if (a > bv) { bv = a; bi = (int)i; } }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(ov, oi, bv, bi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) argmax_take(sv[w], si[w], bv, bi);
        g_argmax_rows_val[row][blockIdx.x] = bv;
        g_argmax_rows_idx[row][blockIdx.x] = bi;
        __threadfence();
        s_last = atomicAdd(&g_argmax_rows_done[row], 1u) + 1 == gridDim.x;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        float fv = -1e30f;
        int fi = 0x7fffffff;
        for (uint32_t b = 0; b < gridDim.x; b++)
            argmax_take(__ldcg(&g_argmax_rows_val[row][b]), __ldcg(&g_argmax_rows_idx[row][b]), fv, fi);
        y[row] = (fi == 0x7fffffff) ? 0 : fi;
        g_argmax_rows_done[row] = 0;
    }
}
bool k_argmax_rows(cudaStream_t st, const uint16_t* x, int32_t* y, uint32_t rows, uint32_t n) {
    if (!rows || rows > kArgmaxMaxRows || !n) return false;
    unsigned gx = (n + 4095) / 4096;
    if (gx < 1) gx = 1;
    if (gx > 128) gx = 128;
    if (launch_pdl(argmax_rows_kernel, dim3(gx, rows), dim3(256), 0, st, x, y, n) != cudaSuccess) { cudaGetLastError(); return false; }
    g_launches++;
    return true;
}

// im2col for the conv pipeline (oplist_exec.c:615-645).
struct U15 { uint32_t v[15]; };
__global__ void im2col_kernel(const uint16_t* __restrict__ a, uint16_t* __restrict__ cols, U15 g) {
    uint32_t H = g.v[2], W = g.v[3], C = g.v[4], kh = g.v[5], kw = g.v[6], ph = g.v[7], pw = g.v[8];
    uint32_t sh = g.v[9], sw = g.v[10], y0 = g.v[11], x0 = g.v[12], th = g.v[13], tw = g.v[14];
    uint32_t K = kh * kw * C;
    size_t total = (size_t)th * tw * K;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        uint32_t row = (uint32_t)(e / K), col = (uint32_t)(e % K);
        uint32_t oy = row / tw, ox = row % tw;
        uint32_t c = col % C, kl = col / C, l = kl % kw, k = kl / kw;
        long gy = (long)(y0 + oy) * sh + (long)k - ph;
        long gx = (long)(x0 + ox) * sw + (long)l - pw;
        uint16_t v = 0;
        if (gy >= 0 && gy < (long)H && gx >= 0 && gx < (long)W) v = a[((size_t)gy * W + gx) * C + c];
        cols[e] = v;
    }
}
void k_im2col(cudaStream_t st, const uint16_t* a, uint16_t* cols, const uint32_t* args15) {
    U15 g;
    for (int i = 0; i < 15; i++) g.v[i] = args15[i];
    size_t total = (size_t)g.v[13] * g.v[14] * g.v[5] * g.v[6] * g.v[4];
    if (!total) return;
    im2col_kernel<<<grid_for(total, 256), 256, 0, st>>>(a, cols, g);
    g_launches++;
}

// conv2d as GEMM over im2col rows, bias as the start value, k ascending
// (oplist_exec.c:761-800).
__global__ void conv2d_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ Wm,
                              const uint16_t* __restrict__ Bm, uint16_t* __restrict__ out,
                              uint32_t M, uint32_t K, uint32_t N, uint32_t oy0, uint32_t ox0,
                              uint32_t out_W, uint32_t co0, uint32_t co_n) {
    size_t total = (size_t)M * co_n;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        uint32_t r = (uint32_t)(e / co_n), c = co0 + (uint32_t)(e % co_n);
        float acc = h2f(Bm[c]);
        for (uint32_t k = 0; k < K; k++) acc += h2f(A[(size_t)r * K + k]) * h2f(Wm[(size_t)k * N + c]);
        uint32_t oy = oy0 + r / out_W, ox = ox0 + r % out_W;
        out[((size_t)oy * out_W + ox) * N + c] = f2h(acc);
    }
}
void k_conv2d(cudaStream_t st, const uint16_t* A, const uint16_t* W, const uint16_t* Bv,
              uint16_t* out, uint32_t M, uint32_t K, uint32_t N, uint32_t oy0, uint32_t ox0,
              uint32_t out_W, uint32_t co0, uint32_t co_n) {
    if (!M || !co_n) return;
    conv2d_kernel<<<grid_for((size_t)M * co_n, 128), 128, 0, st>>>(A, W, Bv, out, M, K, N, oy0, ox0,
                                                                  out_W, co0, co_n);
    g_launches++;
}

}  // namespace gehtp
