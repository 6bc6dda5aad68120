/* See oracle.h. Plain C, scalar loops in the reference's order. */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include "oracle.h"

float orc_f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, bits;
    if (e == 0) {
        if (!m) bits = s;
        else {
            int sh = 0;
            while (!(m & 1024u)) { m <<= 1; sh++; }
            bits = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
        }
    } else if (e == 31u) bits = s | 0x7f800000u | (m << 13);
    else bits = s | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &bits, 4); return f;
}

/* round to nearest even incl. subnormals; NaN -> signed inf as the reference does */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t s = (x >> 16) & 0x8000u, be = (x >> 23) & 255u, m = x & 0x7fffffu;
    int32_t e = (int32_t)be - 112;
    if (be == 255u || e >= 31) return (uint16_t)(s | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000u;
        uint32_t sh = (uint32_t)(14 - e), q = m >> sh, r = m & ((1u << sh) - 1u), half = 1u << (sh - 1u);
        if (r > half || (r == half && (q & 1u))) q++;
        return (uint16_t)(s | q);
    }
    uint32_t h = s | ((uint32_t)e << 10) | (m >> 13);
    if ((m >> 12) & 1u) if ((m & 0xfffu) || (h & 1u)) h++;
    return (uint16_t)h;
}
#define H2F orc_f16_to_f32
#define F2H orc_f32_to_f16

void orc_w4_unpack_i8(const uint8_t* nib, int8_t* out, uint32_t K, uint32_t N) {
    for (uint32_t k = 0; k < K; k++)
        for (uint32_t n = 0; n < N; n++) {
            uint8_t b = nib[(size_t)k * (N / 2) + n / 2];
            out[(size_t)k * N + n] = (int8_t)((int)((n & 1u) ? (b >> 4) : (b & 15u)) - 8);
        }
}

void orc_w4_dequant(const uint8_t* slot, uint16_t* w, uint32_t K, uint32_t N) {
    const uint16_t* sc = (const uint16_t*)(slot + (size_t)K * N / 2);
    for (uint32_t k = 0; k < K; k++)
        for (uint32_t n = 0; n < N; n++) {
            uint8_t b = slot[(size_t)k * (N / 2) + n / 2];
            int q = (int)((n & 1u) ? (b >> 4) : (b & 15u)) - 8;
            w[(size_t)k * N + n] = F2H((float)q * H2F(sc[(size_t)(k / 64) * N + n]));
        }
}

void orc_matmul_f16(const uint16_t* a, const uint16_t* w, uint16_t* y, uint32_t M, uint32_t K,
                    uint32_t N, uint32_t n0, uint32_t N_full, int t0, int t1, int batched, uint32_t Bn) {
    if (!batched) Bn = 1;
    for (uint32_t bb = 0; bb < Bn; bb++) {
        const uint16_t* ab = a + (size_t)bb * M * K;
        const uint16_t* wb = w + (size_t)bb * K * N_full;
        uint16_t* yb = y + (size_t)bb * M * N_full;
        int ta = batched ? 0 : t0;
#pragma omp parallel for collapse(2) schedule(static)
        for (uint32_t m = 0; m < M; m++)
            for (uint32_t n = 0; n < N; n++) {
                float acc = 0.0f;
                for (uint32_t k = 0; k < K; k++) {
                    float av = H2F(ab[ta ? (size_t)k * M + m : (size_t)m * K + k]);
                    float wv = H2F(wb[t1 ? (size_t)(n0 + n) * K + k : (size_t)k * N_full + (n0 + n)]);
                    acc += av * wv;
                }
                yb[(size_t)m * N_full + n0 + n] = F2H(acc);
            }
    }
}

void orc_w4a16_matmul(const uint16_t* a, const uint8_t* slot, uint16_t* y, uint32_t M, uint32_t K, uint32_t N) {
    /* fp32 copies first: the scalar converters dominate otherwise */
    float* wf = (float*)malloc((size_t)K * N * 4);
    float* af = (float*)malloc((size_t)M * K * 4);
    uint16_t* w16 = (uint16_t*)malloc((size_t)K * N * 2);
    orc_w4_dequant(slot, w16, K, N);
    for (size_t i = 0; i < (size_t)K * N; i++) wf[i] = H2F(w16[i]);
    for (size_t i = 0; i < (size_t)M * K; i++) af[i] = H2F(a[i]);
#pragma omp parallel for schedule(static)
    for (uint32_t m = 0; m < M; m++) {
        float* acc = (float*)calloc(N, 4);
        for (uint32_t k = 0; k < K; k++) {           /* k ascending per output, as orc_matmul_f16 */
            float av = af[(size_t)m * K + k];
            const float* wr = wf + (size_t)k * N;
            for (uint32_t n = 0; n < N; n++) acc[n] += av * wr[n];
        }
        for (uint32_t n = 0; n < N; n++) y[(size_t)m * N + n] = F2H(acc[n]);
        free(acc);
    }
    free(wf); free(af); free(w16);
}

void orc_rmsnorm2(const uint16_t* x, const uint16_t* g, const uint16_t* b, uint16_t* y, uint32_t rows, uint32_t width) {
    for (uint32_t r = 0; r < rows; r++) {
        double acc = 0.0;
        for (uint32_t i = 0; i < width; i++) { float v = H2F(x[(size_t)r * width + i]); acc += (double)v * (double)v; }
        float rms = (float)sqrt(acc / (double)width + 1e-6);
        for (uint32_t i = 0; i < width; i++) {
            float v = H2F(x[(size_t)r * width + i]) / rms;
            v = v * H2F(g[i]) + (b ? H2F(b[i]) : 0.0f);
            y[(size_t)r * width + i] = F2H(v);
        }
    }
}

void orc_softmax(const uint16_t* x, uint16_t* y, uint32_t rows, uint32_t n) {
    int wide = rows >= 1u && (n % 32u) == 0u && (size_t)rows * n >= 32u;
    for (uint32_t r = 0; r < rows; r++) {
        const uint16_t* xr = x + (size_t)r * n; uint16_t* yr = y + (size_t)r * n;
        if (wide) {
            float mx = -3.402823466e38f;
            for (uint32_t i = 0; i < n; i++) { float v = H2F(xr[i]); if (v > mx) mx = v; }
            double sum = 0.0;
            float* e = (float*)malloc((size_t)n * 4);
            for (uint32_t i = 0; i < n; i++) { e[i] = expf(H2F(xr[i]) - mx); sum += e[i]; }
            float inv = sum > 0.0 ? (float)(1.0 / sum) : 0.0f;
            for (uint32_t i = 0; i < n; i++) yr[i] = F2H(e[i] * inv);
            free(e);
        } else {
            float mx = H2F(xr[0]);
            for (uint32_t i = 1; i < n; i++) mx = fmaxf(mx, H2F(xr[i]));
            float sum = 0.0f;
            for (uint32_t i = 0; i < n; i++) { float e = expf(H2F(xr[i]) - mx); yr[i] = F2H(e); sum += e; }
            for (uint32_t i = 0; i < n; i++) yr[i] = F2H(H2F(yr[i]) / sum);
        }
    }
}

void orc_binary(const uint16_t* a, const uint16_t* b, uint16_t* y, uint32_t n, uint32_t subtype) {
    for (uint32_t i = 0; i < n; i++) {
        float x0 = H2F(a[i]), x1 = H2F(b[i]), r = x0;
        switch (subtype) {
        case 0: r = x0 + x1; break;
        case 1: r = x0 - x1; break;
        case 2: r = x0 * x1; break;
        case 3: r = (n >= 32u) ? x0 / x1 : ((x1 != 0) ? x0 / x1 : 0.0f); break;
        case 4: r = (x0 == x1) ? 1.0f : 0.0f; break;
        case 5: r = ((uint32_t)x0 & (uint32_t)x1) ? 1.0f : 0.0f; break;
        default: break;
        }
        y[i] = F2H(r);
    }
}

int orc_unary(const uint16_t* x, uint16_t* y, uint32_t n, uint32_t subtype) {
    if (subtype > 16u) return -1;
    for (uint32_t i = 0; i < n; i++) {
        float v = H2F(x[i]), r = v;
        switch (subtype) {
        case 0: r = -v; break;
        case 1: r = expf(v); break;
        case 2: r = v >= 0 ? sqrtf(v) : 0.0f; break;
        case 3: r = v > 0 ? 1.0f / sqrtf(v) : 0.0f; break;
        case 4: r = v > 0 ? logf(v) : 0.0f; break;
        case 5: r = fabsf(v); break;
        case 6: r = sinf(v); break;
        case 7: r = cosf(v); break;
        case 8: r = 1.0f / (1.0f + expf(-v)); break;
        case 9: r = tanhf(v); break;
        case 10: r = 0.5f * v * (1.0f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v))); break;
        case 11: r = fmaxf(0.0f, v); break;
        case 12: r = v / (1.0f + expf(-v)); break;
        case 13: r = v > 30.0f ? v : (v < -30.0f ? expf(v) : log1pf(expf(v))); break;
        case 15: r = (v != v) ? 1.0f : 0.0f; break;
        case 16: r = (v == v && (v > 3.4e38f || v < -3.4e38f)) ? 1.0f : 0.0f; break;
        default: break;
        }
        y[i] = F2H(r);
    }
    return 0;
}

void orc_kv_append(uint16_t* ring, uint32_t* posmap, uint32_t nslots, uint32_t kv_elems,
                   const uint16_t* k, const uint16_t* v, uint32_t pos) {
    uint32_t slot = pos % nslots;
    uint16_t* kf = ring + (size_t)slot * kv_elems * 2;
    memcpy(kf, k, (size_t)kv_elems * 2);
    memcpy(kf + kv_elems, v, (size_t)kv_elems * 2);
    posmap[slot] = pos;
}

int orc_kv_gather(const uint16_t* ring, const uint32_t* posmap, uint32_t nslots, uint32_t n_kv,
                  uint32_t pstride, uint32_t n_heads, uint32_t kv_heads, uint32_t hd, uint16_t* kT, uint16_t* vo) {
    uint32_t kv_elems = kv_heads * hd, rep = n_heads / kv_heads;
    if (pstride > n_kv) {
        if (kT) memset(kT, 0, (size_t)n_heads * hd * pstride * 2);
        if (vo) memset(vo, 0, (size_t)n_heads * pstride * hd * 2);
    }
    for (uint32_t p = 0; p < n_kv; p++) {
        uint32_t slot = p % nslots;
        if (posmap && posmap[slot] != p) return -1;
        const uint16_t* kf = ring + (size_t)slot * kv_elems * 2;
        const uint16_t* vf = kf + kv_elems;
        for (uint32_t h = 0; h < n_heads; h++) {
            const uint16_t* ks = kf + (h / rep) * hd; const uint16_t* vs = vf + (h / rep) * hd;
            if (kT) for (uint32_t d = 0; d < hd; d++) kT[((size_t)h * hd + d) * pstride + p] = ks[d];
            if (vo) memcpy(vo + ((size_t)h * pstride + p) * hd, vs, (size_t)hd * 2);
        }
    }
    return 0;
}

int orc_attn_decode_chain(const uint16_t* q, const uint16_t* ring, const uint32_t* posmap,
                          uint32_t nslots, uint32_t n_kv, uint32_t n_heads, uint32_t kv_heads,
                          uint32_t hd, float scale, int scale_div, const uint16_t* mask, uint16_t* out) {
    size_t fe = (size_t)n_heads * hd * n_kv;
    uint16_t* kT = (uint16_t*)malloc(fe * 2); uint16_t* vo = (uint16_t*)malloc(fe * 2);
    uint16_t* s = (uint16_t*)malloc((size_t)n_heads * n_kv * 2);
    uint16_t* t = (uint16_t*)malloc((size_t)n_heads * n_kv * 2);
    uint16_t* bc = (uint16_t*)malloc((size_t)n_heads * n_kv * 2);
    int rc = orc_kv_gather(ring, posmap, nslots, n_kv, n_kv, n_heads, kv_heads, hd, kT, vo);
    if (rc == 0) {
        orc_matmul_f16(q, kT, s, 1, hd, n_kv, 0, n_kv, 0, 0, 1, n_heads);
        uint16_t sc16 = F2H(scale);
        for (size_t i = 0; i < (size_t)n_heads * n_kv; i++) bc[i] = sc16;
        orc_binary(s, bc, t, n_heads * n_kv, scale_div ? 3 : 2);
        if (mask) {
            for (uint32_t h = 0; h < n_heads; h++) memcpy(bc + (size_t)h * n_kv, mask, (size_t)n_kv * 2);
            orc_binary(t, bc, s, n_heads * n_kv, 0);
        } else memcpy(s, t, (size_t)n_heads * n_kv * 2);
        orc_softmax(s, t, n_heads, n_kv);
        orc_matmul_f16(t, vo, out, 1, n_kv, hd, 0, hd, 0, 0, 1, n_heads);
    }
    free(kT); free(vo); free(s); free(t); free(bc);
    return rc;
}

void orc_attn_decode_f64(const uint16_t* q, const uint16_t* ring, uint32_t nslots, uint32_t n_kv,
                         uint32_t n_heads, uint32_t kv_heads, uint32_t hd, double scale,
                         const uint16_t* mask, double* out) {
    uint32_t kv_elems = kv_heads * hd, rep = n_heads / kv_heads;
    double* sc = (double*)malloc((size_t)n_kv * 8);
    for (uint32_t h = 0; h < n_heads; h++) {
        double mx = -1e300;
        for (uint32_t p = 0; p < n_kv; p++) {
            const uint16_t* kf = ring + (size_t)(p % nslots) * kv_elems * 2 + (h / rep) * hd;
            double d = 0;
            for (uint32_t i = 0; i < hd; i++) d += (double)H2F(q[(size_t)h * hd + i]) * (double)H2F(kf[i]);
            sc[p] = d * scale + (mask ? (double)H2F(mask[p]) : 0.0);
            if (sc[p] > mx) mx = sc[p];
        }
        double sum = 0;
        for (uint32_t p = 0; p < n_kv; p++) { sc[p] = exp(sc[p] - mx); sum += sc[p]; }
        for (uint32_t i = 0; i < hd; i++) {
            double acc = 0;
            for (uint32_t p = 0; p < n_kv; p++)
                acc += sc[p] * (double)H2F(ring[(size_t)(p % nslots) * kv_elems * 2 + kv_elems + (h / rep) * hd + i]);
            out[(size_t)h * hd + i] = acc / sum;
        }
    }
    free(sc);
}

void orc_conv1d_ssm(const uint16_t* x, const uint16_t* w, uint16_t* y, uint32_t seq, uint32_t C, uint32_t k) {
    int32_t in_rows = seq >= k ? (int32_t)(seq - k + 1) : 0;
    for (uint32_t t = 0; t < seq; t++)
        for (uint32_t c = 0; c < C; c++) {
            float acc = 0.0f;
            for (uint32_t j = 0; j < k; j++) {
                int32_t src = (int32_t)t - (int32_t)(k - 1) + (int32_t)j;
                if (src < 0 || src >= in_rows) continue;
                acc += H2F(x[(size_t)src * C + c]) * H2F(w[(size_t)j * C + c]);
            }
            y[(size_t)t * C + c] = F2H(acc);
        }
}

void orc_conv1d_step(const uint16_t* x, const uint16_t* w, uint16_t* y, float* win, uint32_t C, uint32_t dc) {
    for (uint32_t c = 0; c < C; c++) {
        float xf = H2F(x[c]), s = 0.0f;
        for (uint32_t i = 0; i + 1 < dc; i++) s += H2F(w[(size_t)i * C + c]) * win[(size_t)i * C + c];
        s += H2F(w[(size_t)(dc - 1) * C + c]) * xf;
        y[c] = F2H(s / (1.0f + expf(-s)));
    }
    memmove(win, win + C, (size_t)(dc - 2) * C * 4);
    for (uint32_t c = 0; c < C; c++) win[(size_t)(dc - 2) * C + c] = H2F(x[c]);
}

int orc_delta_chunk(const uint16_t* k, const uint16_t* v, const uint16_t* q, const uint16_t* beta,
                    const uint16_t* g, uint16_t* y, float* Sall, int c, int ntok, int H, int D, int q_raw) {
    if (c < 1 || c > 64) return 1;
    float scale = q_raw ? 1.0f : 1.0f / sqrtf((float)D);
    float *kf = malloc((size_t)c * D * 4), *vf = malloc((size_t)c * D * 4), *qf = malloc((size_t)c * D * 4);
    float *u = malloc((size_t)c * D * 4), *bm = malloc((size_t)c * D * 4), *G = malloc((size_t)c * 4), *row = malloc((size_t)D * 4);
    uint16_t *L = malloc((size_t)c * c * 2), *T = malloc((size_t)c * c * 2);
    for (int h = 0; h < H; h++) {
        const uint16_t *kh = k + (size_t)h * ntok * D, *vh = v + (size_t)h * ntok * D, *qh = q + (size_t)h * ntok * D;
        const uint16_t *bh = beta + (size_t)h * ntok, *gh = g + (size_t)h * ntok;
        float* S = Sall + (size_t)h * D * D;
        float acc = 0.0f;
        for (int t = 0; t < c; t++) {
            acc += H2F(gh[t]); G[t] = acc;
            for (int n = 0; n < D; n++) {
                kf[t * D + n] = H2F(kh[t * D + n]); vf[t * D + n] = H2F(vh[t * D + n]);
                qf[t * D + n] = H2F(qh[t * D + n]) * scale;
            }
        }
        for (int j = 0; j < c; j++) {
            float bj = H2F(bh[j]);
            for (int i = 0; i < c; i++) {
                uint16_t r = 0;
                if (i < j) {
                    float s = 0.0f;
                    for (int n = 0; n < D; n++) s += kf[j * D + n] * kf[i * D + n];
                    r = F2H(expf(G[j] - G[i]) * s * bj);
                }
                L[j * c + i] = r;
            }
        }
        for (int r = 0; r < c; r++)
            for (int j = 0; j < c; j++) {
                uint16_t o = 0;
                if (j <= r) {
                    float s = (r == j) ? 1.0f : 0.0f;
                    for (int i = j; i < r; i++) s -= H2F(L[r * c + i]) * H2F(T[i * c + j]);
                    o = F2H(s);
                }
                T[r * c + j] = o;
            }
        for (int j = 0; j < c; j++) {
            float ej = expf(G[j]), bj = H2F(bh[j]);
            for (int m = 0; m < D; m++) {
                float sk = 0.0f;
                for (int n = 0; n < D; n++) sk += S[m * D + n] * kf[j * D + n];
                bm[j * D + m] = bj * (vf[j * D + m] - ej * sk);
                u[j * D + m] = 0.0f;
            }
            for (int i = 0; i <= j; i++) {
                float tij = H2F(T[j * c + i]);
                if (tij == 0.0f) continue;
                for (int m = 0; m < D; m++) u[j * D + m] += tij * bm[i * D + m];
            }
        }
        for (int t = 0; t < c; t++) {
            float et = expf(G[t]);
            for (int m = 0; m < D; m++) {
                float s = 0.0f;
                for (int n = 0; n < D; n++) s += S[m * D + n] * qf[t * D + n];
                row[m] = et * s;
            }
            for (int i = 0; i <= t; i++) {
                float qk = 0.0f, w = expf(G[t] - G[i]);
                for (int n = 0; n < D; n++) qk += qf[t * D + n] * kf[i * D + n];
                qk *= w;
                if (qk == 0.0f) continue;
                for (int m = 0; m < D; m++) row[m] += qk * u[i * D + m];
            }
            for (int m = 0; m < D; m++) y[(size_t)h * ntok * D + (size_t)t * D + m] = F2H(row[m]);
        }
        float eC = expf(G[c - 1]);
        for (size_t z = 0; z < (size_t)D * D; z++) S[z] *= eC;
        for (int i = 0; i < c; i++) {
            float w = expf(G[c - 1] - G[i]);
            for (int m = 0; m < D; m++) {
                float wu = w * u[i * D + m];
                if (wu == 0.0f) continue;
                for (int n = 0; n < D; n++) S[m * D + n] += wu * kf[i * D + n];
            }
        }
    }
    free(kf); free(vf); free(qf); free(u); free(bm); free(G); free(row); free(L); free(T);
    return 0;
}

void orc_delta_token(float* S, int D, const float* k, const float* v, const float* q, float beta, float g, float* y) {
    float a = expf(g), scale = 1.0f / sqrtf((float)D);
    float* yk = (float*)malloc((size_t)D * 4);
    for (int j = 0; j < D; j++) {
        float s = 0.0f;
        for (int n = 0; n < D; n++) { S[j * D + n] *= a; s += S[j * D + n] * k[n]; }
        yk[j] = s;
    }
    for (int j = 0; j < D; j++) {
        float dj = beta * (v[j] - yk[j]), s = 0.0f;
        for (int n = 0; n < D; n++) { S[j * D + n] += dj * k[n]; s += S[j * D + n] * q[n]; }
        y[j] = s * scale;
    }
    free(yk);
}
