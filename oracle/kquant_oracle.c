/*
 * kquant_oracle.c -- CPU oracle for the K-quant forward pass.  TEST INFRASTRUCTURE ONLY.
 *
 * Restates, in plain C, the arithmetic of the quantised forward pass that every mesh-llm stage
 * runs inside llama.cpp/ggml (pin: third_party/llama.cpp/upstream.txt:1; sources not vendored,
 * see the header for the parity status).  What each function follows:
 *   - block layouts: the in-tree facts about GGUF tensor types in
 *     mesh-client/src/models/gguf.rs:19-35 (type ids) plus the published Q4_K / Q6_K block
 *     layout (256 elements, 144 / 210 bytes);
 *   - graph order of one layer and of the MoE FFN: third_party/llama.cpp/patches/0003 lines
 *     82-108 (probs -> mask -> top-k) and 945-955 (expert tensor names);
 *   - stage split (layer ranges, embeddings first, output last):
 *     mesh-llm/src/inference/election.rs:3095-3114.
 * Only tests, the smoke check and the bench's cpu_baseline leg may call into this file.
 */
#define _GNU_SOURCE
#include "kquant_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#if defined(__x86_64__) && defined(__GNUC__) && !defined(ORC_NO_CLONES)
#define ORC_CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))
#else
#define ORC_CLONES
#endif

static int g_threads = 0;
void orc_set_threads(int n) {
    g_threads = n;
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}
int orc_get_threads(void) {
#ifdef _OPENMP
    return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- f16 <-> f32 (IEEE, RNE) */
static inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x38800000u) { /* subnormal or zero in f16 */
        if (absx < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        int e = (int)(absx >> 23);                      /* biased f32 exponent */
        uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
        int shift = 126 - e; /* 113 - e + 13 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t e = (absx >> 23) - 112u;
    uint32_t man = absx & 0x7FFFFFu;
    uint32_t half = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

void orc_f32_to_f16(const float *x, int64_t n, uint16_t *y) {
    for (int64_t i = 0; i < n; i++) y[i] = f2h(x[i]);
}
void orc_f16_to_f32(const uint16_t *x, int64_t n, float *y) {
    for (int64_t i = 0; i < n; i++) y[i] = h2f(x[i]);
}

/* ---------------------------------------------------------------- block formats */
/* Q4_K: 6-bit scale / min j of a super-block from the 12 packed bytes */
static inline void q4k_scale_min(const uint8_t *s, int j, int *sc, int *mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/* unpack the 256 4-bit codes of one Q4_K block in element order */
static inline void q4k_unpack(const uint8_t *blk, uint8_t *q /*256*/) {
    const uint8_t *qs = blk + 16;
    for (int g = 0; g < 4; g++)
        for (int i = 0; i < 32; i++) {
            uint8_t b = qs[32 * g + i];
            q[64 * g + i] = b & 0x0F;
            q[64 * g + 32 + i] = b >> 4;
        }
}

/* unpack the 256 6-bit codes of one Q6_K block as signed values (q - 32) in element order */
static inline void q6k_unpack(const uint8_t *blk, int8_t *q /*256*/) {
    const uint8_t *ql = blk, *qh = blk + 128;
    for (int h = 0; h < 2; h++)
        for (int i = 0; i < 32; i++) {
            uint8_t hb = qh[32 * h + i];
            uint8_t l0 = ql[64 * h + i], l1 = ql[64 * h + 32 + i];
            q[128 * h + i] = (int8_t)(((l0 & 0x0F) | (((hb >> 0) & 3) << 4)) - 32);
            q[128 * h + 32 + i] = (int8_t)(((l1 & 0x0F) | (((hb >> 2) & 3) << 4)) - 32);
            q[128 * h + 64 + i] = (int8_t)(((l0 >> 4) | (((hb >> 4) & 3) << 4)) - 32);
            q[128 * h + 96 + i] = (int8_t)(((l1 >> 4) | (((hb >> 6) & 3) << 4)) - 32);
        }
}

void orc_dequant_q4k(const uint8_t *blocks, int64_t nblocks, float *out) {
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * ORC_Q4K_BYTES;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        float d = h2f(dh), dmin = h2f(mh);
        uint8_t q[256];
        q4k_unpack(blk, q);
        for (int j = 0; j < 8; j++) {
            int sc, mn;
            q4k_scale_min(blk + 4, j, &sc, &mn);
            float dl = d * (float)sc, ml = dmin * (float)mn;
            for (int i = 0; i < 32; i++) out[b * 256 + 32 * j + i] = dl * (float)q[32 * j + i] - ml;
        }
    }
}

void orc_dequant_q6k(const uint8_t *blocks, int64_t nblocks, float *out) {
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * ORC_Q6K_BYTES;
        const int8_t *sc = (const int8_t *)(blk + 192);
        uint16_t dh;
        memcpy(&dh, blk + 208, 2);
        float d = h2f(dh);
        int8_t q[256];
        q6k_unpack(blk, q);
        for (int t = 0; t < 16; t++) {
            float dl = d * (float)sc[t];
            for (int i = 0; i < 16; i++) out[b * 256 + 16 * t + i] = dl * (float)q[16 * t + i];
        }
    }
}

int64_t orc_row_bytes(int type, int64_t k) {
    switch (type) {
    case ORC_TYPE_F32: return k * 4;
    case ORC_TYPE_F16: return k * 2;
    case ORC_TYPE_Q8_0: return k / 32 * 34;
    case ORC_TYPE_Q4_0: return k / 32 * 18;
    case ORC_TYPE_Q4_K: return k / 256 * ORC_Q4K_BYTES;
    case ORC_TYPE_Q6_K: return k / 256 * ORC_Q6K_BYTES;
    default: return -1;
    }
}

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Plain affine quantiser: per 32 elements scale=(max-min)/15 with min clamped to <= 0;
 * super-block d = max(scale)/63 and dmin = max(-min)/63, both rounded to f16 first.        */
void orc_quantize_q4k(const float *x, int64_t n, uint8_t *out) {
    int64_t nb = n / 256;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const float *xb = x + b * 256;
        uint8_t *blk = out + b * ORC_Q4K_BYTES;
        float scale[8], mins[8], smax = 0.f, mmax = 0.f;
        for (int j = 0; j < 8; j++) {
            float lo = 0.f, hi = 0.f;
            for (int i = 0; i < 32; i++) {
                float v = xb[32 * j + i];
                if (v < lo) lo = v;
                if (v > hi) hi = v;
            }
            scale[j] = (hi - lo) / 15.0f;
            mins[j] = -lo;
            if (scale[j] > smax) smax = scale[j];
            if (mins[j] > mmax) mmax = mins[j];
        }
        uint16_t dh = f2h(smax / 63.0f), mh = f2h(mmax / 63.0f);
        float d = h2f(dh), dmin = h2f(mh);
        int sc[8], mn[8];
        for (int j = 0; j < 8; j++) {
            sc[j] = d > 0.f ? clampi((int)lrintf(scale[j] / d), 0, 63) : 0;
            mn[j] = dmin > 0.f ? clampi((int)lrintf(mins[j] / dmin), 0, 63) : 0;
        }
        memcpy(blk, &dh, 2);
        memcpy(blk + 2, &mh, 2);
        uint8_t *s = blk + 4;
        memset(s, 0, 12);
        for (int j = 0; j < 8; j++) {
            if (j < 4) {
                s[j] |= (uint8_t)sc[j];
                s[j + 4] |= (uint8_t)mn[j];
            } else {
                s[j + 4] = (uint8_t)((sc[j] & 0x0F) | ((mn[j] & 0x0F) << 4));
                s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
                s[j] |= (uint8_t)((mn[j] >> 4) << 6);
            }
        }
        uint8_t q[256];
        for (int j = 0; j < 8; j++) {
            float dl = d * (float)sc[j], ml = dmin * (float)mn[j];
            for (int i = 0; i < 32; i++) {
                int v = dl > 0.f ? (int)lrintf((xb[32 * j + i] + ml) / dl) : 0;
                q[32 * j + i] = (uint8_t)clampi(v, 0, 15);
            }
        }
        uint8_t *qs = blk + 16;
        for (int g = 0; g < 4; g++)
            for (int i = 0; i < 32; i++)
                qs[32 * g + i] = (uint8_t)(q[64 * g + i] | (q[64 * g + 32 + i] << 4));
    }
}

/* Symmetric quantiser: per 16 elements scale = max|x|/31; d = max(scale)/127 rounded to f16. */
void orc_quantize_q6k(const float *x, int64_t n, uint8_t *out) {
    int64_t nb = n / 256;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const float *xb = x + b * 256;
        uint8_t *blk = out + b * ORC_Q6K_BYTES;
        float scale[16], smax = 0.f;
        for (int t = 0; t < 16; t++) {
            float am = 0.f;
            for (int i = 0; i < 16; i++) {
                float a = fabsf(xb[16 * t + i]);
                if (a > am) am = a;
            }
            scale[t] = am / 31.0f;
            if (scale[t] > smax) smax = scale[t];
        }
        uint16_t dh = f2h(smax / 127.0f);
        float d = h2f(dh);
        int8_t *sc = (int8_t *)(blk + 192);
        uint8_t q[256];
        for (int t = 0; t < 16; t++) {
            int s = d > 0.f ? clampi((int)lrintf(scale[t] / d), 0, 127) : 0;
            sc[t] = (int8_t)s;
            float dl = d * (float)s;
            for (int i = 0; i < 16; i++) {
                int v = dl > 0.f ? (int)lrintf(xb[16 * t + i] / dl) : 0;
                q[16 * t + i] = (uint8_t)(clampi(v, -32, 31) + 32);
            }
        }
        memcpy(blk + 208, &dh, 2);
        uint8_t *ql = blk, *qh = blk + 128;
        for (int h = 0; h < 2; h++)
            for (int i = 0; i < 32; i++) {
                uint8_t e0 = q[128 * h + i], e1 = q[128 * h + 32 + i];
                uint8_t e2 = q[128 * h + 64 + i], e3 = q[128 * h + 96 + i];
                ql[64 * h + i] = (uint8_t)((e0 & 0x0F) | ((e2 & 0x0F) << 4));
                ql[64 * h + 32 + i] = (uint8_t)((e1 & 0x0F) | ((e3 & 0x0F) << 4));
                qh[32 * h + i] =
                    (uint8_t)((e0 >> 4) | ((e1 >> 4) << 2) | ((e2 >> 4) << 4) | ((e3 >> 4) << 6));
            }
    }
}

/* ---------------------------------------------------------------- activation quantiser */
void orc_quantize_act(const float *x, int64_t M, int64_t K, int8_t *q, float *d, int16_t *bsum16) {
    int64_t nb = K / 256;
#pragma omp parallel for schedule(static) if (M * nb >= 64)
    for (int64_t mb = 0; mb < M * nb; mb++) {
        const float *xb = x + mb * 256;
        int8_t *qb = q + mb * 256;
        float amax = 0.f;
        for (int i = 0; i < 256; i++) {
            float a = fabsf(xb[i]);
            if (a > amax) amax = a;
        }
        float dd = amax / 127.0f;
        float id = dd > 0.f ? 1.0f / dd : 0.f;
        d[mb] = dd;
        for (int t = 0; t < 16; t++) {
            int s = 0;
            for (int i = 0; i < 16; i++) {
                int v = clampi((int)lrintf(xb[16 * t + i] * id), -127, 127);
                qb[16 * t + i] = (int8_t)v;
                s += v;
            }
            if (bsum16) bsum16[mb * 16 + t] = (int16_t)s;
        }
    }
}

/* ---------------------------------------------------------------- integer block dots */
ORC_CLONES
static void q4k_block_ints(const uint8_t *blk, const int8_t *a, const int16_t *bs, int32_t *sumi,
                           int32_t *summ) {
    uint8_t q[256];
    q4k_unpack(blk, q);
    int32_t si = 0, sm = 0;
    for (int j = 0; j < 8; j++) {
        int sc, mn;
        q4k_scale_min(blk + 4, j, &sc, &mn);
        int32_t dot = 0;
        for (int i = 0; i < 32; i++) dot += (int32_t)q[32 * j + i] * (int32_t)a[32 * j + i];
        si += sc * dot;
        sm += mn * ((int32_t)bs[2 * j] + (int32_t)bs[2 * j + 1]);
    }
    *sumi = si;
    *summ = sm;
}

ORC_CLONES
static void q6k_block_ints(const uint8_t *blk, const int8_t *a, int32_t *sumi) {
    int8_t q[256];
    q6k_unpack(blk, q);
    const int8_t *sc = (const int8_t *)(blk + 192);
    int32_t si = 0;
    for (int t = 0; t < 16; t++) {
        int32_t dot = 0;
        for (int i = 0; i < 16; i++) dot += (int32_t)q[16 * t + i] * (int32_t)a[16 * t + i];
        si += (int32_t)sc[t] * dot;
    }
    *sumi = si;
}

void orc_block_sums(int type, const uint8_t *W, const int8_t *q, const int16_t *bsum16, int64_t M,
                    int64_t N, int64_t K, int32_t *sumi, int32_t *summ) {
    int64_t nb = K / 256;
    int64_t rb = orc_row_bytes(type, K);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++)
            for (int64_t b = 0; b < nb; b++) {
                int32_t si = 0, sm = 0;
                if (type == ORC_TYPE_Q4_K)
                    q4k_block_ints(W + n * rb + b * ORC_Q4K_BYTES, q + m * K + b * 256,
                                   bsum16 + (m * nb + b) * 16, &si, &sm);
                else
                    q6k_block_ints(W + n * rb + b * ORC_Q6K_BYTES, q + m * K + b * 256, &si);
                sumi[(m * N + n) * nb + b] = si;
                if (summ) summ[(m * N + n) * nb + b] = sm;
            }
}

/* one weight row against M quantised activation rows; weights of a block are unpacked once */
ORC_CLONES
static void row_dot_q4k(const uint8_t *row, int64_t nb, const int8_t *q, const float *d,
                        const int16_t *bs, int64_t M, int64_t K, float *y, int64_t ystride) {
    for (int64_t m = 0; m < M; m++) y[m * ystride] = 0.f;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * ORC_Q4K_BYTES;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        float dw = h2f(dh), dmin = h2f(mh);
        int8_t w[256];
        int sc[8], mn[8];
        q4k_unpack(blk, (uint8_t *)w);
        for (int j = 0; j < 8; j++) q4k_scale_min(blk + 4, j, &sc[j], &mn[j]);
        for (int64_t m = 0; m < M; m++) {
            const int8_t *a = q + m * K + b * 256;
            const int16_t *s16 = bs + (m * nb + b) * 16;
            int32_t si = 0, sm = 0;
            for (int j = 0; j < 8; j++) {
                int32_t dot = 0;
                for (int i = 0; i < 32; i++) dot += (int32_t)w[32 * j + i] * (int32_t)a[32 * j + i];
                si += sc[j] * dot;
                sm += mn[j] * ((int32_t)s16[2 * j] + (int32_t)s16[2 * j + 1]);
            }
            float da = d[m * nb + b];
            y[m * ystride] += (dw * da) * (float)si - (dmin * da) * (float)sm;
        }
    }
}

ORC_CLONES
static void row_dot_q6k(const uint8_t *row, int64_t nb, const int8_t *q, const float *d, int64_t M,
                        int64_t K, float *y, int64_t ystride) {
    for (int64_t m = 0; m < M; m++) y[m * ystride] = 0.f;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * ORC_Q6K_BYTES;
        const int8_t *sc = (const int8_t *)(blk + 192);
        uint16_t dh;
        memcpy(&dh, blk + 208, 2);
        float dw = h2f(dh);
        int8_t w[256];
        q6k_unpack(blk, w);
        for (int64_t m = 0; m < M; m++) {
            const int8_t *a = q + m * K + b * 256;
            int32_t si = 0;
            for (int t = 0; t < 16; t++) {
                int32_t dot = 0;
                for (int i = 0; i < 16; i++) dot += (int32_t)w[16 * t + i] * (int32_t)a[16 * t + i];
                si += (int32_t)sc[t] * dot;
            }
            y[m * ystride] += (dw * d[m * nb + b]) * (float)si;
        }
    }
}

void orc_mul_mat_q8(int type, const uint8_t *W, const int8_t *q, const float *d,
                    const int16_t *bsum16, int64_t M, int64_t N, int64_t K, float *y) {
    int64_t nb = K / 256, rb = orc_row_bytes(type, K);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        if (type == ORC_TYPE_Q4_K)
            row_dot_q4k(W + n * rb, nb, q, d, bsum16, M, K, y + n, N);
        else
            row_dot_q6k(W + n * rb, nb, q, d, M, K, y + n, N);
    }
}

void orc_mul_mat(int type, const uint8_t *W, const float *x, int64_t M, int64_t N, int64_t K,
                 float *y) {
    int8_t *q = (int8_t *)malloc((size_t)(M * K));
    float *d = (float *)malloc(sizeof(float) * (size_t)(M * K / 256));
    int16_t *bs = (int16_t *)malloc(sizeof(int16_t) * (size_t)(M * K / 16));
    orc_quantize_act(x, M, K, q, d, bs);
    orc_mul_mat_q8(type, W, q, d, bs, M, N, K, y);
    free(q);
    free(d);
    free(bs);
}

/* ---------------------------------------------------------------- surrounding ops */
void orc_rms_norm(const float *x, const float *w, int64_t T, int64_t h, float eps, float *y) {
    for (int64_t t = 0; t < T; t++) {
        const float *xr = x + t * h;
        double ss = 0.0; /* the sum is accumulated wide so its order does not matter */
        for (int64_t i = 0; i < h; i++) ss += (double)xr[i] * (double)xr[i];
        float scale = 1.0f / sqrtf((float)(ss / (double)h) + eps);
        for (int64_t i = 0; i < h; i++) y[t * h + i] = xr[i] * scale * (w ? w[i] : 1.0f);
    }
}

void orc_rope_inv_freq(float theta, int64_t hd, float *inv_freq) {
    for (int64_t i = 0; i < hd / 2; i++)
        inv_freq[i] = (float)pow((double)theta, -2.0 * (double)i / (double)hd);
}

void orc_rope(float *x, const int32_t *pos, int64_t T, int64_t n_head, int64_t hd, float theta,
              int neox) {
    float inv[512];
    orc_rope_inv_freq(theta, hd, inv);
    for (int64_t t = 0; t < T; t++)
        for (int64_t h = 0; h < n_head; h++) {
            float *v = x + (t * n_head + h) * hd;
            for (int64_t i = 0; i < hd / 2; i++) {
                float ang = (float)pos[t] * inv[i];
                float c = cosf(ang), s = sinf(ang);
                int64_t i0 = neox ? i : 2 * i, i1 = neox ? i + hd / 2 : 2 * i + 1;
                float a = v[i0], b = v[i1];
                v[i0] = a * c - b * s;
                v[i1] = a * s + b * c;
            }
        }
}

void orc_swiglu(const float *gate, const float *up, int64_t n, float *y) {
    for (int64_t i = 0; i < n; i++) {
        float g = gate[i];
        y[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

void orc_attention(const float *q, const uint16_t *kc, const uint16_t *vc, int64_t T, int64_t pos0,
                   int64_t n_head, int64_t n_kv, int64_t hd, float *out) {
    int64_t group = n_head / n_kv;
    float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t t = 0; t < T; t++)
        for (int64_t h = 0; h < n_head; h++) {
            int64_t kvh = h / group, L = pos0 + t + 1;
            const float *qv = q + (t * n_head + h) * hd;
            float *s = (float *)malloc(sizeof(float) * (size_t)L);
            float mx = -INFINITY;
            for (int64_t p = 0; p < L; p++) {
                const uint16_t *kr = kc + (p * n_kv + kvh) * hd;
                float acc = 0.f;
                for (int64_t i = 0; i < hd; i++) acc += qv[i] * h2f(kr[i]);
                s[p] = acc * scale;
                if (s[p] > mx) mx = s[p];
            }
            double den = 0.0;
            for (int64_t p = 0; p < L; p++) {
                s[p] = expf(s[p] - mx);
                den += s[p];
            }
            float *o = out + (t * n_head + h) * hd;
            for (int64_t i = 0; i < hd; i++) o[i] = 0.f;
            for (int64_t p = 0; p < L; p++) {
                const uint16_t *vr = vc + (p * n_kv + kvh) * hd;
                float w = s[p];
                for (int64_t i = 0; i < hd; i++) o[i] += w * h2f(vr[i]);
            }
            float inv = (float)(1.0 / den);
            for (int64_t i = 0; i < hd; i++) o[i] *= inv;
            free(s);
        }
}

/* ---------------------------------------------------------------- KV-cache row formats */
void orc_quantize_q8_0(const float *x, int64_t n, uint8_t *blocks) {
    for (int64_t b = 0; b < n / 32; b++) {
        const float *xb = x + b * 32;
        uint8_t *blk = blocks + b * 34;
        float amax = 0.f;
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(xb[j]));
        const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
        const uint16_t dh = f2h(d);
        memcpy(blk, &dh, 2);
        for (int j = 0; j < 32; j++) blk[2 + j] = (uint8_t)(int8_t)roundf(xb[j] * id);
    }
}

void orc_quantize_q4_0(const float *x, int64_t n, uint8_t *blocks) {
    for (int64_t b = 0; b < n / 32; b++) {
        const float *xb = x + b * 32;
        uint8_t *blk = blocks + b * 18;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < 32; j++)
            if (amax < fabsf(xb[j])) {
                amax = fabsf(xb[j]);
                mx = xb[j];
            }
        const float d = mx / -8.f, id = d ? 1.f / d : 0.f;
        const uint16_t dh = f2h(d);
        memcpy(blk, &dh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)(int8_t)(xb[j] * id + 8.5f), q1 = (int)(int8_t)(xb[j + 16] * id + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            blk[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

void orc_dequant_q8_0(const uint8_t *blocks, int64_t nblocks, float *out) {
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 34;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        const float d = h2f(dh);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = (float)(int8_t)blk[2 + j] * d;
    }
}

void orc_dequant_q4_0(const uint8_t *blocks, int64_t nblocks, float *out) {
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 18;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        const float d = h2f(dh);
        for (int j = 0; j < 16; j++) {
            out[b * 32 + j] = (float)((int)(blk[2 + j] & 0x0F) - 8) * d;
            out[b * 32 + 16 + j] = (float)((int)(blk[2 + j] >> 4) - 8) * d;
        }
    }
}

void orc_kv_round_trip(int type, const float *x, int64_t n, uint16_t *y) {
    if (type == ORC_TYPE_Q8_0 || type == ORC_TYPE_Q4_0) {
        uint8_t *blk = (uint8_t *)malloc((size_t)(n / 32 * 34));
        float *f = (float *)malloc(sizeof(float) * (size_t)n);
        if (type == ORC_TYPE_Q8_0) {
            orc_quantize_q8_0(x, n, blk);
            orc_dequant_q8_0(blk, n / 32, f);
        } else {
            orc_quantize_q4_0(x, n, blk);
            orc_dequant_q4_0(blk, n / 32, f);
        }
        orc_f32_to_f16(f, n, y);
        free(f);
        free(blk);
    } else {
        orc_f32_to_f16(x, n, y);
    }
}

void orc_get_rows(int type, const uint8_t *W, const int32_t *ids, int64_t T, int64_t K, float *y) {
    int64_t rb = orc_row_bytes(type, K);
    for (int64_t t = 0; t < T; t++) {
        const uint8_t *row = W + (int64_t)ids[t] * rb;
        if (type == ORC_TYPE_Q4_K)
            orc_dequant_q4k(row, K / 256, y + t * K);
        else if (type == ORC_TYPE_Q6_K)
            orc_dequant_q6k(row, K / 256, y + t * K);
        else if (type == ORC_TYPE_F32)
            memcpy(y + t * K, row, (size_t)K * 4);
        else if (type == ORC_TYPE_F16)
            orc_f16_to_f32((const uint16_t *)row, K, y + t * K);
    }
}

void orc_argmax(const float *x, int64_t T, int64_t n, int32_t *idx) {
    for (int64_t t = 0; t < T; t++) {
        int64_t best = 0;
        for (int64_t i = 1; i < n; i++)
            if (x[t * n + i] > x[t * n + best]) best = i;
        idx[t] = (int32_t)best;
    }
}

/* Router of build_moe_ffn (third_party/llama.cpp/patches/0003-moe-add-expert-analysis-and-split-
 * tools.patch lines 82-108): probs = softmax over all experts; selection_probs = probs + mask, the
 * mask being 0 for an allowed expert and -inf for a masked one (lines 44-48 and 159-181: one bool per
 * expert, set on the model); top-k by selection_probs; the weights are the *unmasked* probs of the
 * selected experts, renormalised to sum 1.  Ties go to the lower expert index.  mask == NULL: all
 * experts allowed.  If fewer than k experts are allowed, masked ones fill the remaining slots in
 * index order (all their selection values are equal). */
void orc_moe_route_masked(const float *logits, int64_t T, int64_t E, int64_t k, const uint8_t *mask,
                          int32_t *ids, float *w) {
    float *p = (float *)malloc(sizeof(float) * (size_t)E);
    for (int64_t t = 0; t < T; t++) {
        const float *l = logits + t * E;
        float mx = l[0];
        for (int64_t e = 1; e < E; e++)
            if (l[e] > mx) mx = l[e];
        float den = 0.f;
        for (int64_t e = 0; e < E; e++) {
            p[e] = expf(l[e] - mx);
            den += p[e];
        }
        for (int64_t e = 0; e < E; e++) p[e] /= den;
        float wsum = 0.f;
        for (int64_t s = 0; s < k; s++) {
            int64_t best = -1;
            float best_sel = 0.f;
            for (int64_t e = 0; e < E; e++) {
                int taken = 0;
                for (int64_t u = 0; u < s; u++)
                    if (ids[t * k + u] == e) taken = 1;
                if (taken) continue;
                const float sel = (mask && !mask[e]) ? -INFINITY : p[e];
                if (best < 0 || sel > best_sel) {
                    best = e;
                    best_sel = sel;
                }
            }
            ids[t * k + s] = (int32_t)best;
            w[t * k + s] = p[best];
            wsum += p[best];
        }
        for (int64_t s = 0; s < k; s++) w[t * k + s] /= wsum;
    }
    free(p);
}

void orc_moe_route(const float *logits, int64_t T, int64_t E, int64_t k, int32_t *ids, float *w) {
    orc_moe_route_masked(logits, T, E, k, NULL, ids, w);
}

/* ---------------------------------------------------------------- whole stage */
typedef struct {
    char name[64];
    int32_t type;
    int64_t ne[3]; /* ne[0] contiguous */
    int64_t nbytes;
    void *data;
} orc_tensor;

struct orc_model {
    orc_config c;
    int n_tensors;
    orc_tensor *t;
    uint16_t *kc, *vc; /* [layer_local][seq][ctx][n_kv][hd] */
    uint8_t *expert_mask; /* one byte per expert (1 = allowed) or NULL: llama_model_set_expert_mask */
};

static orc_tensor *add_tensor(orc_model *m, const char *name, int type, int64_t ne0, int64_t ne1,
                              int64_t ne2) {
    m->t = (orc_tensor *)realloc(m->t, sizeof(orc_tensor) * (size_t)(m->n_tensors + 1));
    orc_tensor *t = &m->t[m->n_tensors++];
    memset(t, 0, sizeof(*t));
    snprintf(t->name, sizeof(t->name), "%s", name);
    t->type = type;
    t->ne[0] = ne0;
    t->ne[1] = ne1;
    t->ne[2] = ne2;
    t->nbytes = orc_row_bytes(type, ne0) * ne1 * ne2;
    t->data = calloc(1, (size_t)t->nbytes);
    return t;
}

static void add_layer_tensor(orc_model *m, int l, const char *what, int type, int64_t ne0,
                             int64_t ne1, int64_t ne2) {
    char name[64];
    snprintf(name, sizeof(name), "blk.%d.%s", l, what);
    add_tensor(m, name, type, ne0, ne1, ne2);
}

orc_model *orc_model_create(const orc_config *cfg) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->c = *cfg;
    const orc_config *c = &m->c;
    int64_t h = c->n_embd, hd = c->head_dim;
    int64_t nq = (int64_t)c->n_head * hd, nkv = (int64_t)c->n_head_kv * hd;
    if (c->has_embd) add_tensor(m, "token_embd.weight", ORC_TYPE_Q4_K, h, c->n_vocab, 1);
    for (int l = c->layer_begin; l < c->layer_end; l++) {
        int alt = (l & 1) ? ORC_TYPE_Q6_K : ORC_TYPE_Q4_K; /* attn_v / ffn_down on odd layers */
        add_layer_tensor(m, l, "attn_norm.weight", ORC_TYPE_F32, h, 1, 1);
        add_layer_tensor(m, l, "attn_q.weight", ORC_TYPE_Q4_K, h, nq, 1);
        add_layer_tensor(m, l, "attn_k.weight", ORC_TYPE_Q4_K, h, nkv, 1);
        add_layer_tensor(m, l, "attn_v.weight", alt, h, nkv, 1);
        add_layer_tensor(m, l, "attn_output.weight", ORC_TYPE_Q4_K, nq, h, 1);
        if (c->qkv_bias) {
            add_layer_tensor(m, l, "attn_q.bias", ORC_TYPE_F32, nq, 1, 1);
            add_layer_tensor(m, l, "attn_k.bias", ORC_TYPE_F32, nkv, 1, 1);
            add_layer_tensor(m, l, "attn_v.bias", ORC_TYPE_F32, nkv, 1, 1);
        }
        if (c->qk_norm) {
            add_layer_tensor(m, l, "attn_q_norm.weight", ORC_TYPE_F32, hd, 1, 1);
            add_layer_tensor(m, l, "attn_k_norm.weight", ORC_TYPE_F32, hd, 1, 1);
        }
        add_layer_tensor(m, l, "ffn_norm.weight", ORC_TYPE_F32, h, 1, 1);
        if (c->n_expert > 0) {
            int64_t fe = c->n_ff_exp, E = c->n_expert;
            add_layer_tensor(m, l, "ffn_gate_inp.weight", ORC_TYPE_F32, h, E, 1);
            add_layer_tensor(m, l, "ffn_gate_exps.weight", ORC_TYPE_Q4_K, h, fe, E);
            add_layer_tensor(m, l, "ffn_up_exps.weight", ORC_TYPE_Q4_K, h, fe, E);
            add_layer_tensor(m, l, "ffn_down_exps.weight", alt, fe, h, E);
        } else {
            add_layer_tensor(m, l, "ffn_gate.weight", ORC_TYPE_Q4_K, h, c->n_ff, 1);
            add_layer_tensor(m, l, "ffn_up.weight", ORC_TYPE_Q4_K, h, c->n_ff, 1);
            add_layer_tensor(m, l, "ffn_down.weight", alt, c->n_ff, h, 1);
        }
    }
    if (c->has_output) {
        add_tensor(m, "output_norm.weight", ORC_TYPE_F32, h, 1, 1);
        add_tensor(m, "output.weight", ORC_TYPE_Q6_K, h, c->n_vocab, 1);
    }
    int64_t nl = c->layer_end - c->layer_begin;
    size_t kv = (size_t)(nl * c->n_seq * c->n_ctx * nkv);
    m->kc = (uint16_t *)calloc(kv ? kv : 1, 2);
    m->vc = (uint16_t *)calloc(kv ? kv : 1, 2);
    return m;
}

void orc_model_free(orc_model *m) {
    if (!m) return;
    for (int i = 0; i < m->n_tensors; i++) free(m->t[i].data);
    free(m->t);
    free(m->kc);
    free(m->vc);
    free(m->expert_mask);
    free(m);
}

/* llama_model_set_expert_mask (patches/0003 lines 159-181): NULL clears; a mask whose length is not
 * the model's expert count is refused with -1. */
int orc_model_set_expert_mask(orc_model *m, const uint8_t *mask, int32_t n_mask) {
    if (!mask) {
        free(m->expert_mask);
        m->expert_mask = NULL;
        return 0;
    }
    if (n_mask != m->c.n_expert) return -1;
    if (!m->expert_mask) m->expert_mask = (uint8_t *)malloc((size_t)n_mask);
    for (int i = 0; i < n_mask; i++) m->expert_mask[i] = mask[i] ? 1 : 0;
    return 0;
}

int orc_model_n_tensors(orc_model *m) { return m->n_tensors; }
const char *orc_model_tensor_name(orc_model *m, int i) {
    return (i >= 0 && i < m->n_tensors) ? m->t[i].name : NULL;
}

static orc_tensor *find_tensor(orc_model *m, const char *name) {
    for (int i = 0; i < m->n_tensors; i++)
        if (strcmp(m->t[i].name, name) == 0) return &m->t[i];
    return NULL;
}

int orc_model_get_tensor(orc_model *m, const char *name, int32_t *type, const void **data,
                         int64_t *nbytes, int64_t ne[3]) {
    orc_tensor *t = find_tensor(m, name);
    if (!t) return 0;
    if (type) *type = t->type;
    if (data) *data = t->data;
    if (nbytes) *nbytes = t->nbytes;
    if (ne) memcpy(ne, t->ne, sizeof(t->ne));
    return 1;
}

int orc_model_set_tensor(orc_model *m, const char *name, int32_t type, const void *data,
                         int64_t nbytes) {
    orc_tensor *t = find_tensor(m, name);
    if (!t) return 0;
    if (type != t->type) { /* allow a different quantisation of the same shape */
        int64_t nb = orc_row_bytes(type, t->ne[0]) * t->ne[1] * t->ne[2];
        if (nb != nbytes) return 0;
        free(t->data);
        t->data = malloc((size_t)nb);
        t->type = type;
        t->nbytes = nb;
    }
    if (nbytes != t->nbytes) return 0;
    memcpy(t->data, data, (size_t)nbytes);
    return 1;
}

/* counter-based generator: value i of stream (seed, name) */
static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static uint64_t name_hash(const char *s) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (; *s; s++) h = (h ^ (uint8_t)*s) * 0x100000001B3ull;
    return h;
}
static inline float gauss_at(uint64_t key, uint64_t i) {
    uint64_t r = mix64(key + i * 0xD1342543DE82EF95ull);
    uint32_t a = (uint32_t)(r >> 32), b = (uint32_t)r;
    float u1 = ((float)(a >> 8) + 1.0f) * (1.0f / 16777216.0f); /* (0,1] */
    float u2 = (float)(b >> 8) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

void orc_model_generate(orc_model *m, uint64_t seed) {
    for (int ti = 0; ti < m->n_tensors; ti++) {
        orc_tensor *t = &m->t[ti];
        uint64_t key = mix64(seed ^ name_hash(t->name));
        int64_t n = t->ne[0] * t->ne[1] * t->ne[2];
        int is_norm = strstr(t->name, "norm.weight") != NULL;
        if (t->type == ORC_TYPE_F32) {
            float *f = (float *)t->data;
            for (int64_t i = 0; i < n; i++)
                f[i] = (is_norm ? 1.0f : 0.0f) + 0.02f * gauss_at(key, (uint64_t)i);
            continue;
        }
        /* quantise in slabs to bound the f32 scratch */
        int64_t slab = 1 << 22;
        float *buf = (float *)malloc(sizeof(float) * (size_t)(n < slab ? n : slab));
        int64_t bpb = t->type == ORC_TYPE_Q4_K ? ORC_Q4K_BYTES : ORC_Q6K_BYTES;
        for (int64_t o = 0; o < n; o += slab) {
            int64_t cnt = n - o < slab ? n - o : slab;
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < cnt; i++) buf[i] = 0.02f * gauss_at(key, (uint64_t)(o + i));
            uint8_t *dst = (uint8_t *)t->data + o / 256 * bpb;
            if (t->type == ORC_TYPE_Q4_K)
                orc_quantize_q4k(buf, cnt, dst);
            else
                orc_quantize_q6k(buf, cnt, dst);
        }
        free(buf);
    }
}

static orc_tensor *layer_tensor(orc_model *m, int l, const char *what) {
    char name[64];
    snprintf(name, sizeof(name), "blk.%d.%s", l, what);
    return find_tensor(m, name);
}

static void mm(const orc_tensor *w, const float *x, int64_t T, float *y) {
    orc_mul_mat(w->type, (const uint8_t *)w->data, x, T, w->ne[1], w->ne[0], y);
}

static void add_bias(float *y, const orc_tensor *b, int64_t T, int64_t n) {
    if (!b) return;
    const float *bv = (const float *)b->data;
    for (int64_t t = 0; t < T; t++)
        for (int64_t i = 0; i < n; i++) y[t * n + i] += bv[i];
}

int orc_model_forward(orc_model *m, int32_t seq, const int32_t *tokens, const float *hidden_in,
                      int64_t T, int64_t pos0, float *hidden_out, float *logits) {
    const orc_config *c = &m->c;
    int64_t h = c->n_embd, hd = c->head_dim, nh = c->n_head, nkvh = c->n_head_kv;
    int64_t nq = nh * hd, nkv = nkvh * hd;
    if (seq < 0 || seq >= c->n_seq || pos0 + T > c->n_ctx) return -1;
    float *x = (float *)malloc(sizeof(float) * (size_t)(T * h));
    float *xn = (float *)malloc(sizeof(float) * (size_t)(T * h));
    float *q = (float *)malloc(sizeof(float) * (size_t)(T * nq));
    float *k = (float *)malloc(sizeof(float) * (size_t)(T * nkv));
    float *v = (float *)malloc(sizeof(float) * (size_t)(T * nkv));
    float *att = (float *)malloc(sizeof(float) * (size_t)(T * nq));
    float *o = (float *)malloc(sizeof(float) * (size_t)(T * h));
    int64_t ff = c->n_expert > 0 ? c->n_ff_exp : c->n_ff;
    float *g = (float *)malloc(sizeof(float) * (size_t)(T * ff));
    float *u = (float *)malloc(sizeof(float) * (size_t)(T * ff));
    int32_t *pos = (int32_t *)malloc(sizeof(int32_t) * (size_t)T);
    for (int64_t t = 0; t < T; t++) pos[t] = (int32_t)(pos0 + t);

    if (c->has_embd) {
        if (!tokens) return -2;
        orc_tensor *te = find_tensor(m, "token_embd.weight");
        orc_get_rows(te->type, (const uint8_t *)te->data, tokens, T, h, x);
    } else {
        if (!hidden_in) return -2;
        memcpy(x, hidden_in, sizeof(float) * (size_t)(T * h));
    }

    for (int l = c->layer_begin; l < c->layer_end; l++) {
        int64_t ll = l - c->layer_begin;
        orc_rms_norm(x, (const float *)layer_tensor(m, l, "attn_norm.weight")->data, T, h,
                     c->rms_eps, xn);
        mm(layer_tensor(m, l, "attn_q.weight"), xn, T, q);
        mm(layer_tensor(m, l, "attn_k.weight"), xn, T, k);
        mm(layer_tensor(m, l, "attn_v.weight"), xn, T, v);
        if (c->qkv_bias) {
            add_bias(q, layer_tensor(m, l, "attn_q.bias"), T, nq);
            add_bias(k, layer_tensor(m, l, "attn_k.bias"), T, nkv);
            add_bias(v, layer_tensor(m, l, "attn_v.bias"), T, nkv);
        }
        if (c->qk_norm) {
            orc_rms_norm(q, (const float *)layer_tensor(m, l, "attn_q_norm.weight")->data, T * nh,
                         hd, c->rms_eps, q);
            orc_rms_norm(k, (const float *)layer_tensor(m, l, "attn_k_norm.weight")->data,
                         T * nkvh, hd, c->rms_eps, k);
        }
        orc_rope(q, pos, T, nh, hd, c->rope_theta, c->rope_neox);
        orc_rope(k, pos, T, nkvh, hd, c->rope_theta, c->rope_neox);
        uint16_t *kc = m->kc + ((ll * c->n_seq + seq) * c->n_ctx) * nkv;
        uint16_t *vc = m->vc + ((ll * c->n_seq + seq) * c->n_ctx) * nkv;
        orc_kv_round_trip(c->kv_type_k, k, T * nkv, kc + pos0 * nkv);
        orc_kv_round_trip(c->kv_type_v, v, T * nkv, vc + pos0 * nkv);
        orc_attention(q, kc, vc, T, pos0, nh, nkvh, hd, att);
        mm(layer_tensor(m, l, "attn_output.weight"), att, T, o);
        for (int64_t i = 0; i < T * h; i++) x[i] += o[i];

        orc_rms_norm(x, (const float *)layer_tensor(m, l, "ffn_norm.weight")->data, T, h,
                     c->rms_eps, xn);
        if (c->n_expert > 0) {
            int64_t E = c->n_expert, ku = c->n_expert_used, fe = c->n_ff_exp;
            const float *wr = (const float *)layer_tensor(m, l, "ffn_gate_inp.weight")->data;
            float *rl = (float *)malloc(sizeof(float) * (size_t)(T * E));
            int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * (size_t)(T * ku));
            float *rw = (float *)malloc(sizeof(float) * (size_t)(T * ku));
            for (int64_t t = 0; t < T; t++)
                for (int64_t e = 0; e < E; e++) {
                    float acc = 0.f;
                    for (int64_t i = 0; i < h; i++) acc += wr[e * h + i] * xn[t * h + i];
                    rl[t * E + e] = acc;
                }
            orc_moe_route_masked(rl, T, E, ku, m->expert_mask, ids, rw);
            orc_tensor *ge = layer_tensor(m, l, "ffn_gate_exps.weight");
            orc_tensor *ue = layer_tensor(m, l, "ffn_up_exps.weight");
            orc_tensor *de = layer_tensor(m, l, "ffn_down_exps.weight");
            int64_t gb = orc_row_bytes(ge->type, h) * fe, db = orc_row_bytes(de->type, fe) * h;
            float *ye = (float *)malloc(sizeof(float) * (size_t)h);
            for (int64_t t = 0; t < T; t++) {
                float *acc = o + t * h;
                for (int64_t i = 0; i < h; i++) acc[i] = 0.f;
                for (int64_t s = 0; s < ku; s++) {
                    int64_t e = ids[t * ku + s];
                    orc_mul_mat(ge->type, (const uint8_t *)ge->data + e * gb, xn + t * h, 1, fe, h, g);
                    orc_mul_mat(ue->type, (const uint8_t *)ue->data + e * gb, xn + t * h, 1, fe, h, u);
                    orc_swiglu(g, u, fe, g);
                    orc_mul_mat(de->type, (const uint8_t *)de->data + e * db, g, 1, h, fe, ye);
                    float w = rw[t * ku + s];
                    for (int64_t i = 0; i < h; i++) acc[i] += w * ye[i];
                }
            }
            free(ye);
            free(rl);
            free(ids);
            free(rw);
        } else {
            mm(layer_tensor(m, l, "ffn_gate.weight"), xn, T, g);
            mm(layer_tensor(m, l, "ffn_up.weight"), xn, T, u);
            orc_swiglu(g, u, T * ff, g);
            mm(layer_tensor(m, l, "ffn_down.weight"), g, T, o);
        }
        for (int64_t i = 0; i < T * h; i++) x[i] += o[i];
    }

    if (c->has_output && logits) {
        orc_rms_norm(x, (const float *)find_tensor(m, "output_norm.weight")->data, T, h, c->rms_eps,
                     xn);
        mm(find_tensor(m, "output.weight"), xn, T, logits);
    }
    if (hidden_out) memcpy(hidden_out, x, sizeof(float) * (size_t)(T * h));
    free(x); free(xn); free(q); free(k); free(v); free(att); free(o); free(g); free(u); free(pos);
    return 0;
}
