/*
 * zmoe_oracle.c -- scalar CPU restatement of the reference MoE expert path.
 * TEST INFRASTRUCTURE ONLY (see zmoe_oracle.h for what is pinned and how).
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -shared).
 */
#include "zmoe_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ */
/* block layouts (byte-exact; reference kernels/quant/kquant_matmul.cu:35-39,
 * kernels/quant/iq2_matmul.cu:27, backends/cpu/kernels_cpu.cpp:22-26)     */
/* ------------------------------------------------------------------ */
#pragma pack(push, 1)
typedef struct { uint8_t scales[16]; uint8_t qs[64]; uint16_t d, dmin; } blk_q2_K;      /* 84  */
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; } blk_q3_K; /* 110 */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_K;     /* 144 */
typedef struct { uint16_t d; uint16_t qs[32]; } blk_iq2_xxs;                            /* 66  */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_K;               /* 292 */
#pragma pack(pop)

_Static_assert(sizeof(blk_q2_K) == 84, "q2_K");
_Static_assert(sizeof(blk_q3_K) == 110, "q3_K");
_Static_assert(sizeof(blk_q4_K) == 144, "q4_K");
_Static_assert(sizeof(blk_iq2_xxs) == 66, "iq2_xxs");
_Static_assert(sizeof(blk_q8_K) == 292, "q8_K");

static const uint64_t iq2xxs_grid[256] = {
#include "iq2xxs_grid.inc"
};

/* sign byte for a 7-bit index: bit 7 makes the parity even */
static inline uint8_t ksign(uint32_t i) {
    i &= 127u;
    return (uint8_t)(i | ((uint32_t)(__builtin_popcount(i) & 1) << 7));
}

size_t zo_block_bytes(int type) {
    switch (type) {
    case ZO_TYPE_Q2_K: return 84;
    case ZO_TYPE_Q3_K: return 110;
    case ZO_TYPE_Q4_K: return 144;
    case ZO_TYPE_IQ2_XXS: return 66;
    default: return 0;
    }
}

float zo_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ------------------------------------------------------------------ */
/* Q8_K quantiser.  Published ggml rule (ggml-quants.c, quantize_row_q8_K_ref),
 * restated: the element of largest magnitude, WITH its sign, maps to -127;
 * iscale = -127/max; q = round-half-even(iscale*x) clipped above at 127;
 * d = 1/iscale; bsums are the sums of each 16 consecutive q.  An all-zero
 * block gives d = 0, q = 0 (bsums are written as 0 here).                */
/* ------------------------------------------------------------------ */
static inline int nearest_int(float f) {
    /* 1.5*2^23 trick == round-to-nearest-even for |f| < 2^22 */
    float v = f + 12582912.f;
    int32_t i;
    memcpy(&i, &v, 4);
    return (i & 0x007fffff) - 0x00400000;
}

void zo_quantize_row_q8_K(const float *x, void *vy, int64_t k) {
    blk_q8_K *y = (blk_q8_K *)vy;
    const int64_t nb = k / ZO_QK_K;
    for (int64_t b = 0; b < nb; ++b, x += ZO_QK_K) {
        float max = 0.f, amax = 0.f;
        for (int j = 0; j < ZO_QK_K; ++j) {
            const float ax = fabsf(x[j]);
            if (ax > amax) { amax = ax; max = x[j]; }
        }
        if (amax == 0.f) {
            y[b].d = 0.f;
            memset(y[b].qs, 0, ZO_QK_K);
            memset(y[b].bsums, 0, sizeof(y[b].bsums));
            continue;
        }
        const volatile float iscale_v = -127.f / max; /* volatile: forbid reassociation */
        const float iscale = iscale_v;
        for (int j = 0; j < ZO_QK_K; ++j) {
            const volatile float p = iscale * x[j];
            int v = nearest_int(p);
            y[b].qs[j] = (int8_t)(v > 127 ? 127 : v);
        }
        for (int g = 0; g < 16; ++g) {
            int s = 0;
            for (int t = 0; t < 16; ++t) s += y[b].qs[16 * g + t];
            y[b].bsums[g] = (int16_t)s;
        }
        y[b].d = 1.f / iscale;
    }
}

/* ------------------------------------------------------------------ */
/* scale unpacking                                                      */
/* ------------------------------------------------------------------ */
/* Q4_K 6-bit scale/min pair j (reference kernels/quant/kquant_matmul.cu:41-48) */
static inline void q4k_scale_min(int j, const uint8_t *s, int *sc, int *m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/* Q3_K sixteen 6-bit scales (reference kernels/quant/kquant_matmul.cu:163-175) */
static inline void q3k_scales(const uint8_t *s12, int8_t sc[16]) {
    uint32_t a0, a1, tmp, aux[4];
    memcpy(&a0, s12, 4);
    memcpy(&a1, s12 + 4, 4);
    memcpy(&tmp, s12 + 8, 4);
    aux[0] = (a0 & 0x0f0f0f0fu) | ((tmp & 0x03030303u) << 4);
    aux[1] = (a1 & 0x0f0f0f0fu) | (((tmp >> 2) & 0x03030303u) << 4);
    aux[2] = ((a0 >> 4) & 0x0f0f0f0fu) | (((tmp >> 4) & 0x03030303u) << 4);
    aux[3] = ((a1 >> 4) & 0x0f0f0f0fu) | (((tmp >> 6) & 0x03030303u) << 4);
    for (int k = 0; k < 16; ++k) sc[k] = (int8_t)(((aux[k >> 2] >> (8 * (k & 3))) & 0xff) - 32);
}

/* ------------------------------------------------------------------ */
/* integer element views: q[256] (weight integer before scaling), and per
 * sub-block integer scale.  Everything else is derived from these.       */
/* ------------------------------------------------------------------ */
/* Q2_K element e: n=e/128, j=(e%128)/32, l=e%32, q=(qs[32n+l]>>2j)&3, group e/16
 * (reference kernels/quant/kquant_matmul.cu:55-72) */
static void q2k_ints(const blk_q2_K *b, int q[256]) {
    for (int e = 0; e < 256; ++e) {
        const int n = e >> 7, j = (e & 127) >> 5, l = e & 31;
        q[e] = (b->qs[32 * n + l] >> (2 * j)) & 3;
    }
}
/* Q3_K (reference kernels/quant/kquant_matmul.cu:179-199): the high-bit plane
 * index is 4n+j and hmask is indexed by l only. */
static void q3k_ints(const blk_q3_K *b, int q[256]) {
    for (int e = 0; e < 256; ++e) {
        const int n = e >> 7, j = (e & 127) >> 5, l = e & 31;
        const int q2 = (b->qs[32 * n + l] >> (2 * j)) & 3;
        const int hb = (b->hmask[l] >> (4 * n + j)) & 1;
        q[e] = q2 - (hb ? 0 : 4);
    }
}
/* Q4_K (reference kernels/quant/kquant_matmul.cu:74-92) */
static void q4k_ints(const blk_q4_K *b, int q[256]) {
    for (int e = 0; e < 256; ++e) {
        const int c = e >> 6, l = e & 63;
        q[e] = l < 32 ? (b->qs[32 * c + l] & 0xF) : (b->qs[32 * c + l - 32] >> 4);
    }
}
/* IQ2_XXS (reference kernels/quant/iq2_matmul.cu:73-91): signed grid magnitude,
 * ls[ib32] = 4-bit scale */
static void iq2xxs_ints(const blk_iq2_xxs *b, int q[256], int ls[8]) {
    for (int ib = 0; ib < 8; ++ib) {
        const uint16_t *p = b->qs + 4 * ib;
        const uint32_t aux0 = (uint32_t)p[0] | ((uint32_t)p[1] << 16);
        const uint32_t aux1 = (uint32_t)p[2] | ((uint32_t)p[3] << 16);
        ls[ib] = (int)(aux1 >> 28);
        for (int l = 0; l < 4; ++l) {
            const uint64_t g = iq2xxs_grid[(aux0 >> (8 * l)) & 255];
            const uint8_t s = ksign(aux1 >> (7 * l));
            for (int j = 0; j < 8; ++j) {
                const int mag = (int)((g >> (8 * j)) & 255);
                q[32 * ib + 8 * l + j] = (s >> j) & 1 ? -mag : mag;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* dequantisers                                                         */
/* ------------------------------------------------------------------ */
void zo_dequantize_row(int type, const void *w, float *y, int64_t k) {
    const int64_t nb = k / ZO_QK_K;
    int q[256];
    for (int64_t i = 0; i < nb; ++i, y += 256) {
        if (type == ZO_TYPE_Q2_K) {
            const blk_q2_K *b = (const blk_q2_K *)w + i;
            const float d = zo_fp16_to_fp32(b->d), dmin = zo_fp16_to_fp32(b->dmin);
            q2k_ints(b, q);
            for (int e = 0; e < 256; ++e) {
                const uint8_t sc = b->scales[e >> 4];
                /* separate multiply and subtract, as the reference's scalar form
                 * (backends/cpu/kernels_cpu.hpp:85-98) */
                const volatile float dl = d * (float)(sc & 0xF);
                const volatile float ml = dmin * (float)(sc >> 4);
                const volatile float t = dl * (float)q[e];
                y[e] = t - ml;
            }
        } else if (type == ZO_TYPE_Q3_K) {
            const blk_q3_K *b = (const blk_q3_K *)w + i;
            const float d = zo_fp16_to_fp32(b->d);
            int8_t sc[16];
            q3k_scales(b->scales, sc);
            q3k_ints(b, q);
            for (int e = 0; e < 256; ++e) {
                const volatile float dl = d * (float)sc[e >> 4];
                y[e] = dl * (float)q[e];
            }
        } else if (type == ZO_TYPE_Q4_K) {
            const blk_q4_K *b = (const blk_q4_K *)w + i;
            const float d = zo_fp16_to_fp32(b->d), dmin = zo_fp16_to_fp32(b->dmin);
            q4k_ints(b, q);
            for (int e = 0; e < 256; ++e) {
                int sc, m;
                q4k_scale_min(e >> 5, b->scales, &sc, &m);
                const volatile float dl = d * (float)sc;
                const volatile float ml = dmin * (float)m;
                const volatile float t = dl * (float)q[e];
                y[e] = t - ml;
            }
        } else if (type == ZO_TYPE_IQ2_XXS) {
            const blk_iq2_xxs *b = (const blk_iq2_xxs *)w + i;
            const float d = zo_fp16_to_fp32(b->d);
            int ls[8];
            iq2xxs_ints(b, q, ls);
            for (int e = 0; e < 256; ++e) {
                const volatile float t = d * (0.5f + (float)ls[e >> 5]);
                const volatile float db = t * 0.25f;
                y[e] = db * (float)q[e];
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* per-block integer sums, split over the 8 float lanes the AVX2 kernels
 * use: lane = (e % 32) / 4.  lane sums add up to the block isum.        */
/* ------------------------------------------------------------------ */
static void block_lane_isums(int type, const void *wb, const blk_q8_K *y, int32_t lane[8]) {
    int q[256], sc[16];
    int shift; /* log2 elements per scale group */
    memset(lane, 0, 8 * sizeof(int32_t));
    if (type == ZO_TYPE_Q2_K) {
        const blk_q2_K *b = (const blk_q2_K *)wb;
        q2k_ints(b, q);
        for (int g = 0; g < 16; ++g) sc[g] = b->scales[g] & 0xF;
        shift = 4;
    } else if (type == ZO_TYPE_Q3_K) {
        const blk_q3_K *b = (const blk_q3_K *)wb;
        int8_t s8[16];
        q3k_ints(b, q);
        q3k_scales(b->scales, s8);
        for (int g = 0; g < 16; ++g) sc[g] = s8[g];
        shift = 4;
    } else if (type == ZO_TYPE_Q4_K) {
        const blk_q4_K *b = (const blk_q4_K *)wb;
        q4k_ints(b, q);
        for (int g = 0; g < 8; ++g) { int m; q4k_scale_min(g, b->scales, &sc[g], &m); }
        shift = 5;
    } else {
        const blk_iq2_xxs *b = (const blk_iq2_xxs *)wb;
        int ls[8];
        iq2xxs_ints(b, q, ls);
        for (int g = 0; g < 8; ++g) sc[g] = 2 * ls[g] + 1;
        shift = 5;
    }
    for (int e = 0; e < 256; ++e)
        lane[(e & 31) >> 2] += sc[e >> shift] * q[e] * (int)y->qs[e];
}

void zo_block_isums(int type, const void *wb, const void *q8, int32_t *isum, int32_t *msum) {
    const blk_q8_K *y = (const blk_q8_K *)q8;
    int32_t lane[8];
    block_lane_isums(type, wb, y, lane);
    int32_t s = 0;
    for (int l = 0; l < 8; ++l) s += lane[l];
    *isum = s;
    int32_t m = 0;
    if (type == ZO_TYPE_Q2_K) {
        const blk_q2_K *b = (const blk_q2_K *)wb;
        for (int g = 0; g < 16; ++g) m += (b->scales[g] >> 4) * (int)y->bsums[g];
    } else if (type == ZO_TYPE_Q4_K) {
        const blk_q4_K *b = (const blk_q4_K *)wb;
        for (int g = 0; g < 8; ++g) {
            int scv, mn;
            q4k_scale_min(g, b->scales, &scv, &mn);
            m += mn * ((int)y->bsums[2 * g] + (int)y->bsums[2 * g + 1]);
        }
    }
    *msum = m;
}

static inline float hsum8(const float a[8]) {
    const float t0 = a[4] + a[0], t1 = a[5] + a[1], t2 = a[6] + a[2], t3 = a[7] + a[3];
    const float u0 = t0 + t2, u1 = t1 + t3;
    return u0 + u1;
}

/* horizontal sum of reference backends/cpu/kernels_cpu.cpp:1965-1974 (adjacent pairs first) */
static inline float hsum8_pairs(const float a[8]) {
    const float t0 = a[0] + a[4], t1 = a[1] + a[5], t2 = a[2] + a[6], t3 = a[3] + a[7];
    const float s0 = t0 + t1, s2 = t2 + t3;
    return s0 + s2;
}

/* variant bit 0 clear: acc = fma(d, s, acc) as the AVX2 kernels with FMA3 do;
 *         bit 0 set:   separate multiply and add (reference backends/cpu/kernels_cpu.cpp:2066-2072)
 * variant bit 1 set:   final reduction in the order of the reference's IQ2_XXS prototype */
static float vec_dot_ex(int type, int n, const void *w, const void *q8, int variant) {
    const int fused = !(variant & 1);
    const int nb = n / ZO_QK_K;
    const size_t bb = zo_block_bytes(type);
    const blk_q8_K *y = (const blk_q8_K *)q8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float acc_m[4] = {0, 0, 0, 0};
    for (int i = 0; i < nb; ++i) {
        const uint8_t *wb = (const uint8_t *)w + (size_t)i * bb;
        int32_t lane[8];
        block_lane_isums(type, wb, &y[i], lane);
        float d;
        if (type == ZO_TYPE_Q2_K) {
            /* bench/q2k_dot_bench.cpp:39-61: mins first, then the scaled sums,
             * both into the same 8 lanes */
            const blk_q2_K *b = (const blk_q2_K *)wb;
            d = y[i].d * zo_fp16_to_fp32(b->d);
            const float dmin = -y[i].d * zo_fp16_to_fp32(b->dmin);
            for (int l = 0; l < 8; ++l) {
                const int32_t p = (b->scales[2 * l] >> 4) * (int)y[i].bsums[2 * l] +
                                  (b->scales[2 * l + 1] >> 4) * (int)y[i].bsums[2 * l + 1];
                acc[l] = fmaf(dmin, (float)p, acc[l]);
            }
        } else if (type == ZO_TYPE_Q3_K) {
            const blk_q3_K *b = (const blk_q3_K *)wb;
            d = y[i].d * zo_fp16_to_fp32(b->d);
        } else if (type == ZO_TYPE_Q4_K) {
            /* bench/q3k_q4k_dot_bench.cpp:80-120: mins in their own 4 lanes */
            const blk_q4_K *b = (const blk_q4_K *)wb;
            d = y[i].d * zo_fp16_to_fp32(b->d);
            const float dmin = -y[i].d * zo_fp16_to_fp32(b->dmin);
            for (int l = 0; l < 4; ++l) {
                int s0, m0, s1, m1;
                q4k_scale_min(2 * l, b->scales, &s0, &m0);
                q4k_scale_min(2 * l + 1, b->scales, &s1, &m1);
                const int32_t p = m0 * (int)(int16_t)(y[i].bsums[4 * l] + y[i].bsums[4 * l + 1]) +
                                  m1 * (int)(int16_t)(y[i].bsums[4 * l + 2] + y[i].bsums[4 * l + 3]);
                acc_m[l] = fmaf(dmin, (float)p, acc_m[l]);
            }
        } else {
            const blk_iq2_xxs *b = (const blk_iq2_xxs *)wb;
            d = zo_fp16_to_fp32(b->d) * y[i].d;
        }
        for (int l = 0; l < 8; ++l) {
            if (fused) {
                acc[l] = fmaf(d, (float)lane[l], acc[l]);
            } else {
                const volatile float p = d * (float)lane[l];
                acc[l] = p + acc[l];
            }
        }
    }
    if (type == ZO_TYPE_Q4_K) {
        const float r0 = acc_m[0] + acc_m[2], r1 = acc_m[1] + acc_m[3];
        return hsum8(acc) + (r0 + r1);
    }
    if (type == ZO_TYPE_IQ2_XXS) return 0.125f * ((variant & 2) ? hsum8_pairs(acc) : hsum8(acc));
    return hsum8(acc);
}

float zo_vec_dot_q8_K(int type, int n, const void *w, const void *q8) {
    return vec_dot_ex(type, n, w, q8, 0);
}
/* for the pins against the reference's IQ2_XXS prototype (see vec_dot_ex) */
float zo_vec_dot_q8_K_variant(int type, int n, const void *w, const void *q8, int variant) {
    return vec_dot_ex(type, n, w, q8, variant);
}

/* ------------------------------------------------------------------ */
/* matmul / mul_mat_id                                                  */
/* ------------------------------------------------------------------ */
void zo_matmul(int type, float *y, const float *x, const void *w, int S, int I, int O) {
    const int nb = I / ZO_QK_K;
    const size_t row_bytes = (size_t)nb * zo_block_bytes(type);
    blk_q8_K *xq = (blk_q8_K *)malloc((size_t)nb * sizeof(blk_q8_K));
    for (int s = 0; s < S; ++s) {
        zo_quantize_row_q8_K(x + (size_t)s * I, xq, I);
        for (int o = 0; o < O; ++o)
            y[(size_t)s * O + o] = zo_vec_dot_q8_K(type, I, (const uint8_t *)w + (size_t)o * row_bytes, xq);
    }
    free(xq);
}

void zo_mul_mat_id(int type, float *y, const float *x, const void *w, size_t expert_stride,
                   const int32_t *ids, int T, int K, int E, int I, int O, int x_per_route) {
    const int nb = I / ZO_QK_K;
    const size_t row_bytes = (size_t)nb * zo_block_bytes(type);
    blk_q8_K *xq = (blk_q8_K *)malloc((size_t)nb * sizeof(blk_q8_K));
    for (int t = 0; t < T; ++t) {
        for (int k = 0; k < K; ++k) {
            float *out = y + ((size_t)t * K + k) * O;
            const int e = ids[(size_t)t * K + k];
            if (e < 0 || e >= E) {
                const float v = e < 0 ? 0.f : NAN;
                for (int o = 0; o < O; ++o) out[o] = v;
                continue;
            }
            const float *xr = x + ((size_t)t * (x_per_route ? K : 1) + (x_per_route ? k : 0)) * I;
            zo_quantize_row_q8_K(xr, xq, I);
            const uint8_t *we = (const uint8_t *)w + (size_t)e * expert_stride;
            for (int o = 0; o < O; ++o)
                out[o] = zo_vec_dot_q8_K(type, I, we + (size_t)o * row_bytes, xq);
        }
    }
    free(xq);
}

/* ------------------------------------------------------------------ */
/* SwiGLU                                                               */
/* ------------------------------------------------------------------ */
void zo_swiglu(float *prod, const float *gate, const float *up, int n, float clamp, int fused) {
    for (int i = 0; i < n; ++i) {
        float g = gate[i], u = up[i], out;
        if (fused) {
            if (clamp > 0.f) {
                g = fminf(g, clamp);
                u = fmaxf(-clamp, fminf(clamp, u));
            }
            out = g / (1.0f + expf(-g)) * u;
        } else {
            g = g / (1.0f + expf(-g));
            out = g * u;
            if (clamp > 0.f) out = fmaxf(-clamp, fminf(clamp, out));
        }
        prod[i] = out;
    }
}

/* ------------------------------------------------------------------ */
/* router                                                               */
/* ------------------------------------------------------------------ */
void zo_router_logits(float *logits, const float *x, const float *wr, int T, int D, int E) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < T; ++t)
        for (int e = 0; e < E; ++e) {
            double a = 0.0;
            for (int d = 0; d < D; ++d) a += (double)x[(size_t)t * D + d] * (double)wr[(size_t)e * D + d];
            logits[(size_t)t * E + e] = (float)a;
        }
}

static void gating_row(int gating, float *row, int n) {
    if (gating == 1) {
        for (int e = 0; e < n; ++e) row[e] = 1.0f / (1.0f + expf(-row[e]));
    } else if (gating == 2) {
        for (int e = 0; e < n; ++e) {
            const float x = row[e];
            const float sp = x > 0.f ? x + log1pf(expf(-x)) : log1pf(expf(x));
            row[e] = sqrtf(sp);
        }
    } else {
        float mx = row[0];
        for (int e = 1; e < n; ++e) mx = fmaxf(mx, row[e]);
        float sum = 0.f;
        for (int e = 0; e < n; ++e) { row[e] = expf(row[e] - mx); sum += row[e]; }
        const float inv = 1.0f / sum;
        for (int e = 0; e < n; ++e) row[e] *= inv;
    }
}

/* selection scores of one token after bias and group limiting */
static void selection_row(const zo_router_spec *sp, const float *probs, const float *bias, float *sel) {
    const int E = sp->n_experts;
    for (int e = 0; e < E; ++e) sel[e] = probs[e] + (bias ? bias[e] : 0.f);
    if (sp->n_groups > 1 && sp->n_groups_used > 0 && sp->n_groups_used < sp->n_groups &&
        E % sp->n_groups == 0) {
        const int G = sp->n_groups, gs = E / G;
        float *score = (float *)malloc(sizeof(float) * (size_t)G);
        char *keep = (char *)calloc((size_t)G, 1);
        for (int g = 0; g < G; ++g) {
            float first = -INFINITY, second = -INFINITY;
            for (int j = 0; j < gs; ++j) {
                const float s = sel[g * gs + j];
                if (s > first) { second = first; first = s; }
                else if (s > second) second = s;
            }
            score[g] = first + second;
        }
        for (int u = 0; u < sp->n_groups_used; ++u) {
            int best = -1;
            for (int g = 0; g < G; ++g)
                if (!keep[g] && (best < 0 || score[g] > score[best])) best = g;
            keep[best] = 1;
        }
        for (int e = 0; e < E; ++e)
            if (!keep[e / gs]) sel[e] = -INFINITY;
        free(score);
        free(keep);
    }
}

void zo_router_select(const zo_router_spec *sp, float *probs, const float *bias,
                      int32_t *ids, float *weights, int T) {
    const int E = sp->n_experts, K = sp->topk;
    float *sel = (float *)malloc(sizeof(float) * (size_t)E);
    char *taken = (char *)malloc((size_t)E);
    for (int t = 0; t < T; ++t) {
        float *row = probs + (size_t)t * E;
        gating_row(sp->gating, row, E);
        selection_row(sp, row, bias, sel);
        memset(taken, 0, (size_t)E);
        float sum_w = 0.f;
        for (int k = 0; k < K; ++k) {
            int best = -1;
            for (int e = 0; e < E; ++e)
                if (!taken[e] && (best < 0 || sel[e] > sel[best])) best = e;
            taken[best] = 1;
            ids[(size_t)t * K + k] = best;
            weights[(size_t)t * K + k] = row[best];
            sum_w += row[best];
        }
        if (sp->normalize) {
            const float inv = 1.0f / fmaxf(sum_w, 6.103515625e-5f);
            for (int k = 0; k < K; ++k) weights[(size_t)t * K + k] *= inv;
        }
        if (sp->weight_scale != 0.0f)
            for (int k = 0; k < K; ++k) weights[(size_t)t * K + k] *= sp->weight_scale;
    }
    free(sel);
    free(taken);
}

float zo_router_min_margin(const zo_router_spec *sp, const float *probs, const float *bias, int T) {
    const int E = sp->n_experts, K = sp->topk;
    float *sel = (float *)malloc(sizeof(float) * (size_t)E);
    float margin = INFINITY;
    for (int t = 0; t < T; ++t) {
        selection_row(sp, probs + (size_t)t * E, bias, sel);
        /* selection sort of the first K+1 */
        for (int k = 0; k <= K && k < E; ++k) {
            int best = k;
            for (int e = k + 1; e < E; ++e) if (sel[e] > sel[best]) best = e;
            const float tmp = sel[k]; sel[k] = sel[best]; sel[best] = tmp;
            if (k > 0 && isfinite(sel[k]) && isfinite(sel[k - 1])) {
                const float gap = (sel[k - 1] - sel[k]) / fmaxf(fabsf(sel[k - 1]), 1e-30f);
                if (gap < margin) margin = gap;
            }
        }
    }
    free(sel);
    return margin;
}

void zo_group_by_expert(const int32_t *ids, int T, int K, int E, int32_t *offs, int32_t *slot) {
    int32_t *cursor = (int32_t *)calloc((size_t)E + 1, sizeof(int32_t));
    memset(offs, 0, sizeof(int32_t) * ((size_t)E + 1));
    for (int p = 0; p < T * K; ++p)
        if (ids[p] >= 0 && ids[p] < E) offs[ids[p] + 1]++;
    for (int e = 0; e < E; ++e) offs[e + 1] += offs[e];
    memcpy(cursor, offs, sizeof(int32_t) * (size_t)E);
    for (int p = 0; p < T * K; ++p)
        if (ids[p] >= 0 && ids[p] < E) slot[cursor[ids[p]]++] = p;
    free(cursor);
}

void zo_combine(float *out, const float *y, const float *weights, int T, int K, int D) {
    for (int t = 0; t < T; ++t)
        for (int d = 0; d < D; ++d) {
            /* ggml: MUL(expert_out, w) then k-ordered ADDs of the products */
            float acc = weights[(size_t)t * K] * y[((size_t)t * K) * D + d];
            for (int k = 1; k < K; ++k) {
                const volatile float p = weights[(size_t)t * K + k] * y[((size_t)t * K + k) * D + d];
                acc = acc + p;
            }
            out[(size_t)t * D + d] = acc;
        }
}

/* ------------------------------------------------------------------ */
/* layer                                                                */
/* ------------------------------------------------------------------ */
int zo_moe_ffn(const zo_layer *L, const float *x, const int32_t *ids, const float *weights,
               int T, float *out, float *dbg_act) {
    const int D = L->D, F = L->F, K = L->K, P = T * K;
    if (D % 256 || F % 256) return -1;
    float *gate = (float *)malloc(sizeof(float) * (size_t)P * F);
    float *up = (float *)malloc(sizeof(float) * (size_t)P * F);
    float *act = (float *)malloc(sizeof(float) * (size_t)P * F);
    float *down = (float *)malloc(sizeof(float) * (size_t)P * D);
    if (!gate || !up || !act || !down) return -2;
    zo_mul_mat_id(L->type_up, up, x, L->w_up, L->stride_up, ids, T, K, L->E, D, F, 0);
    zo_mul_mat_id(L->type_gate, gate, x, L->w_gate, L->stride_gate, ids, T, K, L->E, D, F, 0);
    zo_swiglu(act, gate, up, P * F, L->clamp, L->clamp_fused);
    if (dbg_act) memcpy(dbg_act, act, sizeof(float) * (size_t)P * F);
    zo_mul_mat_id(L->type_down, down, act, L->w_down, L->stride_down, ids, T, K, L->E, F, D, 1);
    zo_combine(out, down, weights, T, K, D);
    free(gate); free(up); free(act); free(down);
    return 0;
}
