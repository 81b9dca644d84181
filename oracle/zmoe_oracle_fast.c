/*
 * zmoe_oracle_fast.c -- the timed CPU baseline: the same arithmetic as
 * zmoe_oracle.c with vector integer dots (AVX-512 VNNI where the CPU has it,
 * else AVX2, else scalar) and OpenMP over weight rows.
 * TEST / BENCHMARK INFRASTRUCTURE ONLY; never linked into the shipped library.
 *
 * The AVX2 forms follow what the reference's CPU path runs: the pinned
 * ggml uses its AVX2 kernels for these types on x86 (reference
 * bench/q2k_dot_bench.cpp:33 labels the Q2_K one "stock"; bench/q3k_q4k_dot_bench.cpp:1-3).
 * Rows are grouped by expert like reference core/batched_dispatch_pipeline.cpp:1185-1204.
 * Every dot here is checked bit-for-bit against the scalar zo_vec_dot_q8_K.
 */
#include "zmoe_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#pragma pack(push, 1)
typedef struct { uint8_t scales[16]; uint8_t qs[64]; uint16_t d, dmin; } blk_q2_K;
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; } blk_q3_K;
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_K;
typedef struct { uint16_t d; uint16_t qs[32]; } blk_iq2_xxs;
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_K;
#pragma pack(pop)

static const uint64_t iq2xxs_grid[256] = {
#include "iq2xxs_grid.inc"
};
static uint64_t sign_bytes[128]; /* +1 / -1 per element, from the parity rule */
static int sign_ready = 0;

static void init_signs(void) {
    if (sign_ready) return;
    for (uint32_t i = 0; i < 128; ++i) {
        const uint32_t s = i | ((uint32_t)(__builtin_popcount(i) & 1) << 7);
        uint64_t v = 0;
        for (int j = 0; j < 8; ++j) v |= (uint64_t)(((s >> j) & 1) ? 0xffu : 0x01u) << (8 * j);
        sign_bytes[i] = v;
    }
    sign_ready = 1;
}

int zo_have_avx2(void) {
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}

#define TGT __attribute__((target("avx2,fma")))

TGT static inline float hsum8v(__m256 x) {
    __m128 r = _mm_add_ps(_mm256_extractf128_ps(x, 1), _mm256_castps256_ps128(x));
    r = _mm_add_ps(r, _mm_movehl_ps(r, r));
    r = _mm_add_ss(r, _mm_movehdup_ps(r));
    return _mm_cvtss_f32(r);
}

TGT static inline __m256i scale_pair(int lo, int hi) {
    return _mm256_set_m128i(_mm_set1_epi16((short)hi), _mm_set1_epi16((short)lo));
}

TGT static float dot_q2k(int n, const blk_q2_K *x, const blk_q8_K *y) {
    const __m256i m3 = _mm256_set1_epi8(3);
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        const float dmin = -y[i].d * zo_fp16_to_fp32(x[i].dmin);
        const __m128i sb = _mm_loadu_si128((const __m128i *)x[i].scales);
        const __m128i mn8 = _mm_and_si128(_mm_srli_epi16(sb, 4), _mm_set1_epi8(0xF));
        const __m256i pm = _mm256_madd_epi16(_mm256_cvtepi8_epi16(mn8),
                                             _mm256_loadu_si256((const __m256i *)y[i].bsums));
        acc = _mm256_fmadd_ps(_mm256_set1_ps(dmin), _mm256_cvtepi32_ps(pm), acc);
        __m256i sumi = _mm256_setzero_si256();
        for (int h = 0; h < 2; ++h) {
            const __m256i qb = _mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * h));
            for (int j = 0; j < 4; ++j) {
                const __m256i q = _mm256_and_si256(_mm256_srli_epi16(qb, 2 * j), m3);
                const __m256i a = _mm256_loadu_si256((const __m256i *)(y[i].qs + 128 * h + 32 * j));
                const __m256i p = _mm256_maddubs_epi16(q, a);
                const int g = 8 * h + 2 * j;
                sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(
                    scale_pair(x[i].scales[g] & 0xF, x[i].scales[g + 1] & 0xF), p));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum8v(acc);
}

static inline void q3k_scales16(const uint8_t *s12, int8_t sc[16]) {
    uint32_t a0, a1, tmp, aux[4];
    memcpy(&a0, s12, 4); memcpy(&a1, s12 + 4, 4); memcpy(&tmp, s12 + 8, 4);
    aux[0] = (a0 & 0x0f0f0f0fu) | ((tmp & 0x03030303u) << 4);
    aux[1] = (a1 & 0x0f0f0f0fu) | (((tmp >> 2) & 0x03030303u) << 4);
    aux[2] = ((a0 >> 4) & 0x0f0f0f0fu) | (((tmp >> 4) & 0x03030303u) << 4);
    aux[3] = ((a1 >> 4) & 0x0f0f0f0fu) | (((tmp >> 6) & 0x03030303u) << 4);
    for (int k = 0; k < 16; ++k) sc[k] = (int8_t)(((aux[k >> 2] >> (8 * (k & 3))) & 0xff) - 32);
}

TGT static float dot_q3k(int n, const blk_q3_K *x, const blk_q8_K *y) {
    const __m256i m3 = _mm256_set1_epi8(3), one = _mm256_set1_epi8(1);
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        int8_t sc[16];
        q3k_scales16(x[i].scales, sc);
        const __m256i hm = _mm256_loadu_si256((const __m256i *)x[i].hmask);
        __m256i sumi = _mm256_setzero_si256();
        for (int h = 0; h < 2; ++h) {
            const __m256i qb = _mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * h));
            for (int j = 0; j < 4; ++j) {
                const __m256i q = _mm256_and_si256(_mm256_srli_epi16(qb, 2 * j), m3);
                const __m256i hb = _mm256_and_si256(_mm256_srli_epi16(hm, 4 * h + j), one);
                const __m256i off = _mm256_slli_epi16(_mm256_xor_si256(hb, one), 2); /* 4 where bit clear */
                const __m256i a = _mm256_loadu_si256((const __m256i *)(y[i].qs + 128 * h + 32 * j));
                const __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(q, a), _mm256_maddubs_epi16(off, a));
                const int g = 8 * h + 2 * j;
                sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(scale_pair(sc[g], sc[g + 1]), p));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum8v(acc);
}

static inline void q4k_sm(int j, const uint8_t *s, int *sc, int *m) {
    if (j < 4) { *sc = s[j] & 63; *m = s[j + 4] & 63; }
    else { *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4); *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

TGT static float dot_q4k(int n, const blk_q4_K *x, const blk_q8_K *y) {
    const __m256i m4 = _mm256_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    float am[4] = {0, 0, 0, 0};
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        const float dmin = -y[i].d * zo_fp16_to_fp32(x[i].dmin);
        int sc[8], mn[8];
        for (int j = 0; j < 8; ++j) q4k_sm(j, x[i].scales, &sc[j], &mn[j]);
        for (int l = 0; l < 4; ++l) {
            const int p = mn[2 * l] * (int)(int16_t)(y[i].bsums[4 * l] + y[i].bsums[4 * l + 1]) +
                          mn[2 * l + 1] * (int)(int16_t)(y[i].bsums[4 * l + 2] + y[i].bsums[4 * l + 3]);
            am[l] = fmaf(dmin, (float)p, am[l]);
        }
        __m256i sumi = _mm256_setzero_si256();
        for (int c = 0; c < 4; ++c) {
            const __m256i qb = _mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * c));
            const __m256i lo = _mm256_and_si256(qb, m4);
            const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4);
            const __m256i al = _mm256_loadu_si256((const __m256i *)(y[i].qs + 64 * c));
            const __m256i ah = _mm256_loadu_si256((const __m256i *)(y[i].qs + 64 * c + 32));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16((short)sc[2 * c]), _mm256_maddubs_epi16(lo, al)));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16((short)sc[2 * c + 1]), _mm256_maddubs_epi16(hi, ah)));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum8v(acc) + ((am[0] + am[2]) + (am[1] + am[3]));
}

TGT static float dot_iq2xxs(int n, const blk_iq2_xxs *x, const blk_q8_K *y) {
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < n / 256; ++i) {
        const float d = zo_fp16_to_fp32(x[i].d) * y[i].d;
        __m256i sumi = _mm256_setzero_si256();
        for (int ib = 0; ib < 8; ++ib) {
            uint32_t a0, a1;
            memcpy(&a0, x[i].qs + 4 * ib, 4);
            memcpy(&a1, x[i].qs + 4 * ib + 2, 4);
            const __m256i g = _mm256_set_epi64x((long long)iq2xxs_grid[(a0 >> 24) & 255], (long long)iq2xxs_grid[(a0 >> 16) & 255],
                                                (long long)iq2xxs_grid[(a0 >> 8) & 255], (long long)iq2xxs_grid[a0 & 255]);
            const __m256i s = _mm256_set_epi64x((long long)sign_bytes[(a1 >> 21) & 127], (long long)sign_bytes[(a1 >> 14) & 127],
                                                (long long)sign_bytes[(a1 >> 7) & 127], (long long)sign_bytes[a1 & 127]);
            const __m256i a = _mm256_loadu_si256((const __m256i *)(y[i].qs + 32 * ib));
            const __m256i p = _mm256_maddubs_epi16(g, _mm256_sign_epi8(a, s));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(p, _mm256_set1_epi16((short)(2 * (a1 >> 28) + 1))));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return 0.125f * hsum8v(acc);
}

/* ---------------------------------------------------------------------------------------------------
 * AVX-512 VNNI forms of the K-quant dots.  The integer part runs on 64 bytes at a time with vpdpbusd; its 16 int32
 * lanes fold onto the 8 lanes the AVX2 form keeps (lane l and lane l + 8 hold the same four element positions of
 * two adjacent 32-element planes), so the int32 vector that is converted and accumulated in f32 is the same vector,
 * and the result is bit-identical to the AVX2 form and to the scalar oracle.
 * ------------------------------------------------------------------------------------------------- */
#define TGT512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni,avx2,fma")))

static int force_kind = -1;   /* tests: 0 scalar, 1 AVX2, 2 AVX-512 VNNI; -1 the best the CPU has */
int zo_fast_kind(void) {
    int best = 0;
    if (zo_have_avx2()) best = 1;
    if (best == 1 && __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
        __builtin_cpu_supports("avx512vl") && __builtin_cpu_supports("avx512vnni"))
        best = 2;
    return force_kind >= 0 && force_kind < best ? force_kind : best;
}
void zo_fast_force(int kind) { force_kind = kind; }

TGT512 static inline __m256i fold512(__m512i v) {
    return _mm256_add_epi32(_mm512_castsi512_si256(v), _mm512_extracti64x4_epi64(v, 1));
}
/* 16-bit shift counts: `lo` in the low 256 bits, `hi` in the high 256 bits */
TGT512 static inline __m512i shift_pair(int lo, int hi) {
    return _mm512_inserti64x4(_mm512_set1_epi16((short)lo), _mm256_set1_epi16((short)hi), 1);
}

TGT512 static float dot_q2k_vnni(int n, const blk_q2_K *x, const blk_q8_K *y) {
    const __m512i m3 = _mm512_set1_epi8(3);
    /* 16-bit lane l of plane pair jp takes the scale of group g0 + l / 8 */
    const __m512i grp = _mm512_srli_epi16(_mm512_set_epi16(31, 30, 29, 28, 27, 26, 25, 24, 23, 22, 21, 20, 19, 18, 17, 16, 15, 14,
                                                           13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0), 3);
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        const float dmin = -y[i].d * zo_fp16_to_fp32(x[i].dmin);
        const __m128i sb = _mm_loadu_si128((const __m128i *)x[i].scales);
        const __m128i mn8 = _mm_and_si128(_mm_srli_epi16(sb, 4), _mm_set1_epi8(0xF));
        const __m256i pm = _mm256_madd_epi16(_mm256_cvtepi8_epi16(mn8),
                                             _mm256_loadu_si256((const __m256i *)y[i].bsums));
        acc = _mm256_fmadd_ps(_mm256_set1_ps(dmin), _mm256_cvtepi32_ps(pm), acc);
        /* the sixteen 4-bit scales as 16-bit values */
        const __m512i sc16 = _mm512_castsi256_si512(_mm256_cvtepu8_epi16(_mm_and_si128(sb, _mm_set1_epi8(0xF))));
        __m512i sumi = _mm512_setzero_si512();
        for (int h = 0; h < 2; ++h) {
            const __m512i qb = _mm512_broadcast_i64x4(_mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * h)));
            for (int jp = 0; jp < 2; ++jp) {
                /* planes j = 2 jp (low half) and 2 jp + 1 (high half); two bytes of a 16-bit lane share a group,
                 * and 3 * 15 fits a byte, so one 16-bit multiply scales both */
                const __m512i q = _mm512_and_si512(_mm512_srlv_epi16(qb, shift_pair(4 * jp, 4 * jp + 2)), m3);
                const __m512i sc = _mm512_permutexvar_epi16(_mm512_add_epi16(grp, _mm512_set1_epi16((short)(8 * h + 4 * jp))), sc16);
                const __m512i a = _mm512_loadu_si512((const void *)(y[i].qs + 128 * h + 64 * jp));
                sumi = _mm512_dpbusd_epi32(sumi, _mm512_mullo_epi16(q, sc), a);
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(fold512(sumi)), acc);
    }
    return hsum8v(acc);
}

TGT512 static float dot_q3k_vnni(int n, const blk_q3_K *x, const blk_q8_K *y) {
    const __m512i m3 = _mm512_set1_epi8(3), one = _mm512_set1_epi8(1), four = _mm512_set1_epi8(4);
    const __m512i grp = _mm512_srli_epi32(_mm512_set_epi32(15, 14, 13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0), 2);
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        int8_t sc[16];
        q3k_scales16(x[i].scales, sc);
        const __m512i sc32 = _mm512_cvtepi8_epi32(_mm_loadu_si128((const __m128i *)sc));
        const __m512i hm = _mm512_broadcast_i64x4(_mm256_loadu_si256((const __m256i *)x[i].hmask));
        __m512i sumi = _mm512_setzero_si512();
        for (int h = 0; h < 2; ++h) {
            const __m512i qb = _mm512_broadcast_i64x4(_mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * h)));
            for (int jp = 0; jp < 2; ++jp) {
                const __m512i q2 = _mm512_and_si512(_mm512_srlv_epi16(qb, shift_pair(4 * jp, 4 * jp + 2)), m3);
                const __m512i hb = _mm512_and_si512(_mm512_srlv_epi16(hm, shift_pair(4 * h + 2 * jp, 4 * h + 2 * jp + 1)), one);
                const __m512i q = _mm512_or_si512(q2, _mm512_slli_epi16(hb, 2));      /* 0 .. 7 */
                const __m512i a = _mm512_loadu_si512((const void *)(y[i].qs + 128 * h + 64 * jp));
                /* (q - 4) . a per four elements, times the signed 6-bit scale of the lane's group */
                const __m512i dp = _mm512_sub_epi32(_mm512_dpbusd_epi32(_mm512_setzero_si512(), q, a),
                                                    _mm512_dpbusd_epi32(_mm512_setzero_si512(), four, a));
                const __m512i scl = _mm512_permutexvar_epi32(_mm512_add_epi32(grp, _mm512_set1_epi32(8 * h + 4 * jp)), sc32);
                sumi = _mm512_add_epi32(sumi, _mm512_mullo_epi32(dp, scl));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(fold512(sumi)), acc);
    }
    return hsum8v(acc);
}

TGT512 static float dot_q4k_vnni(int n, const blk_q4_K *x, const blk_q8_K *y) {
    const __m512i m4 = _mm512_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    float am[4] = {0, 0, 0, 0};
    for (int i = 0; i < n / 256; ++i) {
        const float d = y[i].d * zo_fp16_to_fp32(x[i].d);
        const float dmin = -y[i].d * zo_fp16_to_fp32(x[i].dmin);
        int sc[8], mn[8];
        for (int j = 0; j < 8; ++j) q4k_sm(j, x[i].scales, &sc[j], &mn[j]);
        for (int l = 0; l < 4; ++l) {
            const int p = mn[2 * l] * (int)(int16_t)(y[i].bsums[4 * l] + y[i].bsums[4 * l + 1]) +
                          mn[2 * l + 1] * (int)(int16_t)(y[i].bsums[4 * l + 2] + y[i].bsums[4 * l + 3]);
            am[l] = fmaf(dmin, (float)p, am[l]);
        }
        __m512i sumi = _mm512_setzero_si512();
        for (int c = 0; c < 4; ++c) {
            /* low nibbles (elements 64c .. 64c+31) in the low half, high nibbles (64c+32 ..) in the high half */
            const __m512i qb = _mm512_broadcast_i64x4(_mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * c)));
            const __m512i q = _mm512_and_si512(_mm512_srlv_epi16(qb, shift_pair(0, 4)), m4);
            const __m512i a = _mm512_loadu_si512((const void *)(y[i].qs + 64 * c));
            const __m512i dp = _mm512_dpbusd_epi32(_mm512_setzero_si512(), q, a);
            const __m512i scl = _mm512_inserti64x4(_mm512_set1_epi32(sc[2 * c]), _mm256_set1_epi32(sc[2 * c + 1]), 1);
            sumi = _mm512_add_epi32(sumi, _mm512_mullo_epi32(dp, scl));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(fold512(sumi)), acc);
    }
    return hsum8v(acc) + ((am[0] + am[2]) + (am[1] + am[3]));
}

/* exported for the bit-exactness test against the scalar oracle */
float zo_vec_dot_q8_K_fast(int type, int n, const void *w, const void *q8) {
    const int kind = zo_fast_kind();
    if (kind == 0) return zo_vec_dot_q8_K(type, n, w, q8);
    init_signs();
    if (kind == 2) {
        switch (type) {
        case ZO_TYPE_Q2_K: return dot_q2k_vnni(n, (const blk_q2_K *)w, (const blk_q8_K *)q8);
        case ZO_TYPE_Q3_K: return dot_q3k_vnni(n, (const blk_q3_K *)w, (const blk_q8_K *)q8);
        case ZO_TYPE_Q4_K: return dot_q4k_vnni(n, (const blk_q4_K *)w, (const blk_q8_K *)q8);
        default: break;   /* IQ2_XXS: the table lookups dominate; the AVX2 form serves */
        }
    }
    switch (type) {
    case ZO_TYPE_Q2_K: return dot_q2k(n, (const blk_q2_K *)w, (const blk_q8_K *)q8);
    case ZO_TYPE_Q3_K: return dot_q3k(n, (const blk_q3_K *)w, (const blk_q8_K *)q8);
    case ZO_TYPE_Q4_K: return dot_q4k(n, (const blk_q4_K *)w, (const blk_q8_K *)q8);
    case ZO_TYPE_IQ2_XXS: return dot_iq2xxs(n, (const blk_iq2_xxs *)w, (const blk_q8_K *)q8);
    default: return NAN;
    }
}

int zo_moe_ffn_fast(const zo_layer *L, const float *x, const int32_t *ids, const float *weights,
                    int T, float *out, int n_threads) {
    const int D = L->D, F = L->F, K = L->K, E = L->E, P = T * K;
    const int nbD = D / 256, nbF = F / 256;
    init_signs();
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_num_procs();
#else
    n_threads = 1;
#endif
    blk_q8_K *xq = (blk_q8_K *)malloc(sizeof(blk_q8_K) * (size_t)T * nbD);
    blk_q8_K *aq = (blk_q8_K *)malloc(sizeof(blk_q8_K) * (size_t)P * nbF);
    float *act = (float *)malloc(sizeof(float) * (size_t)P * F);
    float *down = (float *)malloc(sizeof(float) * (size_t)P * D);
    int32_t *offs = (int32_t *)malloc(sizeof(int32_t) * ((size_t)E + 1));
    int32_t *slot = (int32_t *)malloc(sizeof(int32_t) * (size_t)(P > 0 ? P : 1));
    int32_t *active = (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
    zo_group_by_expert(ids, T, K, E, offs, slot);
    int na = 0;
    for (int e = 0; e < E; ++e) if (offs[e + 1] > offs[e]) active[na++] = e;
    const size_t rb_g = (size_t)nbD * zo_block_bytes(L->type_gate);
    const size_t rb_u = (size_t)nbD * zo_block_bytes(L->type_up);
    const size_t rb_d = (size_t)nbF * zo_block_bytes(L->type_down);

#pragma omp parallel num_threads(n_threads)
    {
#pragma omp for schedule(static)
        for (int t = 0; t < T; ++t) zo_quantize_row_q8_K(x + (size_t)t * D, xq + (size_t)t * nbD, D);
        /* rows with a negative or out-of-range id keep zeros / NaN */
#pragma omp for schedule(static)
        for (int p = 0; p < P; ++p) {
            const int e = ids[p];
            if (e < 0 || e >= E) {
                const float v = e < 0 ? 0.f : NAN;
                for (int d = 0; d < D; ++d) down[(size_t)p * D + d] = v;
            }
        }
#pragma omp for schedule(static)
        for (long w = 0; w < (long)na * F; ++w) {
            const int e = active[w / F], f = (int)(w % F);
            const uint8_t *gr = (const uint8_t *)L->w_gate + (size_t)e * L->stride_gate + (size_t)f * rb_g;
            const uint8_t *ur = (const uint8_t *)L->w_up + (size_t)e * L->stride_up + (size_t)f * rb_u;
            for (int s = offs[e]; s < offs[e + 1]; ++s) {
                const int p = slot[s], t = p / K;
                const float g = zo_vec_dot_q8_K_fast(L->type_gate, D, gr, xq + (size_t)t * nbD);
                const float u = zo_vec_dot_q8_K_fast(L->type_up, D, ur, xq + (size_t)t * nbD);
                zo_swiglu(&act[(size_t)p * F + f], &g, &u, 1, L->clamp, L->clamp_fused);
            }
        }
#pragma omp for schedule(static)
        for (int p = 0; p < P; ++p)
            if (ids[p] >= 0 && ids[p] < E) zo_quantize_row_q8_K(act + (size_t)p * F, aq + (size_t)p * nbF, F);
#pragma omp for schedule(static)
        for (long w = 0; w < (long)na * D; ++w) {
            const int e = active[w / D], dd = (int)(w % D);
            const uint8_t *dr = (const uint8_t *)L->w_down + (size_t)e * L->stride_down + (size_t)dd * rb_d;
            for (int s = offs[e]; s < offs[e + 1]; ++s) {
                const int p = slot[s];
                down[(size_t)p * D + dd] = zo_vec_dot_q8_K_fast(L->type_down, F, dr, aq + (size_t)p * nbF);
            }
        }
#pragma omp for schedule(static)
        for (int t = 0; t < T; ++t)
            zo_combine(out + (size_t)t * D, down + (size_t)t * K * D, weights + (size_t)t * K, 1, K, D);
    }
    free(xq); free(aq); free(act); free(down); free(offs); free(slot); free(active);
    return n_threads;
}
