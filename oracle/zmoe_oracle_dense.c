/*
 * zmoe_oracle_dense.c -- CPU restatement of the dense Q8_0 matmul the decoder step uses for its
 * attention projections and output head.
 *
 * TEST INFRASTRUCTURE ONLY (see zmoe_oracle.h).
 *
 * Q8_0 is ggml's 34-byte block {fp16 d; int8 qs[32]} (layout as read by reference
 * kernels/quant/q8_0_matmul.cu:20-60: w = d * q).  The reference's CUDA kernel multiplies the
 * dequantised weights by f32 activations; the reference's CPU path (ggml MUL_MAT) quantises the
 * activation row to Q8_0 as well and multiplies in integers, and this library follows the CPU path
 * everywhere.  ggml itself is an un-vendored submodule of the reference checkout
 * (ggml-org/llama.cpp @ 8baabd53b77d1c48c6ef8d3b620436292f3f6231), so the activation rule below
 * restates the published quantize_row_q8_0_ref / ggml_vec_dot_q8_0_q8_0:
 *   d = max|x| / 127 over 32 values, id = 1/d (0 for an all-zero block), q = roundf(x * id)
 *   (halves away from zero), d stored as fp16;  dot = sum over blocks of
 *   (sum q_w * q_x) * fp16->f32(d_w) * fp16->f32(d_x), added block after block in f32.
 * PARITY UNPINNED for that activation rule (no executable or golden reference exists in the
 * checkout); the weight dequantisation is pinned against gguf.quants in tests/test_oracle_pins.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "zmoe_oracle.h"

typedef struct {
    uint16_t d;
    int8_t qs[32];
} blk_q8_0;

/* f32 -> fp16 bits, round to nearest even (IEEE 754 binary16) */
uint16_t zo_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t em = x & 0x7fffffffu;
    if (em >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((em > 0x7f800000u) ? 0x200u : 0u)); /* inf / nan */
    if (em >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);                                       /* overflow */
    if (em < 0x33000001u) return (uint16_t)sign;                                                    /* underflow to zero */
    int exp = (int)(em >> 23) - 127;
    uint32_t man = (em & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < -14) { /* subnormal half */
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | (base + q));   /* a carry out of the mantissa bumps the exponent, as it should */
}

void zo_quantize_row_q8_0(const float *x, void *vy, int64_t k) {
    blk_q8_0 *y = (blk_q8_0 *)vy;
    for (int64_t b = 0; b < k / 32; ++b, x += 32) {
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const volatile float d_v = amax / 127.f;
        const float d = d_v;
        const float id = d != 0.f ? 1.0f / d : 0.0f;
        y[b].d = zo_fp32_to_fp16(d);
        for (int j = 0; j < 32; ++j) {
            const volatile float p = x[j] * id;
            y[b].qs[j] = (int8_t)roundf(p);
        }
    }
}

void zo_dequantize_row_q8_0(const void *vw, float *y, int64_t k) {
    const blk_q8_0 *w = (const blk_q8_0 *)vw;
    for (int64_t b = 0; b < k / 32; ++b) {
        const float d = zo_fp16_to_fp32(w[b].d);
        for (int j = 0; j < 32; ++j) y[32 * b + j] = d * (float)w[b].qs[j];
    }
}

float zo_vec_dot_q8_0_q8_0(int n, const void *vw, const void *vx) {
    const blk_q8_0 *w = (const blk_q8_0 *)vw, *x = (const blk_q8_0 *)vx;
    float sumf = 0.f;
    for (int b = 0; b < n / 32; ++b) {
        int sumi = 0;
        for (int j = 0; j < 32; ++j) sumi += (int)w[b].qs[j] * (int)x[b].qs[j];
        const volatile float dd = zo_fp16_to_fp32(w[b].d) * zo_fp16_to_fp32(x[b].d);
        const volatile float term = (float)sumi * dd;
        sumf += term;
    }
    return sumf;
}

/* y[S, O] = x[S, I] . W[O, I]^T, W packed rows of Q8_0 blocks */
void zo_matmul_q8_0(float *y, const float *x, const void *w, int S, int I, int O) {
    const size_t rb = (size_t)(I / 32) * sizeof(blk_q8_0);
    blk_q8_0 *xq = (blk_q8_0 *)malloc((size_t)S * rb);
    for (int s = 0; s < S; ++s) zo_quantize_row_q8_0(x + (size_t)s * I, (uint8_t *)xq + (size_t)s * rb, I);
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; ++o)
        for (int s = 0; s < S; ++s)
            y[(size_t)s * O + o] = zo_vec_dot_q8_0_q8_0(I, (const uint8_t *)w + (size_t)o * rb, (const uint8_t *)xq + (size_t)s * rb);
    free(xq);
}
