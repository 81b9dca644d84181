/* Minimal stand-in for ggml's ggml-common.h, which the reference's
 * bench/kernels/iq2xxs_dot_bench.cpp includes and which is absent from the
 * reference checkout (un-vendored submodule).  Only what that one file uses:
 * the two block layouts, QK_K, ggml_half and the IQ2_XXS codebook.
 * TEST INFRASTRUCTURE ONLY; used solely by oracle/ref_shim.cpp. */
#ifndef ZMOE_STANDIN_GGML_COMMON_H
#define ZMOE_STANDIN_GGML_COMMON_H
#include <stdint.h>
#define QK_K 256
typedef uint16_t ggml_half;
typedef struct { ggml_half d; uint16_t qs[QK_K / 8]; } block_iq2_xxs;
typedef struct { float d; int8_t qs[QK_K]; int16_t bsums[QK_K / 16]; } block_q8_K;
static const uint64_t iq2xxs_grid[256] = {
#include "iq2xxs_grid.inc"
};
#endif
