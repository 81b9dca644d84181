// ref_shim.cpp -- exposes a few functions of the reference's own CPU code so the
// oracle can be checked against them.  TEST INFRASTRUCTURE ONLY.
//
// Nothing from the reference is copied: its source files are #included or
// compiled from where they lie in the reference checkout (see the Makefile's
// `ref` target, which passes -I<reference root>).  Output: oracle/_ref/libzmoe_ref.so.
//
// What is reachable this way:
//   bench/q2k_dot_bench.cpp      dot_stock   (ggml's Q2_K x Q8_K AVX2 dot, "unchanged")
//                                dot_512     (its bit-exact AVX-512 VNNI variant)
//   bench/q3k_q4k_dot_bench.cpp  dot_q4k_512 (Q4_K x Q8_K, same grouping/order as stock)
//   bench/kernels/iq2xxs_dot_bench.cpp dot_ref ("the shipped AVX2 kernel"; its #include of
//                                ggml-common.h resolves to the stand-in oracle/ref_include/ggml-common.h)
//   backends/cpu/kernels_cpu.cpp dot_iq2_xxs_avx2_prototype, dequantize_row_{q2_K,q3_K,iq2_xxs}_avx512,
//                                silu_inplace, softmax_row
//   core/moe_router.cpp          apply_gating_activation
//   core/expert_activation.hpp   swiglu_clamp_fused_inplace, swiglu_clamp_inplace
// The ggml entry points those files declare extern are absent (ggml is an
// un-vendored submodule); they are stubbed to abort and are never reached by
// the wrappers below.
#include <immintrin.h>
#include <omp.h>
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

namespace ref_q2k {
#include "bench/q2k_dot_bench.cpp"
}
namespace ref_q4k {
#include "bench/q3k_q4k_dot_bench.cpp"
}
namespace ref_iq2 {
#include "bench/kernels/iq2xxs_dot_bench.cpp"
}
#include "backends/cpu/kernels_cpu.hpp"
#include "core/expert_activation.hpp"
#include "core/moe_router.hpp"

static const uint64_t shim_iq2xxs_grid[256] = {
#include "iq2xxs_grid.inc"
};

static void absent(const char *what) {
  std::fprintf(stderr, "ref_shim: %s needs ggml, which is not vendored\n", what);
  std::abort();
}

extern "C" {
// grid tables the reference takes from ggml (backends/cpu/ggml_grids.cpp)
const void *ms_grid_iq2xxs() { return shim_iq2xxs_grid; }
const void *ms_grid_iq1s() { absent("ms_grid_iq1s"); return nullptr; }
const void *ms_grid_iq2s() { absent("ms_grid_iq2s"); return nullptr; }
const void *ms_grid_iq2xs() { absent("ms_grid_iq2xs"); return nullptr; }
const void *ms_grid_iq3xxs() { absent("ms_grid_iq3xxs"); return nullptr; }
const void *ms_grid_iq3s() { absent("ms_grid_iq3s"); return nullptr; }
const void *ms_grid_kmask_iq2xs() {
  static const uint8_t k[8] = {1, 2, 4, 8, 16, 32, 64, 128};
  return k;
}
const void *ms_grid_ksigns_iq2xs() {
  static uint8_t t[128];
  static bool ready = false;
  if (!ready) {
    for (unsigned i = 0; i < 128; ++i) t[i] = (uint8_t)(i | ((__builtin_popcount(i) & 1) << 7));
    ready = true;
  }
  return t;
}
void quantize_row_q8_K(const float *, void *, int64_t) { absent("quantize_row_q8_K"); }
void quantize_row_q8_0(const float *, void *, int64_t) { absent("quantize_row_q8_0"); }
void ggml_cpu_init(void) {}
#define STUB_DOT(name) \
  void name(int, float *, size_t, const void *, size_t, const void *, size_t, int) { absent(#name); }
STUB_DOT(ggml_vec_dot_iq1_m_q8_K)
STUB_DOT(ggml_vec_dot_iq2_xxs_q8_K)
STUB_DOT(ggml_vec_dot_iq2_xs_q8_K)
STUB_DOT(ggml_vec_dot_iq3_xxs_q8_K)
STUB_DOT(ggml_vec_dot_iq4_nl_q8_0)
STUB_DOT(ggml_vec_dot_q2_0_q8_0)
STUB_DOT(ggml_vec_dot_q3_K_q8_K)
STUB_DOT(ggml_vec_dot_q4_K_q8_K)

// ---- wrappers -------------------------------------------------------------
float ref_q2k_dot_stock(int n, const void *x, const void *y) {
  return ref_q2k::dot_stock(n, (const ref_q2k::block_q2_K *)x, (const ref_q2k::block_q8_K *)y);
}
float ref_q2k_dot_512(int n, const void *x, const void *y) {
  return ref_q2k::dot_512(n, (const ref_q2k::block_q2_K *)x, (const ref_q2k::block_q8_K *)y);
}
float ref_q4k_dot_512(int n, const void *x, const void *y) {
  return ref_q4k::dot_q4k_512(n, (const ref_q4k::block_q4_K *)x, (const ref_q4k::block_q8_K *)y);
}
float ref_iq2xxs_dot_bench(int n, const void *x, const void *y) {
  return ref_iq2::dot_ref(n, (const ref_iq2::block_iq2_xxs *)x, (const ref_iq2::block_q8_K *)y);
}
float ref_iq2xxs_dot(int n, const void *x, const void *y) {
  return dot_iq2_xxs_avx2_prototype((const uint8_t *)x, (const block_q8_K_local *)y, n);
}
void ref_dequant_q2k(const void *w, float *y, int64_t k) { dequantize_row_q2_K_avx512((const uint8_t *)w, y, k); }
void ref_dequant_q3k(const void *w, float *y, int64_t k) { dequantize_row_q3_K_avx512((const uint8_t *)w, y, k); }
void ref_dequant_iq2xxs(const void *w, float *y, int64_t k) { dequantize_row_iq2_xxs_avx512((const uint8_t *)w, y, k); }
void ref_silu_inplace(float *x, int n) { silu_inplace(x, n); }
void ref_softmax_row(float *x, int n) { softmax_row(x, n); }
void ref_apply_gating(int func, float *row, int n) { apply_gating_activation((GatingFunc)func, row, n); }
void ref_swiglu_fused(float *gate, const float *up, int n, float limit) { swiglu_clamp_fused_inplace(gate, up, n, limit); }
void ref_clamp(float *x, int n, float limit) { swiglu_clamp_inplace(x, n, limit); }
}
