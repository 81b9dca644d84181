/*
 * zmoe_oracle.h -- CPU restatement of the reference MoE expert path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links or calls
 * this file; it exists so the CUDA path can be checked against an
 * independent scalar statement of the same arithmetic, and so the CPU
 * baseline of the benchmark has something to time.
 *
 * The arithmetic restated here is the ggml-cpu MUL_MAT_ID path that the
 * reference runs for CPU experts (ggml-org/llama.cpp pinned at commit
 * 8baabd53b77d1c48c6ef8d3b620436292f3f6231, reference CMakeLists.txt:335):
 *   activation row -> Q8_K blocks -> per-super-block integer dot against the
 *   quantised weight row -> f32 assembly.
 * That source tree is not vendored in the reference checkout, so each function
 * below names the first-party reference file it follows instead.
 *
 * Pinned (bit-exact against reference code compiled from the reference tree,
 * see oracle/ref_shim.cpp and tests/test_oracle_pins.py):
 *   Q2_K x Q8_K dot, Q4_K x Q8_K dot, IQ2_XXS x Q8_K dot, the four weight
 *   dequantisers, SiLU, softmax.
 * PARITY UNPINNED (no executable or golden reference exists in the checkout):
 *   zo_quantize_row_q8_K (restates the published ggml rule) and the f32 lane
 *   order of the Q3_K dot.  The per-block int32 sums of Q3_K are still pinned
 *   through the dequantiser: sum(dequant * q8) must equal d * isum exactly in
 *   integer arithmetic.
 */
#ifndef ZMOE_ORACLE_H
#define ZMOE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF / ggml type ids (reference models/base/gguf_loader.hpp:28-51). */
enum { ZO_TYPE_Q2_K = 10, ZO_TYPE_Q3_K = 11, ZO_TYPE_Q4_K = 12, ZO_TYPE_IQ2_XXS = 16 };

#define ZO_QK_K 256
#define ZO_Q8K_BYTES 292

/* bytes per 256-element super-block; 0 for an unsupported type
 * (reference backends/cpu/kquant_dequant.hpp:463-545). */
size_t zo_block_bytes(int type);

float zo_fp16_to_fp32(uint16_t h);

/* Q8_K activation quantiser: k must be a multiple of 256; y receives k/256
 * blocks of {float d; int8 qs[256]; int16 bsums[16]} (layout: reference
 * backends/cpu/kernels_cpu.cpp:22-33). */
void zo_quantize_row_q8_K(const float *x, void *y, int64_t k);

/* Weight-row dequantisers (layouts: reference kernels/quant/kquant_matmul.cu:35-200,
 * kernels/quant/iq2_matmul.cu:27-91). */
void zo_dequantize_row(int type, const void *w, float *y, int64_t k);

/* Per-super-block integer sums.  isum = sum over sub-blocks of
 * scale * (q . q8); msum = sum over sub-blocks of min * bsum (0 for types
 * without a min term).  These are what "per-block int32 dots" means in the
 * parity tests. */
void zo_block_isums(int type, const void *wblock, const void *q8block,
                    int32_t *isum, int32_t *msum);

/* Whole-row dot against Q8_K blocks, f32 assembly in the 8-lane order of the
 * reference's AVX2 restatements (bench/q2k_dot_bench.cpp:33-66,
 * bench/q3k_q4k_dot_bench.cpp:73-125, backends/cpu/kernels_cpu.cpp:2000-2075). */
float zo_vec_dot_q8_K(int type, int n, const void *w, const void *q8);

/* y[S,O] = x[S,I] . W[O,I]^T with x quantised to Q8_K per row.  Follows the
 * contract of launch_*_matmul (reference kernels/quant/kquant_matmul.cu:576-611)
 * with the ggml-cpu arithmetic. */
void zo_matmul(int type, float *y, const float *x, const void *w, int S, int I, int O);

/* Dense Q8_0 (zmoe_oracle_dense.c): 34-byte blocks {fp16 d; int8 qs[32]}; activations quantised to
 * Q8_0 as ggml's CPU MUL_MAT does (rule restated there; parity unpinned). */
uint16_t zo_fp32_to_fp16(float f);
void zo_quantize_row_q8_0(const float *x, void *y, int64_t k);
void zo_dequantize_row_q8_0(const void *w, float *y, int64_t k);
float zo_vec_dot_q8_0_q8_0(int n, const void *w, const void *x);
void zo_matmul_q8_0(float *y, const float *x, const void *w, int S, int I, int O);

/* MUL_MAT_ID (reference models/graph/moe_routed_ggml.hpp:181-193,
 * kernels/quant/kquant_matmul.cu:647-662 for the id rules):
 *   y[t,k,:] = W[ids[t,k]] . x[t, x_per_route ? k : 0, :]
 * ids<0 -> zero row, ids>=E -> NaN row.  x rows are quantised to Q8_K.
 * expert_stride in bytes; rows inside an expert are packed. */
void zo_mul_mat_id(int type, float *y, const float *x, const void *w,
                   size_t expert_stride, const int32_t *ids, int T, int K,
                   int E, int I, int O, int x_per_route);

/* SwiGLU (reference kernels/math/expert_activation.cu:31-59,
 * core/expert_activation.hpp:6-24). */
void zo_swiglu(float *prod, const float *gate, const float *up, int n,
               float clamp, int fused);

/* Router (reference core/moe_router.cpp:6-37, core/moe_router_service.cpp:1409-1474,
 * kernels/models/glm5next_router.cu:33-93).  gating: 0 softmax, 1 sigmoid,
 * 2 sqrt(softplus).  logits [T,E] are overwritten with probabilities.
 * Ties break to the lowest expert index. */
typedef struct {
    int n_experts, topk;
    int gating;          /* 0 softmax, 1 sigmoid, 2 sqrt-softplus */
    int normalize;       /* expert_weights_norm */
    float weight_scale;  /* applied when not 0 */
    int n_groups;        /* <=1: no group limit */
    int n_groups_used;
} zo_router_spec;

void zo_router_logits(float *logits, const float *x, const float *wr, int T, int D, int E);
void zo_router_select(const zo_router_spec *spec, float *probs_inout, const float *bias,
                      int32_t *ids, float *weights, int T);
/* smallest gap between the K-th and (K+1)-th selection score over all tokens;
 * tests re-draw inputs when this is tiny so that id comparisons are meaningful */
float zo_router_min_margin(const zo_router_spec *spec, const float *probs, const float *bias, int T);

/* CSR grouping (reference core/batched_dispatch_pipeline.cpp:1185-1204):
 * offs[E+1], slot[P] with slot entries = t*K+k in token-major order. */
void zo_group_by_expert(const int32_t *ids, int T, int K, int E, int32_t *offs, int32_t *slot);

/* Weighted combine in k order (reference models/graph/moe_routed_ggml.hpp:198-215):
 * out[t,:] = ((w0*y0 + w1*y1) + w2*y2) + ... */
void zo_combine(float *out, const float *y, const float *weights, int T, int K, int D);

/* One routed MoE layer, ids/weights given.  Scratch is allocated internally.
 * Returns 0 on success. */
typedef struct {
    int D, F, E, K;
    int type_gate, type_up, type_down;
    const void *w_gate, *w_up, *w_down;
    size_t stride_gate, stride_up, stride_down; /* bytes between experts */
    float clamp;
    int clamp_fused;
} zo_layer;

int zo_moe_ffn(const zo_layer *L, const float *x, const int32_t *ids, const float *weights,
               int T, float *out, float *dbg_act /* optional [T,K,F] */);

/* Same arithmetic as zo_moe_ffn with AVX2 dots and OpenMP over rows, rows
 * grouped by expert: the timed CPU baseline.  Falls back to the scalar dots
 * when the host lacks AVX2.  n_threads<=0 -> all cores.  Returns threads used. */
int zo_moe_ffn_fast(const zo_layer *L, const float *x, const int32_t *ids, const float *weights,
                    int T, float *out, int n_threads);
int zo_have_avx2(void);
/* which dots zo_vec_dot_q8_K_fast / zo_moe_ffn_fast run: 0 scalar, 1 AVX2, 2 AVX-512 VNNI (bit-identical results) */
int zo_fast_kind(void);
/* tests: cap the kind (-1: the best the CPU has) */
void zo_fast_force(int kind);

#ifdef __cplusplus
}
#endif
#endif
