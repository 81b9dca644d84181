/*
 * zmoe_b200.h -- C ABI of libzmoe_b200.so: the MoE expert hot path of
 * ray-x/ZeroMoE (router top-k, token-to-expert grouping, quantised expert FFN,
 * weighted combine) for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  All pointers named *_dev are device pointers
 * on the current CUDA device; `stream` is a cudaStream_t passed as void*.
 * Functions that return int return 0 on success and a negative ZMOE_ERR_* code
 * otherwise; there is no CPU fallback anywhere in the library.
 *
 * Numerics.  Activations are quantised to Q8_K per 256 values, as the reference's
 * CPU path (ggml MUL_MAT_ID) does.  Two families of kernels multiply them:
 *   - the decode kernels (every launch_*_matmul symbol, the op hook, and the layer
 *     entry below zmoe_gemm_min_pairs_per_expert() pairs per expert) work in integer
 *     arithmetic: the per-super-block int32 sums are exact, the f32 assembly differs
 *     from the CPU path only in summation order;
 *   - the tensor-core grouped GEMM (the layer entry from that threshold up, or
 *     zmoe_ctx_set_path(ctx, 2)) multiplies fp16 operands with f32 accumulation:
 *     the activation operand is the exact Q8_K value d*q divided by a power of two,
 *     the weight operand is the dequantised weight rounded to fp16 once.  There is no
 *     int32 block sum on that path; results agree with the CPU path to about 3e-4 of
 *     the output norm (1e-3 is the bound the tests hold it to), and a token's output
 *     therefore depends, within that bound, on whether its batch took this path.
 */
#ifndef ZMOE_B200_H
#define ZMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#else
#include <stdbool.h>
#endif

/* ---- status codes ------------------------------------------------------ */
#define ZMOE_OK 0
#define ZMOE_ERR_ARG (-1)         /* null pointer, non-positive size, inconsistent shapes */
#define ZMOE_ERR_TYPE (-2)        /* quantisation type without a kernel */
#define ZMOE_ERR_SHAPE (-3)       /* row length not a multiple of 256 or out of range */
#define ZMOE_ERR_ALIGN (-4)       /* weight pointer / stride not 16-byte aligned */
#define ZMOE_ERR_CUDA (-5)        /* a CUDA runtime call failed */
#define ZMOE_ERR_CAPACITY (-6)    /* more tokens than the context was created for */
#define ZMOE_ERR_DEVICE_WAIT (-7) /* a bounded device-side wait expired */
#define ZMOE_ERR_STATE (-8)       /* wrong call order */
#define ZMOE_ERR_COMM (-9)        /* NCCL is missing or one of its calls failed */

/* GGUF quantisation type ids (reference models/base/gguf_loader.hpp:28-51) */
#define ZMOE_TYPE_Q2_K 10
#define ZMOE_TYPE_Q3_K 11
#define ZMOE_TYPE_Q4_K 12
#define ZMOE_TYPE_IQ2_XXS 16

/* router gating (reference models/base/gguf_loader.hpp:177-181) */
#define ZMOE_GATING_SOFTMAX 0
#define ZMOE_GATING_SIGMOID 1
#define ZMOE_GATING_SQRT_SOFTPLUS 2

/* =========================================================================
 * 1. Kernel-launch ABI -- the symbols the reference's CudaKernelDispatcher and
 *    cuda_manager link against.  y[S,O] = x[S,I] . W[O,I]^T, W packed rows of
 *    quantised super-blocks, device pointers, asynchronous, void return
 *    (errors surface through cudaGetLastError / zmoe_last_status()).
 *    They use the library's per-device scratch for the quantised activations;
 *    call zmoe_reserve() first when launching under stream capture.
 * ========================================================================= */

/* replaces reference kernels/quant/kquant_matmul.cu:576-590 */
void launch_q2_K_matmul(float *y, const float *x, const void *w, int S, int I, int O);
void launch_q2_K_matmul_stream(float *y, const float *x, const void *w, int S, int I, int O, void *stream);
/* replaces reference kernels/quant/kquant_matmul.cu:591-601 */
void launch_q3_K_matmul(float *y, const float *x, const void *w, int S, int I, int O);
void launch_q3_K_matmul_stream(float *y, const float *x, const void *w, int S, int I, int O, void *stream);
/* replaces reference kernels/quant/kquant_matmul.cu:602-607 */
void launch_q4_K_matmul(float *y, const float *x, const void *w, int S, int I, int O);
/* replaces reference kernels/quant/iq2_matmul.cu:180-183 */
void launch_iq2_xxs_matmul(float *y, const float *x, const void *w, int S, int I, int O);
/* replaces reference kernels/quant/q8_0_matmul.cu:189-221: W packed rows of 34-byte Q8_0 blocks
 * {fp16 d; int8 q[32]}, I a multiple of 32.  The activation rows are quantised to Q8_0 as well
 * and blocks are multiplied in integers, as the reference's CPU path (ggml MUL_MAT) does. */
void launch_q8_0_matmul(float *y, const float *x, const void *weights, int S, int I, int O);
void launch_q8_0_matmul_stream(float *y, const float *x, const void *weights, int S, int I, int O, void *stream);
/* replaces reference kernels/math/rmsnorm.cu:80-83: y[S, D] = x * rsqrt(mean(x^2) + eps) * w, D a multiple of 4 */
void launch_rmsnorm(float *y, const float *x, const float *w, int S, int D, float eps);

/* replaces reference kernels/math/expert_activation.cu:61-70 */
void launch_expert_swiglu(float *prod, const float *gate, const float *up, int n, float clamp, int fused,
                          int *d_bad, void *stream);
/* replaces reference kernels/math/expert_accum.cu:39-46 */
void launch_expert_scatter_accum(const float *src, const int *tok, const float *w, float *dst, int n, int D,
                                 int S, void *stream);
/* replaces reference kernels/math/expert_accum.cu:52-60 */
void launch_expert_scatter_add(const float *src, const int *tok, float *dst, int n, int D, int S, void *stream);
/* replaces reference kernels/models/glm5next_router.cu:95-105 */
void launch_glm5next_router_topk(float *logits, const float *bias, int32_t *ids, float *weights, int S,
                                 int n_experts, int topk, int gating_func, int normalize, float weight_scale,
                                 void *stream);

/* No counterpart in the reference.  y[S,O] = x[S,I] . W[O,I]^T like the launch_*_matmul
 * symbols above (type = ZMOE_TYPE_*, same results bit for bit), for callers that must not
 * allocate device memory when they call: engines that gave the whole GPU to their own pool,
 * code running inside someone else's stream capture, real-time loops.  The quantised
 * activations and the work plan live in a fixed array inside the library image instead of
 * cudaMalloc'ed buffers; the call makes no cudaMalloc / cudaFree.
 *   - Every GPU that loads the library holds ZMOE_NOALLOC_SCRATCH_BYTES for this until exit.
 *   - Problems needing more (about S * 1.4 * I bytes) return ZMOE_ERR_CAPACITY.
 *   - The first call on each device looks the array's address up (cudaGetSymbolAddress with
 *     that device current); make that first call before any stream capture begins.
 *   - All calls share the array: calls whose kernels may overlap on the GPU race.  Order
 *     them on one stream or with events.
 * Returns a ZMOE_* status; work is enqueued on `stream`. */
#define ZMOE_NOALLOC_SCRATCH_BYTES (1u << 20)
int zmoe_matmul_noalloc(int type, float *y, const float *x, const void *w, int S, int I, int O, void *stream);

/* grow the per-device scratch of the entry points above to hold `rows`
 * activation rows of `I` elements (allocates; not capturable) */
int zmoe_reserve(int rows, int I);
/* status of the most recent kernel-launch-ABI call on this thread */
int zmoe_last_status(void);
/* The entry points of this section, the op hook of section 2 and zmoe_matmul_noalloc have no handle to
 * report a device-side problem through: their kernels raise an error word in the library's per-device
 * scratch when a bounded wait runs out (the output of that launch is then incomplete).  This call waits
 * for the current device, reads those words and clears them: 0, or ZMOE_ERR_DEVICE_WAIT.
 * Contract of the per-device scratch: host threads may call these entry points concurrently (the scratch
 * is locked from sizing to enqueue, and is only reallocated after the device has drained), but all calls
 * on one device share one set of buffers -- calls whose kernels may overlap on the GPU (different streams
 * with no ordering between them) race on it, exactly as documented for zmoe_matmul_noalloc. */
int zmoe_device_status(void);
/* Self-test of that reporting path, for test suites: enqueues one warp that waits, with a limit of a few
 * hundred polls, on a barrier nothing arrives on; the wait runs out, the warp raises the error word like a
 * matmul kernel would and returns (no hang, no fault).  zmoe_device_status() must then report
 * ZMOE_ERR_DEVICE_WAIT once. */
int zmoe_selftest_wait_expiry(void *stream);

/* =========================================================================
 * 2. ggml backend op hook -- replaces the hook the reference registers with
 *    ggml-cuda for GGML_OP_MUL_MAT / GGML_OP_MUL_MAT_ID nodes
 *    (reference kernels/quant/kquant_matmul.cu:702-765,
 *    patches/ggml/0010-native-f32-quant-graph-hook.patch).  ggml is not part of
 *    this library, so the tensors arrive as a plain mirror of the ggml_tensor
 *    fields the hook reads; a trampoline from real ggml_tensor is a few lines.
 * ========================================================================= */
typedef struct zmoe_tensor {
    int type;       /* ggml type id: 0 = F32, 26 = I32, or a ZMOE_TYPE_* */
    int64_t ne[4];  /* elements per dimension */
    size_t nb[4];   /* strides in bytes */
    void *data;     /* device pointer */
} zmoe_tensor;

/* Same contract as the reference hook: returns false when the node is not
 * handled; execute=false is a side-effect-free support query; with
 * execute=true the work is enqueued on `stream`.
 *   w->ne = [I, O, E, 1], rows packed (w->nb[1] == row bytes), w->nb[2] free;
 *   x->ne = [I, 1|K, T]; ids->ne = [K, T] (I32) or ids == NULL for MUL_MAT;
 *   y->ne = [O, K, T].  ids < 0 -> zero row, ids >= E -> NaN row. */
bool zmoe_f32_quant_hook(const zmoe_tensor *w, const zmoe_tensor *x, const zmoe_tensor *ids, zmoe_tensor *y,
                         void *stream, bool execute);
/* replaces reference kernels/quant/kquant_matmul.cu:757-765; returns false
 * because no ggml-cuda is linked into this library to register with */
bool zeromoe_install_f32_quant_graph_hook(void);
uint64_t zeromoe_f32_quant_graph_launches(void);

/* =========================================================================
 * 3. Layer-level entry -- replaces, for HBM-resident weights,
 *    MoeRouterService::route (reference core/moe_router_service.cpp:430),
 *    BatchedDispatchPipeline::run (reference core/batched_dispatch_pipeline.hpp:5-14)
 *    and expert_ffn_gpu_issue / finish_stage1 / finish_stage2
 *    (reference core/gpu_expert_executor.hpp:42-58).
 * ========================================================================= */
typedef struct zmoe_ctx zmoe_ctx;     /* per-device scratch, one per decode thread */
typedef struct zmoe_layer zmoe_layer; /* borrowed weights of one MoE layer */

typedef struct zmoe_weight {
    const void *data_dev;  /* expert 0, row 0 */
    size_t expert_stride;  /* bytes between experts (>= rows * row bytes) */
    size_t bytes;          /* bytes addressable from data_dev; 0 = n_experts * expert_stride */
    int type;              /* ZMOE_TYPE_* */
} zmoe_weight;

typedef struct zmoe_layer_desc {
    int d_model, d_ff, n_experts, topk;
    zmoe_weight gate, up, down;  /* gate/up: [E][d_ff rows of d_model]; down: [E][d_model rows of d_ff] */
    const float *router_w_dev;   /* [n_experts, d_model] f32, may be NULL when routes are always supplied */
    const float *router_bias_dev;/* [n_experts] selection bias or NULL */
    int gating;                  /* ZMOE_GATING_* */
    int weights_norm;            /* expert_weights_norm */
    float weights_scale;         /* expert_weights_scale; 0 or 1 = none */
    int n_groups, n_groups_used; /* group-limited routing; n_groups <= 1 disables */
    float swiglu_clamp;          /* <= 0: none */
    int swiglu_clamp_fused;      /* clamp gate/up before the activation instead of the product */
} zmoe_layer_desc;

int zmoe_ctx_create(int max_tokens, int max_d_model, int max_d_ff, int max_experts, int max_topk, zmoe_ctx **out);
void zmoe_ctx_destroy(zmoe_ctx *ctx);
int zmoe_layer_create(zmoe_ctx *ctx, const zmoe_layer_desc *desc, zmoe_layer **out);
void zmoe_layer_destroy(zmoe_layer *layer);

/* router + grouping: fills the context's route table (ids, weights, expert
 * histogram, CSR) for T tokens of x_dev [T, d_model]. */
int zmoe_route(zmoe_layer *layer, const float *x_dev, int T, void *stream);
/* supply routes computed elsewhere (ids [T, topk] i32, weights [T, topk] f32, device);
 * negative ids are inactive routes */
int zmoe_set_routes(zmoe_layer *layer, const float *x_dev, const int32_t *ids_dev, const float *weights_dev, int T,
                    void *stream);
/* the same with the rows of ids and weights a given number of bytes apart (multiples of 4, >= topk * 4): ggml's
 * top-k ids are a view [topk, T] of the argsort result whose rows are n_experts * 4 bytes apart */
int zmoe_set_routes_strided(zmoe_layer *layer, const float *x_dev, const int32_t *ids_dev, size_t ids_token_stride,
                            const float *weights_dev, size_t weights_token_stride, int T, void *stream);
/* the same for a layer that holds the experts [first_expert, first_expert + n_experts) of a larger
 * model (one rank of an expert-parallel group): ids are the model's expert numbers, the ones outside
 * the layer's window become inactive routes.  Same convention as the reference's hot / cold branch
 * route_map (backends/ggml/moe_partial_route_ggml.hpp:13-35): an expert owned elsewhere maps to -1. */
int zmoe_set_routes_window(zmoe_layer *layer, const float *x_dev, const int32_t *ids_dev, const float *weights_dev,
                           int T, int first_expert, void *stream);
/* expert FFN + combine over the current routes: out_dev [T, d_model] is
 * overwritten (accumulate = 0) or added to (accumulate = 1) */
int zmoe_expert_ffn(zmoe_layer *layer, float *out_dev, int T, int accumulate, void *stream);
/* zmoe_expert_ffn that also records two caller-owned cudaEvent_t (passed as void*) on
 * `stream`, one before and one after the gate/up matmul, for per-kernel timing */
int zmoe_expert_ffn_events(zmoe_layer *layer, float *out_dev, int T, int accumulate, void *stream,
                           void *ev_before_gate_up, void *ev_after_gate_up);
/* Dense SwiGLU FFN applied to every token -- the shared expert of reference
 * backends/ggml/ggml_moe_graph_builder.cpp:94-129 (build_shared_topology).  `layer` must have been
 * created with n_experts = 1 and topk = 1 over the shared expert's gate / up / down tensors; with
 * accumulate = 1 the result is added to out_dev (the routed sum).  Overwrites the context's route
 * table. */
int zmoe_dense_ffn(zmoe_layer *layer, const float *x_dev, float *out_dev, int T, int accumulate, void *stream);
/* the same with the shared expert's scalar gate (reference models/graph/ggml_moe_graph_builder.cpp:120-124):
 * every token's row is multiplied by sigmoid(gate_w . x[t]) before it is written or added; gate_w_dev [d_model] f32 */
int zmoe_dense_ffn_gated(zmoe_layer *layer, const float *x_dev, const float *gate_w_dev, float *out_dev, int T,
                         int accumulate, void *stream);
/* zmoe_route followed by zmoe_expert_ffn */
int zmoe_moe_forward(zmoe_layer *layer, const float *x_dev, float *out_dev, int T, void *stream);
/* the same for bf16 activations (x_bf16_dev [T, d_model], 16-byte aligned): the third benchmark configuration's
 * input type.  The rows are widened (exactly) into the context's staging buffer, which zmoe_moe_forward_host also
 * uses: one of the two at a time per context. */
int zmoe_moe_forward_bf16(zmoe_layer *layer, const void *x_bf16_dev, float *out_dev, int T, void *stream);
/* the same with host buffers: copies x in, runs the layer, copies out back, synchronises */
int zmoe_moe_forward_host(zmoe_layer *layer, const float *x_host, float *out_host, int T);

/* copies of the current route table / intermediates to host (synchronise the stream first) */
int zmoe_get_routes(zmoe_ctx *ctx, int T, int topk, int32_t *ids_host, float *weights_host);
int zmoe_get_expert_freq(zmoe_ctx *ctx, int n_experts, int32_t *freq_host);
/* device-to-device copy of the current route table, enqueued on `stream` (for exchanging
 * routes between expert-parallel ranks without a host round trip) */
int zmoe_copy_routes(zmoe_ctx *ctx, int T, int topk, int32_t *ids_dev, float *weights_dev, void *stream);
int zmoe_get_probs(zmoe_ctx *ctx, int T, int n_experts, float *probs_host);
int zmoe_get_act(zmoe_ctx *ctx, int n_pairs, int d_ff, float *act_host);
/* which expert-FFN kernels run: 0 = choose by shape (tensor-core grouped GEMM once the call
 * averages 24 or more pairs per expert, decode kernels below that), 1 = decode kernels,
 * 2 = tensor-core GEMM whenever the shapes allow (rows per expert a multiple of 128, gate and
 * up of one type), 3 = decode kernels with one pair at a time (a pair's result then does not
 * depend on which other pairs share its expert; slower once experts hold several pairs).
 * The activations passed to zmoe_route / zmoe_set_routes must stay valid
 * until zmoe_expert_ffn has been enqueued. */
int zmoe_ctx_set_path(zmoe_ctx *ctx, int path);
/* reads and clears the device error flag: 0, or ZMOE_ERR_DEVICE_WAIT */
int zmoe_ctx_check(zmoe_ctx *ctx);
/* Non-finite inputs seen by the fused SwiGLU epilogues of this context's expert FFN calls since the last
 * clear: counts_host[0] = (gate, up) pairs with a NaN, counts_host[1] = pairs without NaN but with an
 * infinity -- the counters of reference kernels/math/expert_activation.cu:42-44, which
 * core/gpu_expert_executor.cpp:406-421 samples.  Synchronise the stream first; clear != 0 resets them. */
int zmoe_ctx_bad_counts(zmoe_ctx *ctx, int32_t *counts_host, int clear);
/* average pairs per expert from which zmoe_expert_ffn takes the tensor-core grouped GEMM when the path is 0 */
int zmoe_gemm_min_pairs_per_expert(void);
/* Profiling aid of the grouped GEMM.  A library built with -DZMOE_GEMM_STATS keeps per-role cycle sums of
 * CTA 0 (waits and work of the converter, MMA, loader and epilogue warps; slots listed in
 * csrc/gemm_sm100.cuh): this call waits for the device, copies the 2 x 16 counters (gate / up launches, then
 * down launches) to counters32_host and clears them.  A normal build returns ZMOE_ERR_STATE and zeros. */
int zmoe_debug_gemm_cycles(uint64_t *counters32_host);
/* number of kernels this library has launched since load (all entry points) */
uint64_t zmoe_kernel_launches(void);

/* =========================================================================
 * 4. Expert parallelism over the GPUs of one node -- no counterpart in the reference (it has no
 *    collectives; its multi-GPU support is placement plus cudaMemcpyPeer, core/gpu_topology.cpp:1644).
 *    Rank r of N holds the experts [r * E / N, (r + 1) * E / N) of a layer in a zmoe_layer of its own and
 *    brings its own tokens.  Per layer, token rows travel once to every rank that owns one of their
 *    experts (all-to-all by per-destination counts, grouped ncclSend / ncclRecv), each rank runs its experts
 *    over what it received with routes of experts held elsewhere inactive -- the ownership convention of
 *    the reference's hot / cold split (backends/ggml/moe_partial_route_ggml.hpp:13-58) -- and one
 *    pre-weighted, pre-reduced row per (token, rank) travels back and is added in ascending rank order.
 *    Remote rows always land in local memory through NCCL before a kernel reads them.  NCCL is loaded with
 *    dlopen at first use: without it these calls return ZMOE_ERR_COMM and the rest of the library works.
 * ========================================================================= */
typedef struct zmoe_ep zmoe_ep;

/* thin wrappers for hosts that do not create NCCL communicators themselves: id128 is a 128-byte
 * ncclUniqueId made on one rank and handed to all; comm_init runs ncclCommInitRank on the current device */
int zmoe_ep_unique_id(void *id128);
int zmoe_ep_comm_init(const void *id128, int rank, int world, void **comm_out);
int zmoe_ep_comm_destroy(void *comm);

/* nccl_comm: an ncclComm_t (as void*) with one rank per GPU, borrowed.  max_tokens: tokens a rank brings per
 * call; max_recv_tokens: rows it may receive (at most world * max_tokens; the local layer's context must be
 * created for that many tokens).  Allocates the exchange buffers. */
int zmoe_ep_create(void *nccl_comm, int rank, int world, int max_tokens, int max_recv_tokens, int d_model, int topk,
                   zmoe_ep **out);
void zmoe_ep_destroy(zmoe_ep *ep);
/* One expert-parallel MoE layer.  router: a layer over ALL experts of the model with the router tensors set
 * (only zmoe_route is run on it); local: the layer holding this rank's experts; shared: the shared expert
 * (zmoe_dense_ffn layer) added on the tokens' home rank, or NULL.  x_dev, out_dev: [T, d_model].
 * Synchronises `stream` once per call (the transfer sizes go through the host); every rank of the
 * communicator must make the call. */
int zmoe_ep_forward(zmoe_ep *ep, zmoe_layer *router, zmoe_layer *local, zmoe_layer *shared, const float *x_dev,
                    float *out_dev, int T, void *stream);
/* the same with routes supplied: ids are the model's expert numbers (n_experts_total of them) */
int zmoe_ep_forward_routed(zmoe_ep *ep, zmoe_layer *local, zmoe_layer *shared, int n_experts_total, const float *x_dev,
                           const int32_t *ids_dev, const float *weights_dev, float *out_dev, int T, void *stream);
/* token rows this rank sent and received in its last exchange */
int zmoe_ep_last_rows(zmoe_ep *ep, int64_t *sent_rows, int64_t *recv_rows);

/* =========================================================================
 * 5. Decoder step around the MoE block -- the fifth benchmark configuration end to end on the device: token
 *    embedding, per layer RMSNorm -> Q8_0 q/k/v projection -> RoPE (interleaved pairs, reference
 *    models/base/rope.hpp:52-118 without YaRN) -> grouped-query attention over an f16 KV cache (scores
 *    q.k / sqrt(head_dim), reference core/attention_layer.cpp:2633-2690) -> Q8_0 output projection added to the
 *    residual -> RMSNorm -> MoE block (sections 3) added to the residual; then RMSNorm, Q8_0 output head and
 *    greedy arg-max on the last token.  One sequence; the position and the sampled token stay on the
 *    device, so steps of one token can be enqueued back to back (or captured once and replayed) without a
 *    host round trip.  All tensors are borrowed device pointers.
 * ========================================================================= */
typedef struct zmoe_decoder zmoe_decoder;
typedef struct zmoe_decoder_desc {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim; /* head_dim 64 or 128 */
    int vocab, max_ctx, max_tokens;                       /* KV cache positions; tokens per step */
    float rms_eps, rope_theta;
    /* arrays of n_layers device pointers */
    const float *const *attn_norm_w; /* [d_model] */
    const void *const *wqkv;         /* Q8_0 [(n_heads + 2 n_kv_heads) * head_dim rows of d_model]: q, k, v rows in this order */
    const void *const *wo;           /* Q8_0 [d_model rows of n_heads * head_dim] */
    const float *const *ffn_norm_w;  /* [d_model] */
    zmoe_layer *const *moe;          /* the layers' MoE blocks, created on a context of at least max_tokens tokens */
    const void *tok_embd;            /* Q8_0 [vocab rows of d_model] */
    const float *out_norm_w;         /* [d_model] */
    const void *lm_head;             /* Q8_0 [vocab rows of d_model] */
} zmoe_decoder_desc;
int zmoe_decoder_create(const zmoe_decoder_desc *desc, zmoe_decoder **out);
void zmoe_decoder_destroy(zmoe_decoder *dec);
/* position back to 0 (the cache is overwritten as positions are reused) */
int zmoe_decoder_reset(zmoe_decoder *dec, void *stream);
/* T tokens at positions pos .. pos + T - 1 (T > 1: prompt processing, causal); tokens_dev == NULL with T == 1
 * takes the token the previous step sampled.  Leaves the arg-max of the last token's logits as the next
 * token and advances the position by T. */
int zmoe_decoder_step(zmoe_decoder *dec, const int32_t *tokens_dev, int T, void *stream);
/* synchronous reads of the sampled token, the position and the first n_logits logits of the last step (NULL
 * to skip); synchronise the stream first */
int zmoe_decoder_read(zmoe_decoder *dec, int32_t *next_token_host, int32_t *pos_host, float *logits_host, int n_logits);

/* =========================================================================
 * 6. Weight ingest -- the conversion between the expert-major [gate|up|down] slab the reference keeps in host
 *    memory and the three planar tensors of its ggml graphs (same signatures and meaning as the reference's
 *    launchers, with the status returned as int = cudaError_t and the stream as void*), and a reader of the
 *    GGUF container that finds a layer's expert tensors (blk.N.ffn_{gate,up,down}_exps.weight, the names and
 *    type ids of reference models/base/gguf_loader.hpp:28-51).  The layer entry of section 3 reads slabs in
 *    place through zmoe_weight.expert_stride, so the unpack is for hosts that keep planar tensors.
 * ========================================================================= */
/* replaces reference kernels/math/ggml_moe_pack.cu:122-149: record i of `src` (count records, src_stride bytes apart,
 * each gate bytes | up bytes | down bytes) goes to expert i of the planar tensors */
int launch_ggml_moe_unpack(const void *src, void *gate, void *up, void *down, int count, size_t src_stride,
                           size_t gate_bytes, size_t up_bytes, size_t down_bytes, size_t gate_stride, size_t up_stride,
                           size_t down_stride, void *stream);
/* replaces reference kernels/math/ggml_moe_pack.cu:151-179: record i goes to expert dst_slots[i] (negative: skipped) */
int launch_ggml_moe_unpack_scatter(const void *src, void *gate, void *up, void *down, const int32_t *dst_slots, int count,
                                   size_t src_stride, size_t gate_bytes, size_t up_bytes, size_t down_bytes,
                                   size_t gate_stride, size_t up_stride, size_t down_stride, void *stream);
/* the opposite direction (no counterpart in the reference, which packs on the host) */
int zmoe_moe_pack(void *slab, const void *gate, const void *up, const void *down, int count, size_t slab_stride,
                  size_t gate_bytes, size_t up_bytes, size_t down_bytes, size_t gate_stride, size_t up_stride,
                  size_t down_stride, void *stream);

typedef struct zmoe_gguf zmoe_gguf;
typedef struct zmoe_gguf_tensor {
    int type;              /* GGUF / ggml type id */
    int n_dims;
    int64_t ne[4];         /* elements per dimension, ne[0] the row length */
    uint64_t file_offset;  /* of the tensor's first byte in the file */
    uint64_t bytes;
} zmoe_gguf_tensor;
/* GGUF versions 2 and 3; host-side, no device needed */
int zmoe_gguf_open(const char *path, zmoe_gguf **out);
void zmoe_gguf_close(zmoe_gguf *g);
int zmoe_gguf_tensor_count(zmoe_gguf *g);
/* ZMOE_ERR_STATE when the file has no tensor of that name */
int zmoe_gguf_find(zmoe_gguf *g, const char *name, zmoe_gguf_tensor *out);
int zmoe_gguf_read(zmoe_gguf *g, const zmoe_gguf_tensor *t, void *dst_host, uint64_t first_byte, uint64_t n_bytes);
/* copies blk.<layer>.ffn_{gate,up,down}_exps.weight to the three device buffers (planar, experts back to back);
 * info3, when given, receives the three tensors' descriptions; synchronises `stream` */
int zmoe_gguf_load_experts(zmoe_gguf *g, int layer, void *gate_dev, void *up_dev, void *down_dev, zmoe_gguf_tensor *info3,
                           void *stream);

/* =========================================================================
 * 7. Parity hooks -- expose the integer stages so tests can compare them
 *    bit-for-bit with the CPU path.
 * ========================================================================= */
/* x_dev [rows, I] f32 -> blocks_dev: rows * I/256 ggml Q8_K blocks of 292 bytes
 * (layout: reference backends/cpu/kernels_cpu.cpp:22-26).  Internally the rows are
 * quantised into the packed layout used against weights of `for_type` and regrouped;
 * the blocks are the same for every type. */
int zmoe_quantize_q8_K(const float *x_dev, void *blocks_dev, int rows, int I, int for_type, void *stream);
/* per-super-block integer sums of weight row r against activation row r:
 * isum = sum scale*(q.q8), msum = sum min*bsum; outputs [rows, I/256] i32 */
int zmoe_block_isums(int type, const void *w_dev, const float *x_dev, int32_t *isum_dev, int32_t *msum_dev, int rows,
                     int I, void *stream);
/* the same sums as the tensor-core consumer path of the decode kernels forms them (mma.sync on a 16-row piece
 * against `pairs` <= 4 activation rows at once): w_dev = 16 weight rows, x_dev [pairs, I];
 * sums_dev [16 rows][4 pair slots][I/256][2] i32 holds {isum, msum} of row r against activation row p at
 * [r][p][block]; slots p >= pairs are scratch.  Q2_K, Q3_K (msum = 0), Q4_K; ZMOE_ERR_TYPE for a type without
 * that path. */
int zmoe_block_isums_pairs(int type, const void *w_dev, const float *x_dev, int32_t *sums_dev, int pairs, int I,
                           void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ZMOE_B200_H */
