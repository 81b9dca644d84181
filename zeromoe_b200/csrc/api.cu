// api.cu -- the C ABI of libzmoe_b200.so (declared in include/zmoe_b200.h):
// reference kernel-launch symbols, the ggml-style op hook on plain tensor
// mirrors, and the layer-level entry with its per-device context.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <utility>

#include "zmoe_common.cuh"
#include "zmoe_internal.h"

using namespace zmoe;

namespace {

std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_hook_launches{0};
thread_local int tl_status = ZMOE_OK;

inline int ok(cudaError_t e) { return e == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA; }

template <typename T>
int dev_alloc(T **p, size_t n) {
    *p = nullptr;
    if (n == 0) n = 1;
    return ok(cudaMalloc(reinterpret_cast<void **>(p), n * sizeof(T)));
}

int sm_count() { return zmoe::device_sm_count(); }

// pairs per expert, averaged over the call, from which the layer entry takes the tensor-core grouped GEMM
constexpr int kGemmMinPairsPerExpert = 24;

struct PlanStore {
    PlanBuffers b;
    int cap_e = 0, cap_p = 0;
    int alloc(int E, int P) {
        int rc = 0;
        rc |= dev_alloc(&b.hdr, 4);
        rc |= dev_alloc(&b.active, E);
        rc |= dev_alloc(&b.offs, E + 1);
        rc |= dev_alloc(&b.slot, P);
        rc |= dev_alloc(&b.item_offs_gu, E + 1);
        rc |= dev_alloc(&b.item_offs_dn, E + 1);
        rc |= dev_alloc(&b.freq, E);
        rc |= dev_alloc(&b.aoffs, E);
        rc |= dev_alloc(&b.antok, E);
        rc |= dev_alloc(&b.pos, P);
        b.cap_e = E;
        cap_e = E;
        cap_p = P;
        return rc ? ZMOE_ERR_CUDA : ZMOE_OK;
    }
    void release() {
        cudaFree(b.hdr); cudaFree(b.active); cudaFree(b.offs); cudaFree(b.slot);
        cudaFree(b.item_offs_gu); cudaFree(b.item_offs_dn); cudaFree(b.freq); cudaFree(b.aoffs); cudaFree(b.antok); cudaFree(b.pos);
        b = PlanBuffers();
        cap_e = cap_p = 0;
    }
};

}  // namespace

namespace zmoe {

int device_sm_count() {
    constexpr int kMax = 64;
    static std::atomic<int> cache[kMax];
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMax && (n = cache[dev].load(std::memory_order_relaxed)) > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMax) cache[dev].store(n, std::memory_order_relaxed);
    return n;
}

void count_launches(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_last_status(int rc) { tl_status = rc; }

int raise_dynamic_smem(const void *fn, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> done;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ZMOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = done[std::make_pair(fn, dev)];
    if (have < bytes) {
        if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
            return ZMOE_ERR_CUDA;
        have = bytes;
    }
    return ZMOE_OK;
}

}  // namespace zmoe

// ---------------------------------------------------------------------------
// context and layer
// ---------------------------------------------------------------------------
struct zmoe_ctx {
    int max_t = 0, max_d = 0, max_f = 0, max_e = 0, max_k = 0;
    int n_sm = 0;
    int device = 0;
    uint8_t *q8x = nullptr;    // packed Q8_K rows of the layer input (unit layout of the gate format)
    uint8_t *q8x2 = nullptr;   // the same in the other unit layout, for an up format that needs it
    float *act = nullptr;      // [P, F] SwiGLU output
    float *act2 = nullptr;     // [2, P, F] gate / up when their types differ (lazy)
    uint8_t *q8act = nullptr;  // packed Q8_K rows of act
    void *xq_f16 = nullptr;   // [P, D] fp16: layer input rows in expert order after the Q8_K round trip
    void *actq_f16 = nullptr; // [P, F] fp16: act after the Q8_K round trip (tensor-core path)
    float *xscale = nullptr, *actscale = nullptr;  // per-row powers of two of the fp16 copies
    int32_t *zero_ids = nullptr;   // [T] zeros / ones: routes of a dense (single-expert) FFN
    float *one_w = nullptr;
    float *gate_s = nullptr;       // [T] per-token scalar gates of a gated shared expert
    const float *x_last = nullptr;  // the activations the current route table was built from
    int path = 0;              // 0 auto, 1 decode kernels, 2 tensor-core GEMM, 3 decode kernels, scalar path only
    float *ydown = nullptr;    // [P, D] per-pair down-projection output
    float *logits = nullptr;   // [T, E] router logits, then probabilities
    float *logits_part = nullptr;  // [ROUTER_MAX_SPLIT][T, E] partial logits of the large-batch router (contexts of > 256 tokens)
    bool q8x_valid = false;    // q8x (and q8x2) hold the quantised rows of x_last
    int32_t *ids = nullptr;    // [T, K]
    float *weights = nullptr;  // [T, K]
    PlanStore plan;
    int *err = nullptr;
    int *bad = nullptr;        // [2] NaN / Inf inputs seen by the fused SwiGLU epilogues
    int *queue = nullptr;      // [4] item tickets of the decode matmuls (two per projection; every launch leaves them zero)
    unsigned *ticket = nullptr;
    float *x_stage = nullptr, *out_stage = nullptr;  // device staging of the host entry
    cudaStream_t host_stream = nullptr;
    int *err_host = nullptr;   // pinned mirror of err: the host entry reads the flag with the same sync as its output
    int routed_t = -1;  // tokens of the current route table
    bool plan_small = false;  // the current plan's items are those of the layer's `small` kernel set
};

struct zmoe_layer {
    zmoe_ctx *ctx;
    zmoe_layer_desc d;
    // Geometries, tile maps and item spaces of the decode kernels.  Two sets: `big` (the K-chunked kernel where
    // the shapes allow it) and `small` (the kernel whose whole CTA works on one 16-row item: shorter latency
    // when there are fewer items than warp sets to give them to).  The plan of a call is built for one of them.
    struct Proj {
        MmidGeom g_gu, g_gate1, g_dn;
        CUtensorMap tm_gate, tm_up, tm_down;
        bool has_tm_gu = false, has_tm_dn = false;
        int nrt_gu = 0, nrt_dn = 0;
        int mt_gu = 4, mt_dn = 4;   // pairs per item of the two projections
    } big, small;
    bool dual;
    size_t bytes_gate, bytes_up, bytes_down;
};
// calls with at most this many pairs take the `small` set
static const int kSmallCallPairs = 8;

namespace zmoe {
int layer_route_table(zmoe_layer *L, const int32_t **ids_dev, const float **weights_dev, int *n_experts) {
    if (!L || !ids_dev || !weights_dev || !n_experts) return ZMOE_ERR_ARG;
    if (L->ctx->routed_t <= 0) return ZMOE_ERR_STATE;
    *ids_dev = L->ctx->ids;
    *weights_dev = L->ctx->weights;
    *n_experts = L->d.n_experts;
    return ZMOE_OK;
}
zmoe_ctx *layer_context(zmoe_layer *L) { return L ? L->ctx : nullptr; }
int context_path(const zmoe_ctx *c) { return c ? c->path : 0; }
}  // namespace zmoe

extern "C" {

int zmoe_ctx_create(int max_tokens, int max_d_model, int max_d_ff, int max_experts, int max_topk, zmoe_ctx **out) {
    if (!out || max_tokens <= 0 || max_d_model <= 0 || max_d_ff <= 0 || max_experts <= 0 || max_topk <= 0)
        return ZMOE_ERR_ARG;
    if (max_d_model % QK_K || max_d_ff % QK_K) return ZMOE_ERR_SHAPE;
    zmoe_ctx *c = new (std::nothrow) zmoe_ctx();
    if (!c) return ZMOE_ERR_ARG;
    c->max_t = max_tokens; c->max_d = max_d_model; c->max_f = max_d_ff; c->max_e = max_experts; c->max_k = max_topk;
    c->n_sm = sm_count();
    cudaGetDevice(&c->device);
    const size_t P = (size_t)max_tokens * max_topk;
    int rc = c->n_sm > 0 ? 0 : ZMOE_ERR_CUDA;
    rc |= dev_alloc(&c->q8x, (size_t)max_tokens * q8row_stride(max_d_model));
    rc |= dev_alloc(&c->q8x2, (size_t)max_tokens * q8row_stride(max_d_model));
    rc |= dev_alloc(&c->act, P * max_d_ff);
    rc |= dev_alloc(&c->q8act, P * q8row_stride(max_d_ff));
    rc |= dev_alloc(reinterpret_cast<uint16_t **>(&c->xq_f16), P * max_d_model);
    rc |= dev_alloc(reinterpret_cast<uint16_t **>(&c->actq_f16), P * max_d_ff);
    rc |= dev_alloc(&c->xscale, P);
    rc |= dev_alloc(&c->zero_ids, (size_t)max_tokens);
    rc |= dev_alloc(&c->one_w, (size_t)max_tokens);
    rc |= dev_alloc(&c->gate_s, (size_t)max_tokens);
    rc |= dev_alloc(&c->actscale, P);
    rc |= dev_alloc(&c->ydown, P * max_d_model);
    rc |= dev_alloc(&c->logits, (size_t)max_tokens * max_experts);
    if (max_tokens > 256) rc |= dev_alloc(&c->logits_part, (size_t)ROUTER_MAX_SPLIT * max_tokens * max_experts);
    rc |= dev_alloc(&c->ids, P);
    rc |= dev_alloc(&c->weights, P);
    rc |= c->plan.alloc(max_experts, (int)P);
    rc |= dev_alloc(&c->err, 1);
    rc |= dev_alloc(&c->bad, 2);
    rc |= dev_alloc(&c->queue, 4);
    rc |= dev_alloc(&c->ticket, 1 + ROUTER_MAX_GROUPS);
    rc |= dev_alloc(&c->x_stage, (size_t)max_tokens * max_d_model);
    rc |= dev_alloc(&c->out_stage, (size_t)max_tokens * max_d_model);
    rc |= ok(cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking));
    rc |= ok(cudaHostAlloc(reinterpret_cast<void **>(&c->err_host), sizeof(int), cudaHostAllocDefault));
    if (!rc) {
        rc |= ok(cudaMemset(c->err, 0, sizeof(int)));
        rc |= ok(cudaMemset(c->bad, 0, 2 * sizeof(int)));
        rc |= ok(cudaMemset(c->queue, 0, 4 * sizeof(int)));
        rc |= ok(cudaMemset(c->ticket, 0, (1 + ROUTER_MAX_GROUPS) * sizeof(unsigned)));
        rc |= ok(cudaMemset(c->plan.b.hdr, 0, 4 * sizeof(int)));
        rc |= ok(cudaMemset(c->zero_ids, 0, (size_t)max_tokens * sizeof(int32_t)));
        // 1.0f = 0x3f800000: fill through a host staging vector (done once)
        {
            float *ones = new (std::nothrow) float[max_tokens];
            if (!ones) rc |= ZMOE_ERR_ARG;
            else {
                for (int i = 0; i < max_tokens; ++i) ones[i] = 1.0f;
                rc |= ok(cudaMemcpy(c->one_w, ones, (size_t)max_tokens * sizeof(float), cudaMemcpyHostToDevice));
                delete[] ones;
            }
        }
    }
    if (rc) {
        zmoe_ctx_destroy(c);
        return ZMOE_ERR_CUDA;
    }
    *out = c;
    return ZMOE_OK;
}

void zmoe_ctx_destroy(zmoe_ctx *c) {
    if (!c) return;
    cudaFree(c->zero_ids); cudaFree(c->one_w); cudaFree(c->gate_s);
    cudaFree(c->xq_f16); cudaFree(c->actq_f16); cudaFree(c->xscale); cudaFree(c->actscale);
    cudaFree(c->q8x); cudaFree(c->q8x2); cudaFree(c->act); cudaFree(c->act2); cudaFree(c->q8act); cudaFree(c->ydown);
    cudaFree(c->logits); cudaFree(c->logits_part); cudaFree(c->ids); cudaFree(c->weights); cudaFree(c->err); cudaFree(c->bad); cudaFree(c->queue); cudaFree(c->ticket);
    cudaFree(c->x_stage); cudaFree(c->out_stage);
    c->plan.release();
    if (c->host_stream) cudaStreamDestroy(c->host_stream);
    if (c->err_host) cudaFreeHost(c->err_host);
    delete c;
}

// geometries, item spaces and tile maps of one set of decode kernels for a layer
static int build_proj(const zmoe_layer_desc &d, bool dual, bool allow_v2, zmoe_layer::Proj *P) {
    int rc = mmid_geometry(d.gate.type, d.d_model, d.d_ff, dual, &P->g_gu, allow_v2);
    if (!rc && !dual) {
        rc = mmid_geometry(d.up.type, d.d_model, d.d_ff, false, &P->g_gate1, allow_v2);
        // the two single projections share one item space: both on the K-chunked kernel (32-row items) or neither
        if (!rc && P->g_gu.v2 != P->g_gate1.v2) {
            rc = mmid_geometry(d.gate.type, d.d_model, d.d_ff, false, &P->g_gu, false);
            if (!rc) rc = mmid_geometry(d.up.type, d.d_model, d.d_ff, false, &P->g_gate1, false);
        }
        if (!rc) {
            // ... with the smaller tile and the fewer pairs per item of the two
            if (P->g_gate1.R < P->g_gu.R) P->g_gu.R = P->g_gate1.R; else P->g_gate1.R = P->g_gu.R;
            const int mt = P->g_gu.maxtok < P->g_gate1.maxtok ? P->g_gu.maxtok : P->g_gate1.maxtok;
            P->g_gu.maxtok = mt; P->g_gate1.maxtok = mt;
        }
    }
    if (!rc) rc = mmid_geometry(d.down.type, d.d_ff, d.d_model, false, &P->g_dn, allow_v2);
    if (rc) return rc;
    P->nrt_gu = (d.d_ff + P->g_gu.R - 1) / P->g_gu.R;
    P->nrt_dn = (d.d_model + P->g_dn.R - 1) / P->g_dn.R;
    P->mt_gu = P->g_gu.maxtok;
    P->mt_dn = P->g_dn.maxtok;
    const int rb_gu = (d.d_model / QK_K) * block_bytes(d.gate.type), rb_dn = (d.d_ff / QK_K) * block_bytes(d.down.type);
    if (P->g_gu.v2) {
        if (P->g_gu.tiled) {
            P->has_tm_gu =
                make_chunk_map(&P->tm_gate, d.gate.data_dev, d.n_experts, d.d_ff, rb_gu, d.gate.expert_stride, P->g_gu.pitch) == ZMOE_OK;
            if (dual)
                P->has_tm_gu = P->has_tm_gu && make_chunk_map(&P->tm_up, d.up.data_dev, d.n_experts, d.d_ff, rb_gu,
                                                              d.up.expert_stride, P->g_gu.pitch) == ZMOE_OK;
            if (!P->has_tm_gu) return ZMOE_ERR_CUDA;
        }
        if (!dual && P->g_gate1.tiled &&
            make_chunk_map(&P->tm_up, d.up.data_dev, d.n_experts, d.d_ff, (d.d_model / QK_K) * block_bytes(d.up.type),
                           d.up.expert_stride, P->g_gate1.pitch) != ZMOE_OK)
            return ZMOE_ERR_CUDA;
    } else if (dual && P->g_gu.rbs != rb_gu) {
        P->has_tm_gu =
            make_rows_map(&P->tm_gate, d.gate.data_dev, d.n_experts, d.d_ff, rb_gu, d.gate.expert_stride, P->g_gu.R) == ZMOE_OK &&
            make_rows_map(&P->tm_up, d.up.data_dev, d.n_experts, d.d_ff, rb_gu, d.up.expert_stride, P->g_gu.R) == ZMOE_OK;
    }
    if (P->g_dn.v2) {
        if (P->g_dn.tiled) {
            P->has_tm_dn = make_chunk_map(&P->tm_down, d.down.data_dev, d.n_experts, d.d_model, rb_dn, d.down.expert_stride,
                                          P->g_dn.pitch) == ZMOE_OK;
            if (!P->has_tm_dn) return ZMOE_ERR_CUDA;
        }
    } else if (P->g_dn.rbs != rb_dn) {
        P->has_tm_dn = make_rows_map(&P->tm_down, d.down.data_dev, d.n_experts, d.d_model, rb_dn, d.down.expert_stride,
                                     P->g_dn.R) == ZMOE_OK;
    }
    return ZMOE_OK;
}

int zmoe_layer_create(zmoe_ctx *ctx, const zmoe_layer_desc *desc, zmoe_layer **out) {
    if (!ctx || !desc || !out) return ZMOE_ERR_ARG;
    const zmoe_layer_desc &d = *desc;
    if (d.d_model <= 0 || d.d_ff <= 0 || d.n_experts <= 0 || d.topk <= 0 || d.topk > d.n_experts) return ZMOE_ERR_ARG;
    if (!d.gate.data_dev || !d.up.data_dev || !d.down.data_dev) return ZMOE_ERR_ARG;
    if (d.d_model > ctx->max_d || d.d_ff > ctx->max_f || d.n_experts > ctx->max_e || d.topk > ctx->max_k)
        return ZMOE_ERR_CAPACITY;
    if (d.d_model % QK_K || d.d_ff % QK_K) return ZMOE_ERR_SHAPE;
    zmoe_layer *L = new (std::nothrow) zmoe_layer();
    if (!L) return ZMOE_ERR_ARG;
    L->ctx = ctx;
    L->d = d;
    L->dual = d.gate.type == d.up.type;
    int rc = build_proj(d, L->dual, true, &L->big);
    if (!rc) rc = build_proj(d, L->dual, false, &L->small);
    const zmoe_weight *ws[3] = {&d.gate, &d.up, &d.down};
    size_t *tot[3] = {&L->bytes_gate, &L->bytes_up, &L->bytes_down};
    for (int i = 0; i < 3 && !rc; ++i) {
        const int I = i < 2 ? d.d_model : d.d_ff, O = i < 2 ? d.d_ff : d.d_model;
        const size_t need = (size_t)O * (I / QK_K) * block_bytes(ws[i]->type);
        if (ws[i]->expert_stride < need) rc = ZMOE_ERR_ARG;
        if ((reinterpret_cast<size_t>(ws[i]->data_dev) & 15) || (ws[i]->expert_stride & 15)) rc = ZMOE_ERR_ALIGN;
        *tot[i] = ws[i]->bytes ? ws[i]->bytes : (size_t)(d.n_experts - 1) * ws[i]->expert_stride + need;
    }
    if (!rc && !L->dual && !ctx->act2)
        rc = dev_alloc(&ctx->act2, (size_t)2 * ctx->max_t * ctx->max_k * ctx->max_f);
    if (rc) {
        delete L;
        return rc;
    }
    if (rc) {
        delete L;
        return rc;
    }
    *out = L;
    return ZMOE_OK;
}

void zmoe_layer_destroy(zmoe_layer *layer) { delete layer; }

// whether zmoe_expert_ffn will take the tensor-core grouped GEMM for T tokens (the rule of the header:
// shapes allow it, and the path is forced to 2 or left at 0 with enough pairs per expert)
static bool takes_gemm(const zmoe_layer *L, int T) {
    const zmoe_layer_desc &d = L->d;
    const zmoe_ctx *c = L->ctx;
    const bool gemm_ok = L->dual && gemm_sm100_supported(d.gate.type, d.d_model, d.d_ff) &&
                         gemm_sm100_supported(d.down.type, d.d_ff, d.d_model) && d.n_experts <= 512;
    const long P = (long)T * d.topk;
    return gemm_ok && (c->path == 2 || (c->path == 0 && P >= (long)kGemmMinPairsPerExpert * d.n_experts));
}

// packed Q8_K rows of the layer input for the decode kernels (both unit layouts where gate and up differ)
static int quantize_input(zmoe_layer *L, const float *x_dev, int T, cudaStream_t st) {
    zmoe_ctx *c = L->ctx;
    int rc = launch_quantize_rows(x_dev, L->d.d_model, c->q8x, T, L->d.d_model, q8_layout_of(L->d.gate.type), st);
    g_launches += 1;
    if (!rc && q8_layout_of(L->d.up.type) != q8_layout_of(L->d.gate.type)) {
        rc = launch_quantize_rows(x_dev, L->d.d_model, c->q8x2, T, L->d.d_model, q8_layout_of(L->d.up.type), st);
        g_launches += 1;
    }
    if (!rc) c->q8x_valid = true;
    return rc;
}

int zmoe_route(zmoe_layer *L, const float *x_dev, int T, void *stream) {
    if (!L || !x_dev || T <= 0) return ZMOE_ERR_ARG;
    zmoe_ctx *c = L->ctx;
    if (T > c->max_t) return ZMOE_ERR_CAPACITY;
    if (!L->d.router_w_dev) return ZMOE_ERR_STATE;
    RouterArgs a;
    a.x = x_dev; a.wr = L->d.router_w_dev; a.bias = L->d.router_bias_dev;
    a.T = T; a.D = L->d.d_model; a.E = L->d.n_experts; a.K = L->d.topk;
    a.gating = L->d.gating; a.normalize = L->d.weights_norm;
    a.weight_scale = L->d.weights_scale;
    a.n_groups = L->d.n_groups; a.n_groups_used = L->d.n_groups_used;
    a.logits = c->logits; a.ids = c->ids; a.weights = c->weights; a.q8x = c->q8x;
    a.q8_layout = q8_layout_of(L->d.gate.type);
    a.plan = c->plan.b;
    a.stats = gemm_stats_buffer(0);
    c->plan_small = (long)T * L->d.topk <= kSmallCallPairs;
    const zmoe_layer::Proj &ps = c->plan_small ? L->small : L->big;
    a.plan.mt_gu = ps.mt_gu; a.plan.mt_dn = ps.mt_dn;
    a.nrt_gu = ps.nrt_gu; a.nrt_dn = ps.nrt_dn;
    a.ticket = c->ticket;
    a.logits_part = c->logits_part;
    a.n_sm = c->n_sm;
    // one CTA per (expert, 4 tokens) re-reads every activation row E times: fine up to a few hundred
    // tokens (the tiled GEMM has only (E / 64) x (T / 64) CTAs: 4 at 128 tokens, 280 us per call)
    const bool big = T > 256;
    // the tensor-core path quantises the rows itself while it gathers them: the large-batch router then skips q8x
    a.want_q8x = !(big && takes_gemm(L, T));
    int rc = big ? launch_router_prefill(a, static_cast<cudaStream_t>(stream))
                 : launch_router_decode(a, static_cast<cudaStream_t>(stream));
    g_launches += big ? (a.want_q8x ? 4 : 3) : 1;
    c->q8x_valid = a.want_q8x;
    if (!rc && a.want_q8x && q8_layout_of(L->d.up.type) != a.q8_layout) {
        rc = launch_quantize_rows(x_dev, L->d.d_model, c->q8x2, T, L->d.d_model, q8_layout_of(L->d.up.type),
                                  static_cast<cudaStream_t>(stream));
        g_launches += 1;
    }
    if (!rc) { c->routed_t = T; c->x_last = x_dev; }
    return rc;
}

static int set_routes_impl(zmoe_layer *L, const float *x_dev, const int32_t *ids_dev, const float *weights_dev, int T,
                           int first_expert, bool window, void *stream, int ids_ld = 0, int w_ld = 0) {
    if (!L || !x_dev || !ids_dev || !weights_dev || T <= 0) return ZMOE_ERR_ARG;
    zmoe_ctx *c = L->ctx;
    if (T > c->max_t) return ZMOE_ERR_CAPACITY;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t P = (size_t)T * L->d.topk;
    int rc = 0;
    c->q8x_valid = false;
    if (!takes_gemm(L, T)) rc = quantize_input(L, x_dev, T, st);   // the tensor-core path quantises while it gathers
    // the planner takes the routes in (copy, window mapping) before it groups them: one launch
    PlanBuffers pb = c->plan.b;
    c->plan_small = (long)P <= kSmallCallPairs;
    const zmoe_layer::Proj &ps = c->plan_small ? L->small : L->big;
    pb.mt_gu = ps.mt_gu; pb.mt_dn = ps.mt_dn;
    if (!rc)
        rc = launch_plan_ingest(ids_dev, weights_dev, c->ids, c->weights, (int)P, L->d.n_experts, first_expert, window,
                                pb, ps.nrt_gu, ps.nrt_dn, st, ids_ld ? L->d.topk : 0, ids_ld, w_ld);
    if (!rc) { g_launches += 1; c->routed_t = T; c->x_last = x_dev; }
    return rc;
}

int zmoe_set_routes(zmoe_layer *L, const float *x_dev, const int32_t *ids_dev, const float *weights_dev, int T,
                    void *stream) {
    return set_routes_impl(L, x_dev, ids_dev, weights_dev, T, 0, false, stream);
}

int zmoe_set_routes_window(zmoe_layer *L, const float *x_dev, const int32_t *ids_dev, const float *weights_dev, int T,
                           int first_expert, void *stream) {
    if (first_expert < 0) return ZMOE_ERR_ARG;
    return set_routes_impl(L, x_dev, ids_dev, weights_dev, T, first_expert, true, stream);
}

int zmoe_set_routes_strided(zmoe_layer *L, const float *x_dev, const int32_t *ids_dev, size_t ids_token_stride,
                            const float *weights_dev, size_t weights_token_stride, int T, void *stream) {
    if (!L) return ZMOE_ERR_ARG;
    const size_t k4 = (size_t)L->d.topk * 4;
    if (ids_token_stride % 4 || weights_token_stride % 4 || ids_token_stride < k4 || weights_token_stride < k4 ||
        ids_token_stride / 4 > INT32_MAX || weights_token_stride / 4 > INT32_MAX)
        return ZMOE_ERR_ALIGN;
    return set_routes_impl(L, x_dev, ids_dev, weights_dev, T, 0, false, stream, (int)(ids_token_stride / 4),
                           (int)(weights_token_stride / 4));
}

int zmoe_expert_ffn(zmoe_layer *L, float *out_dev, int T, int accumulate, void *stream) {
    return zmoe_expert_ffn_events(L, out_dev, T, accumulate, stream, nullptr, nullptr);
}

int zmoe_expert_ffn_events(zmoe_layer *L, float *out_dev, int T, int accumulate, void *stream, void *ev_before,
                           void *ev_after) {
    if (!L || !out_dev || T <= 0) return ZMOE_ERR_ARG;
    zmoe_ctx *c = L->ctx;
    if (c->routed_t != T) return ZMOE_ERR_STATE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const zmoe_layer_desc &d = L->d;
    const int P = T * d.topk;
    MmidLaunch m;
    m.plan = c->plan.b;
    m.err = c->err;
    m.bad = c->bad;
    m.queue = c->queue;
    m.n_sm = c->n_sm;
    m.clamp = d.swiglu_clamp;
    m.clamp_fused = d.swiglu_clamp_fused;
    m.multi = T > 1 && c->path != 3;
    int rc;
    // many pairs per expert: the contraction is compute-bound and goes to the tensor cores
    const bool use_gemm = c->x_last && takes_gemm(L, T);
    if (use_gemm) {
        if (ev_before) cudaEventRecord(static_cast<cudaEvent_t>(ev_before), st);
        GemmLaunch g;
        g.plan = c->plan.b; g.err = c->err; g.bad = c->bad; g.n_sm = c->n_sm;
        g.clamp = d.swiglu_clamp; g.clamp_fused = d.swiglu_clamp_fused;
        g.n_experts = d.n_experts;
        rc = launch_q8_roundtrip_tokens_f16(c->x_last, d.d_model, c->xq_f16, c->xscale, c->plan.b, T, d.topk, d.d_model, st);
        g.type = d.gate.type; g.dual = true;
        g.w0 = d.gate.data_dev; g.w1 = d.up.data_dev;
        g.stride0 = d.gate.expert_stride; g.stride1 = d.up.expert_stride;
        g.I = d.d_model; g.O = d.d_ff;
        g.x_f16 = c->xq_f16; g.xscale = c->xscale; g.x_rows = c->max_t * c->max_k;
        g.y = c->act; g.ldy = d.d_ff;
        if (!rc) rc = launch_gemm_sm100(g, st);
        if (ev_after) cudaEventRecord(static_cast<cudaEvent_t>(ev_after), st);
        if (!rc) rc = launch_q8_roundtrip_f16(c->act, d.d_ff, c->actq_f16, c->actscale, c->plan.b, P, 1, d.d_ff, st);
        g.type = d.down.type; g.dual = false;
        g.w0 = d.down.data_dev; g.w1 = nullptr;
        g.stride0 = d.down.expert_stride; g.stride1 = 0;
        g.I = d.d_ff; g.O = d.d_model;
        g.x_f16 = c->actq_f16; g.xscale = c->actscale; g.x_rows = c->max_t * c->max_k;
        g.y = c->ydown; g.ldy = d.d_model;
        if (!rc) rc = launch_gemm_sm100(g, st);
        if (!rc) rc = launch_combine(out_dev, c->ydown, c->weights, c->ids, T, d.topk, d.d_model, d.n_experts, accumulate, st);
        g_launches += 5;
        return rc;
    }
    // the path may have been changed since the routes were set: the decode kernels need the quantised input
    if (!c->q8x_valid) {
        if (!c->x_last) return ZMOE_ERR_STATE;
        rc = quantize_input(L, c->x_last, T, st);
        if (rc) return rc;
    }
    const zmoe_layer::Proj &ps = c->plan_small ? L->small : L->big;   // the set the plan was built for
    if (ev_before) cudaEventRecord(static_cast<cudaEvent_t>(ev_before), st);
    if (L->dual) {
        m.type = d.gate.type; m.dual = true;
        m.w0 = d.gate.data_dev; m.w1 = d.up.data_dev;
        m.stride0 = d.gate.expert_stride; m.stride1 = d.up.expert_stride;
        m.total0 = L->bytes_gate; m.total1 = L->bytes_up;
        m.I = d.d_model; m.O = d.d_ff;
        m.q8 = c->q8x; m.xdiv = d.topk;
        m.y = c->act; m.ldy = d.d_ff;
        m.down = false;
        if (ps.has_tm_gu) { m.tm0 = &ps.tm_gate; m.tm1 = &ps.tm_up; }
        rc = launch_mmid(m, ps.g_gu, st);
        m.tm0 = nullptr; m.tm1 = nullptr;
        g_launches += 1;
    } else {
        float *gbuf = c->act2, *ubuf = c->act2 + (size_t)P * d.d_ff;
        m.dual = false; m.w1 = nullptr; m.stride1 = 0; m.total1 = 0;
        m.I = d.d_model; m.O = d.d_ff; m.q8 = c->q8x; m.xdiv = d.topk; m.ldy = d.d_ff; m.down = false;
        m.type = d.up.type; m.w0 = d.up.data_dev; m.stride0 = d.up.expert_stride; m.total0 = L->bytes_up; m.y = ubuf;
        if (q8_layout_of(d.up.type) != q8_layout_of(d.gate.type)) m.q8 = c->q8x2;
        m.tm0 = ps.g_gate1.v2 && ps.g_gate1.tiled ? &ps.tm_up : nullptr;
        rc = launch_mmid(m, ps.g_gate1, st);
        m.q8 = c->q8x;
        m.type = d.gate.type; m.w0 = d.gate.data_dev; m.stride0 = d.gate.expert_stride; m.total0 = L->bytes_gate; m.y = gbuf;
        m.tm0 = ps.g_gu.v2 && ps.g_gu.tiled ? &ps.tm_gate : nullptr;
        if (!rc) rc = launch_mmid(m, ps.g_gu, st);
        m.tm0 = nullptr;
        if (!rc) {
            launch_expert_swiglu(c->act, gbuf, ubuf, P * d.d_ff, d.swiglu_clamp, d.swiglu_clamp_fused, c->bad, stream);
            rc = ok(cudaPeekAtLastError());
        }
        g_launches += 3;
    }
    if (ev_after) cudaEventRecord(static_cast<cudaEvent_t>(ev_after), st);
    if (!rc) rc = launch_quantize_rows(c->act, d.d_ff, c->q8act, P, d.d_ff, q8_layout_of(d.down.type), st);
    if (!rc) {
        m.type = d.down.type; m.dual = false;
        m.w0 = d.down.data_dev; m.w1 = nullptr;
        m.stride0 = d.down.expert_stride; m.stride1 = 0;
        m.total0 = L->bytes_down; m.total1 = 0;
        m.I = d.d_ff; m.O = d.d_model;
        m.q8 = c->q8act; m.xdiv = 1;
        m.y = c->ydown; m.ldy = d.d_model;
        m.down = true;
        if (ps.has_tm_dn) m.tm0 = &ps.tm_down;
        rc = launch_mmid(m, ps.g_dn, st);
    }
    if (!rc) rc = launch_combine(out_dev, c->ydown, c->weights, c->ids, T, d.topk, d.d_model, d.n_experts, accumulate, st);
    g_launches += 3;
    return rc;
}

int zmoe_dense_ffn(zmoe_layer *L, const float *x_dev, float *out_dev, int T, int accumulate, void *stream) {
    if (!L || !x_dev || !out_dev || T <= 0) return ZMOE_ERR_ARG;
    if (L->d.n_experts != 1 || L->d.topk != 1) return ZMOE_ERR_STATE;
    if (T > L->ctx->max_t) return ZMOE_ERR_CAPACITY;
    int rc = zmoe_set_routes(L, x_dev, L->ctx->zero_ids, L->ctx->one_w, T, stream);
    if (!rc) rc = zmoe_expert_ffn(L, out_dev, T, accumulate, stream);
    return rc;
}

int zmoe_dense_ffn_gated(zmoe_layer *L, const float *x_dev, const float *gate_w_dev, float *out_dev, int T, int accumulate,
                         void *stream) {
    if (!L || !x_dev || !gate_w_dev || !out_dev || T <= 0) return ZMOE_ERR_ARG;
    if (L->d.n_experts != 1 || L->d.topk != 1) return ZMOE_ERR_STATE;
    if (T > L->ctx->max_t) return ZMOE_ERR_CAPACITY;
    // the scalar gate rides as the route weight: the combine multiplies each token's row by it
    int rc = launch_token_gate(x_dev, gate_w_dev, L->ctx->gate_s, T, L->d.d_model, static_cast<cudaStream_t>(stream));
    g_launches += 1;
    if (!rc) rc = zmoe_set_routes(L, x_dev, L->ctx->zero_ids, L->ctx->gate_s, T, stream);
    if (!rc) rc = zmoe_expert_ffn(L, out_dev, T, accumulate, stream);
    return rc;
}

int zmoe_moe_forward(zmoe_layer *L, const float *x_dev, float *out_dev, int T, void *stream) {
    int rc = zmoe_route(L, x_dev, T, stream);
    if (!rc) rc = zmoe_expert_ffn(L, out_dev, T, 0, stream);
    return rc;
}

int zmoe_moe_forward_bf16(zmoe_layer *L, const void *x_bf16_dev, float *out_dev, int T, void *stream) {
    if (!L || !x_bf16_dev || !out_dev || T <= 0) return ZMOE_ERR_ARG;
    zmoe_ctx *c = L->ctx;
    if (T > c->max_t) return ZMOE_ERR_CAPACITY;
    // widened once into the context's staging rows (exact); router and matmuls then read f32 as ever
    int rc = launch_widen_bf16(x_bf16_dev, c->x_stage, (long)T * L->d.d_model, c->n_sm, static_cast<cudaStream_t>(stream));
    g_launches += 1;
    if (!rc) rc = zmoe_moe_forward(L, c->x_stage, out_dev, T, stream);
    return rc;
}

int zmoe_moe_forward_host(zmoe_layer *L, const float *x_host, float *out_host, int T) {
    if (!L || !x_host || !out_host || T <= 0) return ZMOE_ERR_ARG;
    zmoe_ctx *c = L->ctx;
    if (T > c->max_t) return ZMOE_ERR_CAPACITY;
    const size_t n = (size_t)T * L->d.d_model * sizeof(float);
    int rc = ok(cudaMemcpyAsync(c->x_stage, x_host, n, cudaMemcpyHostToDevice, c->host_stream));
    if (!rc) rc = zmoe_moe_forward(L, c->x_stage, c->out_stage, T, c->host_stream);
    if (!rc) rc = ok(cudaMemcpyAsync(out_host, c->out_stage, n, cudaMemcpyDeviceToHost, c->host_stream));
    // the device error flag rides on the same stream: one synchronisation for output and status
    if (!rc) rc = ok(cudaMemcpyAsync(c->err_host, c->err, sizeof(int), cudaMemcpyDeviceToHost, c->host_stream));
    if (!rc) rc = ok(cudaStreamSynchronize(c->host_stream));
    if (!rc && *c->err_host) {
        cudaMemset(c->err, 0, sizeof(int));
        cudaMemset(c->queue, 0, 4 * sizeof(int));   // a launch that gave up may have left its tickets behind
        rc = ZMOE_ERR_DEVICE_WAIT;
    }
    return rc;
}

int zmoe_get_routes(zmoe_ctx *c, int T, int topk, int32_t *ids_host, float *weights_host) {
    if (!c || T <= 0 || topk <= 0 || (size_t)T * topk > (size_t)c->max_t * c->max_k) return ZMOE_ERR_ARG;
    int rc = 0;
    if (ids_host) rc |= ok(cudaMemcpy(ids_host, c->ids, (size_t)T * topk * sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (weights_host) rc |= ok(cudaMemcpy(weights_host, c->weights, (size_t)T * topk * sizeof(float), cudaMemcpyDeviceToHost));
    return rc ? ZMOE_ERR_CUDA : ZMOE_OK;
}

int zmoe_copy_routes(zmoe_ctx *c, int T, int topk, int32_t *ids_dev, float *weights_dev, void *stream) {
    if (!c || T <= 0 || topk <= 0 || (size_t)T * topk > (size_t)c->max_t * c->max_k) return ZMOE_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = 0;
    if (ids_dev) rc |= ok(cudaMemcpyAsync(ids_dev, c->ids, (size_t)T * topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
    if (weights_dev) rc |= ok(cudaMemcpyAsync(weights_dev, c->weights, (size_t)T * topk * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return rc ? ZMOE_ERR_CUDA : ZMOE_OK;
}

int zmoe_get_expert_freq(zmoe_ctx *c, int n_experts, int32_t *freq_host) {
    if (!c || !freq_host || n_experts <= 0 || n_experts > c->max_e) return ZMOE_ERR_ARG;
    return ok(cudaMemcpy(freq_host, c->plan.b.freq, (size_t)n_experts * sizeof(int32_t), cudaMemcpyDeviceToHost));
}

int zmoe_get_probs(zmoe_ctx *c, int T, int n_experts, float *probs_host) {
    if (!c || !probs_host || T <= 0 || (size_t)T * n_experts > (size_t)c->max_t * c->max_e) return ZMOE_ERR_ARG;
    return ok(cudaMemcpy(probs_host, c->logits, (size_t)T * n_experts * sizeof(float), cudaMemcpyDeviceToHost));
}

int zmoe_get_act(zmoe_ctx *c, int n_pairs, int d_ff, float *act_host) {
    if (!c || !act_host || n_pairs <= 0 || (size_t)n_pairs * d_ff > (size_t)c->max_t * c->max_k * c->max_f) return ZMOE_ERR_ARG;
    return ok(cudaMemcpy(act_host, c->act, (size_t)n_pairs * d_ff * sizeof(float), cudaMemcpyDeviceToHost));
}

int zmoe_ctx_set_path(zmoe_ctx *c, int path) {
    if (!c || path < 0 || path > 3) return ZMOE_ERR_ARG;
    c->path = path;
    return ZMOE_OK;
}

int zmoe_ctx_check(zmoe_ctx *c) {
    if (!c) return ZMOE_ERR_ARG;
    int e = 0;
    if (cudaMemcpy(&e, c->err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ZMOE_ERR_CUDA;
    if (e) {
        cudaMemset(c->err, 0, sizeof(int));
        cudaMemset(c->queue, 0, 4 * sizeof(int));   // a launch that gave up may have left its tickets behind
        return ZMOE_ERR_DEVICE_WAIT;
    }
    return ZMOE_OK;
}

int zmoe_ctx_bad_counts(zmoe_ctx *c, int32_t *counts_host, int clear) {
    if (!c || !counts_host) return ZMOE_ERR_ARG;
    if (cudaMemcpy(counts_host, c->bad, 2 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ZMOE_ERR_CUDA;
    if (clear && (counts_host[0] | counts_host[1]) && cudaMemset(c->bad, 0, 2 * sizeof(int)) != cudaSuccess)
        return ZMOE_ERR_CUDA;
    return ZMOE_OK;
}

int zmoe_gemm_min_pairs_per_expert(void) { return kGemmMinPairsPerExpert; }

int zmoe_debug_gemm_cycles(uint64_t *counters32_host) {
    if (!counters32_host) return ZMOE_ERR_ARG;
    if (cudaDeviceSynchronize() != cudaSuccess) return ZMOE_ERR_CUDA;
    return gemm_stats_read(reinterpret_cast<unsigned long long *>(counters32_host));
}

uint64_t zmoe_kernel_launches(void) { return g_launches.load(); }

}  // extern "C"

// ---------------------------------------------------------------------------
// per-device scratch of the handle-free entry points
// ---------------------------------------------------------------------------
namespace {

struct DeviceScratch {
    uint8_t *q8 = nullptr;
    size_t q8_bytes = 0;
    PlanStore plan;
    int *err = nullptr;
    int32_t *ids = nullptr;
    size_t ids_cap = 0;
    int n_sm = 0;
};
constexpr int kMaxDevices = 64;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_scratch_mu;

using ScratchLock = std::unique_lock<std::mutex>;

// Makes sure the current device's scratch can hold `rows` packed rows of I elements, a plan for E experts
// and P pairs, and hands it out LOCKED: the caller keeps `lock` until its kernels are enqueued, so no other
// host thread can grow (free and reallocate) the buffers between this call's launches.  Growing waits for
// the device first, so kernels already enqueued never see a freed buffer.
int scratch_get(int rows, int I, int E, int P, DeviceScratch **out, ScratchLock &lock) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ZMOE_ERR_CUDA;
    lock = ScratchLock(g_scratch_mu);
    DeviceScratch &s = g_scratch[dev];
    if (!s.n_sm) s.n_sm = sm_count();
    const size_t need = (size_t)rows * q8row_stride(I);
    if (need > s.q8_bytes) {
        if (s.q8) { cudaDeviceSynchronize(); cudaFree(s.q8); }
        if (dev_alloc(&s.q8, need)) return ZMOE_ERR_CUDA;
        s.q8_bytes = need;
    }
    if (E > s.plan.cap_e || P > s.plan.cap_p) {
        const int ne = E > s.plan.cap_e ? E : s.plan.cap_e, np = P > s.plan.cap_p ? P : s.plan.cap_p;
        if (s.plan.cap_e) { cudaDeviceSynchronize(); s.plan.release(); }
        if (s.plan.alloc(ne, np)) return ZMOE_ERR_CUDA;
    }
    if ((size_t)P > s.ids_cap) {
        if (s.ids) { cudaDeviceSynchronize(); cudaFree(s.ids); }
        if (dev_alloc(&s.ids, (size_t)P)) return ZMOE_ERR_CUDA;
        s.ids_cap = P;
    }
    if (!s.err) {
        if (dev_alloc(&s.err, 1)) return ZMOE_ERR_CUDA;
        cudaMemset(s.err, 0, sizeof(int));
    }
    *out = &s;
    return ZMOE_OK;
}

int dense_matmul(int type, float *y, const float *x, int ldx, const void *w, int S, int I, int O, int ldy,
                 cudaStream_t st) {
    if (!y || !x || !w || S <= 0 || I <= 0 || O <= 0) return ZMOE_ERR_ARG;
    MmidGeom g;
    int rc = mmid_geometry(type, I, O, false, &g);
    if (rc) return rc;
    DeviceScratch *s;
    ScratchLock lock;
    rc = scratch_get(S, I, 1, S, &s, lock);
    if (rc) return rc;
    const int nrt = (O + g.R - 1) / g.R;
    rc = launch_quantize_rows(x, ldx, s->q8, S, I, q8_layout_of(type), st);
    if (!rc) rc = launch_plan_dense(S, s->plan.b, nrt, st);
    if (rc) return rc;
    MmidLaunch m;
    m.type = type; m.dual = false;
    m.w0 = w; m.w1 = nullptr;
    m.stride0 = 0; m.stride1 = 0;
    m.total0 = (size_t)O * (I / QK_K) * block_bytes(type); m.total1 = 0;
    m.I = I; m.O = O;
    m.q8 = s->q8; m.xdiv = 1;
    m.y = y; m.ldy = ldy;
    m.plan = s->plan.b;
    m.down = false;
    m.clamp = 0.f; m.clamp_fused = 0;
    m.err = s->err;
    m.n_sm = s->n_sm;
    m.multi = S > 1;
    rc = launch_mmid(m, g, st);
    g_launches += 3;
    return rc;
}

// rows of y whose expert id is >= E become NaN (ids < 0 stay zero)
__global__ void fill_bad_rows_kernel(float *y, int ldy, const int32_t *ids, int P, int E, int O) {
    const int p = blockIdx.x;
    if (p >= P || ids[p] < E) return;
    for (int o = threadIdx.x; o < O; o += blockDim.x) y[(size_t)p * ldy + o] = nanf("");
}
void fill_bad_rows(float *y, int ldy, const int32_t *ids, int P, int E, int O, cudaStream_t st) {
    fill_bad_rows_kernel<<<P, 128, 0, st>>>(y, ldy, ids, P, E, O);
}

// One warp waits, with a short limit, on a barrier that nobody arrives on: the wait runs out, the warp raises
// the error word exactly as the matmul kernels do, and returns.  Exists so that the path from an expired
// device-side wait to ZMOE_ERR_DEVICE_WAIT can be exercised without a hang or a fault.
__global__ void wait_expiry_probe_kernel(int *err) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncwarp();
    if (!mbar_wait(&bar, 0, 256) && threadIdx.x == 0) atomicExch(err, 1);
}

__global__ void gather_ids_kernel(const uint8_t *src, size_t nb0, size_t nb1, int32_t *dst, int K, int T) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= K * T) return;
    const int t = i / K, k = i % K;
    dst[i] = *reinterpret_cast<const int32_t *>(src + t * nb1 + k * nb0);
}

}  // namespace

extern "C" {

int zmoe_reserve(int rows, int I) {
    if (rows <= 0 || I <= 0 || I % QK_K) return ZMOE_ERR_ARG;
    DeviceScratch *s;
    ScratchLock lock;
    return scratch_get(rows, I, 1, rows, &s, lock);
}

int zmoe_last_status(void) { return tl_status; }

int zmoe_device_status(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ZMOE_ERR_CUDA;
    if (cudaDeviceSynchronize() != cudaSuccess) return ZMOE_ERR_CUDA;
    int seen = 0;
    {
        ScratchLock lock(g_scratch_mu);
        DeviceScratch &s = g_scratch[dev];
        if (s.err) {
            int e = 0;
            if (cudaMemcpy(&e, s.err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ZMOE_ERR_CUDA;
            if (e) {
                seen = e;
                if (cudaMemset(s.err, 0, sizeof(int)) != cudaSuccess) return ZMOE_ERR_CUDA;
            }
        }
    }
    int e2 = 0;
    if (noalloc_take_error(&e2)) return ZMOE_ERR_CUDA;
    return (seen || e2) ? ZMOE_ERR_DEVICE_WAIT : ZMOE_OK;
}

int zmoe_selftest_wait_expiry(void *stream) {
    DeviceScratch *s;
    ScratchLock lock;
    int rc = scratch_get(1, QK_K, 1, 1, &s, lock);
    if (rc) return rc;
    wait_expiry_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(s->err);
    g_launches += 1;
    return ok(cudaPeekAtLastError());
}

#define ZMOE_DENSE(name, type)                                                                         \
    void name##_stream(float *y, const float *x, const void *w, int S, int I, int O, void *stream) {     \
        tl_status = dense_matmul(type, y, x, I, w, S, I, O, O, static_cast<cudaStream_t>(stream));      \
    }                                                                                                    \
    void name(float *y, const float *x, const void *w, int S, int I, int O) {                            \
        tl_status = dense_matmul(type, y, x, I, w, S, I, O, O, nullptr);                                \
    }

ZMOE_DENSE(launch_q2_K_matmul, Q2_K)
ZMOE_DENSE(launch_q3_K_matmul, Q3_K)
ZMOE_DENSE(launch_q4_K_matmul, Q4_K)
ZMOE_DENSE(launch_iq2_xxs_matmul, IQ2_XXS)

bool zmoe_f32_quant_hook(const zmoe_tensor *w, const zmoe_tensor *x, const zmoe_tensor *ids,
                         zmoe_tensor *y, void *stream, bool execute) {
    constexpr int GGML_F32 = 0, GGML_I32 = 26;
    if (!w || !x || !y || block_bytes(w->type) == 0 || x->type != GGML_F32 || y->type != GGML_F32 || w->ne[0] <= 0 ||
        w->ne[0] > INT32_MAX || w->ne[1] <= 0 || w->ne[1] > INT32_MAX || w->ne[0] % 256 || x->nb[0] != sizeof(float) ||
        y->nb[0] != sizeof(float))
        return false;
    const int I = (int)w->ne[0], O = (int)w->ne[1];
    const size_t row = (size_t)(I / 256) * block_bytes(w->type);
    if (w->nb[1] != row || x->ne[0] != I || y->ne[0] != O) return false;
    MmidGeom g;
    if (mmid_geometry(w->type, I, O, false, &g) != ZMOE_OK) return false;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (ids) {
        if (ids->type != GGML_I32 || ids->nb[0] != sizeof(int32_t) || ids->ne[0] <= 0 || ids->ne[0] > 65535 ||
            ids->ne[1] <= 0 || ids->ne[1] > 65535 || w->ne[2] <= 0 || w->ne[2] > INT32_MAX || w->ne[3] != 1 ||
            (x->ne[1] != 1 && x->ne[1] != ids->ne[0]) || x->ne[2] != ids->ne[1] || x->ne[3] != 1 ||
            y->ne[1] != ids->ne[0] || y->ne[2] != ids->ne[1] || y->ne[3] != 1)
            return false;
        const int K = (int)ids->ne[0], T = (int)ids->ne[1], E = (int)w->ne[2];
        const int xr = (int)x->ne[1];
        // rows of x and y must form one evenly strided list of pairs
        if (x->nb[1] % 4 || x->nb[2] % 4 || y->nb[1] % 4) return false;
        if (xr != 1 && x->nb[2] != (size_t)xr * x->nb[1]) return false;
        if (y->nb[2] != (size_t)K * y->nb[1]) return false;
        if ((reinterpret_cast<size_t>(w->data) & 15) || (w->nb[2] & 15)) return false;
        if (!execute) return true;
        DeviceScratch *s;
        ScratchLock lock;
        const int rows = T * xr;
        if (scratch_get(rows, I, E, K * T, &s, lock)) return false;
        const int ldx = xr == 1 ? (int)(x->nb[2] / 4) : (int)(x->nb[1] / 4);
        int rc = launch_quantize_rows(static_cast<const float *>(x->data), ldx, s->q8, rows, I, q8_layout_of(w->type), st);
        gather_ids_kernel<<<(K * T + 255) / 256, 256, 0, st>>>(static_cast<const uint8_t *>(ids->data), ids->nb[0],
                                                               ids->nb[1], s->ids, K, T);
        const int nrt = (O + g.R - 1) / g.R;
        if (!rc) rc = launch_plan_from_ids(s->ids, K * T, E, s->plan.b, nrt, nrt, st);
        // inactive and out-of-range routes: zero / NaN rows (reference kernels/quant/kquant_matmul.cu:659-662)
        if (!rc) rc = ok(cudaMemsetAsync(y->data, 0, (size_t)T * y->nb[2], st));
        MmidLaunch m;
        m.type = w->type; m.dual = false;
        m.w0 = w->data; m.w1 = nullptr;
        m.stride0 = w->nb[2]; m.stride1 = 0;
        m.total0 = (size_t)(E - 1) * w->nb[2] + (size_t)O * row; m.total1 = 0;
        m.I = I; m.O = O;
        m.q8 = s->q8; m.xdiv = xr == 1 ? K : 1;
        m.y = static_cast<float *>(y->data); m.ldy = (int)(y->nb[1] / 4);
        m.plan = s->plan.b; m.down = false;
        m.clamp = 0.f; m.clamp_fused = 0;
        m.err = s->err; m.n_sm = s->n_sm;
        m.multi = T > 1;
        if (!rc) rc = launch_mmid(m, g, st);
        if (!rc) fill_bad_rows(m.y, m.ldy, s->ids, K * T, E, O, st);
        g_launches += 5;
        if (rc) return false;
    } else if (w->ne[2] == 1 && w->ne[3] == 1 && x->ne[2] == 1 && x->ne[3] == 1 && x->ne[1] > 0 && x->ne[1] <= 65535 &&
               y->ne[1] == x->ne[1] && x->nb[1] % 4 == 0 && y->nb[1] % 4 == 0) {
        if (reinterpret_cast<size_t>(w->data) & 15) return false;
        if (!execute) return true;
        if (dense_matmul(w->type, static_cast<float *>(y->data), static_cast<const float *>(x->data), (int)(x->nb[1] / 4),
                         w->data, (int)x->ne[1], I, O, (int)(y->nb[1] / 4), st))
            return false;
    } else {
        return false;
    }
    g_hook_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaPeekAtLastError() == cudaSuccess;
}

bool zeromoe_install_f32_quant_graph_hook(void) { return false; }
uint64_t zeromoe_f32_quant_graph_launches(void) { return g_hook_launches.load(std::memory_order_relaxed); }

// ---------------------------------------------------------------------------
// parity hooks
// ---------------------------------------------------------------------------
int zmoe_quantize_q8_K(const float *x_dev, void *blocks_dev, int rows, int I, int for_type, void *stream) {
    if (!x_dev || !blocks_dev || rows <= 0 || I <= 0 || I % QK_K) return ZMOE_ERR_ARG;
    if (block_bytes(for_type) == 0) return ZMOE_ERR_TYPE;
    DeviceScratch *s;
    ScratchLock lock;
    int rc = scratch_get(rows, I, 1, rows, &s, lock);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // quantise into the packed row layout that weight format uses, then regroup into ggml blocks
    const int layout = q8_layout_of(for_type);
    if (!rc) rc = launch_quantize_rows(x_dev, I, s->q8, rows, I, layout, st);
    if (!rc) rc = launch_q8rows_to_blocks(s->q8, static_cast<uint8_t *>(blocks_dev), rows, I, layout, st);
    g_launches += 2;
    return rc;
}

int zmoe_block_isums(int type, const void *w_dev, const float *x_dev, int32_t *isum_dev, int32_t *msum_dev, int rows,
                     int I, void *stream) {
    if (!w_dev || !x_dev || !isum_dev || !msum_dev || rows <= 0 || I <= 0 || I % QK_K) return ZMOE_ERR_ARG;
    if (block_bytes(type) == 0) return ZMOE_ERR_TYPE;
    DeviceScratch *s;
    ScratchLock lock;
    int rc = scratch_get(rows, I, 1, rows, &s, lock);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!rc) rc = launch_quantize_rows(x_dev, I, s->q8, rows, I, q8_layout_of(type), st);
    if (!rc) rc = launch_block_isums(type, w_dev, s->q8, isum_dev, msum_dev, rows, I, st);
    g_launches += 2;
    return rc;
}

int zmoe_block_isums_pairs(int type, const void *w_dev, const float *x_dev, int32_t *sums_dev, int pairs, int I, void *stream) {
    if (!w_dev || !x_dev || !sums_dev || pairs < 1 || pairs > 4 || I <= 0 || I % QK_K) return ZMOE_ERR_ARG;
    if (block_bytes(type) == 0) return ZMOE_ERR_TYPE;
    DeviceScratch *s;
    ScratchLock lock;
    int rc = scratch_get(pairs, I, 1, pairs, &s, lock);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!rc) rc = launch_quantize_rows(x_dev, I, s->q8, pairs, I, q8_layout_of(type), st);
    if (!rc) rc = launch_mma_isums(type, w_dev, s->q8, sums_dev, I, pairs, st);
    g_launches += 2;
    return rc;
}

}  // extern "C"

