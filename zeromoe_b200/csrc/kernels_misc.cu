// kernels_misc.cu -- the small kernels around the expert matmuls: router with
// fused activation quantisation and planning, stand-alone planners, the Q8_K
// row quantiser, the weighted combine, and the reference-ABI SwiGLU /
// scatter-accumulate / router-top-k kernels.
#include "q8k.cuh"
#include "router.cuh"
#include "zmoe_internal.h"

namespace zmoe {

// ------------------------------------------------------------------------
// decode-shaped router.  CTA (e, g) computes the logit of expert e for the
// ROUTER_TPB tokens of group g, with the expert's router row held in registers,
// and quantises a share of the activation blocks; the CTA that finishes last
// routes all tokens and builds the plan.
// ------------------------------------------------------------------------
constexpr int ROUTER_TPB = 4;      // tokens per CTA
static_assert(ROUTER_TPB * ROUTER_MAX_GROUPS >= 256, "the decode router serves batches of up to 256 tokens");
constexpr int ROUTER_THREADS = 256;
constexpr int ROUTER_MAXV = 8;     // float4 per thread: rows up to 8192 elements
constexpr int ROUTER_IDS_SMEM = 2048;  // pairs whose ids the planner mirrors in shared memory

__global__ void __launch_bounds__(ROUTER_THREADS) router_decode_kernel(const RouterArgs a) {
    extern __shared__ __align__(16) uint8_t dyn[];
    __shared__ unsigned s_ticket;
    __shared__ float s_part[ROUTER_THREADS / 32][ROUTER_TPB];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int NW = ROUTER_THREADS / 32;
    pdl_wait_prior_grid();
    pdl_launch_dependents();
#ifdef ZMOE_GEMM_STATS
    unsigned long long rt[6];
    auto now = []() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    rt[0] = now();
#endif

    const int e = blockIdx.x % a.E, tg = blockIdx.x / a.E;
    const int t0 = tg * ROUTER_TPB;
    const int nv = a.D / 4;  // float4 per row
    if (t0 < a.T) {
        const float4 *wrow = reinterpret_cast<const float4 *>(a.wr + (size_t)e * a.D);
        float4 w[ROUTER_MAXV];
#pragma unroll
        for (int i = 0; i < ROUTER_MAXV; ++i) {
            const int d = tid + i * ROUTER_THREADS;
            w[i] = d < nv ? __ldg(wrow + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float acc[ROUTER_TPB];
#pragma unroll
        for (int tt = 0; tt < ROUTER_TPB; ++tt) {
            acc[tt] = 0.f;
            const int t = t0 + tt;
            if (t < a.T) {
                const float4 *xr = reinterpret_cast<const float4 *>(a.x + (size_t)t * a.D);
                float4 v[ROUTER_MAXV];
#pragma unroll
                for (int i = 0; i < ROUTER_MAXV; ++i) {
                    const int d = tid + i * ROUTER_THREADS;
                    v[i] = d < nv ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < ROUTER_MAXV; ++i) {
                    acc[tt] = fmaf(w[i].x, v[i].x, acc[tt]); acc[tt] = fmaf(w[i].y, v[i].y, acc[tt]);
                    acc[tt] = fmaf(w[i].z, v[i].z, acc[tt]); acc[tt] = fmaf(w[i].w, v[i].w, acc[tt]);
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < ROUTER_TPB; ++tt) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], off);
            if (lane == 0) s_part[warp][tt] = acc[tt];
        }
        __syncthreads();
        if (tid < ROUTER_TPB && t0 + tid < a.T) {
            float sum = 0.f;
#pragma unroll
            for (int wv = 0; wv < NW; ++wv) sum += s_part[wv][tid];
            a.logits[(size_t)(t0 + tid) * a.E + e] = sum;
        }
    }
    const int nb = a.D / QK_K, stride = q8row_stride(a.D);
    for (int idx = blockIdx.x * NW + warp; idx < a.T * nb; idx += gridDim.x * NW) {
        const int t = idx / nb, b = idx % nb;
        quantize_block_q8k(a.x + (size_t)t * a.D + QK_K * b, a.q8x + (size_t)t * stride, a.D, b, lane, a.q8_layout);
    }
    // Two levels of tickets: the last of the E CTAs of a token group routes that group's tokens (one warp per
    // token) while other groups are still computing logits; the last group to finish builds the plan.
#ifdef ZMOE_GEMM_STATS
    rt[1] = now();
#endif
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&a.ticket[1 + tg], 1u);
    __syncthreads();
    if (s_ticket != (unsigned)a.E - 1) return;
    __threadfence();
#ifdef ZMOE_GEMM_STATS
    rt[2] = now();
#endif

    float *prob_s = reinterpret_cast<float *>(dyn) + (size_t)warp * 2 * a.E;
    float *sel_s = prob_s + a.E;
    int *cnt_s = reinterpret_cast<int *>(reinterpret_cast<float *>(dyn) + (size_t)2 * NW * a.E);
    int *pre_s = cnt_s + a.E + 1;
    int *ids_s = a.T * a.K <= ROUTER_IDS_SMEM ? pre_s + a.E + 1 : nullptr;
    RouterSpec sp{a.E, a.K, a.gating, a.normalize, a.weight_scale, a.n_groups, a.n_groups_used};
    for (int t = t0 + warp; t < a.T && t < t0 + ROUTER_TPB; t += NW)
        route_token_warp(sp, a.logits + (size_t)t * a.E, a.logits + (size_t)t * a.E, a.bias,
                         a.ids + (size_t)t * a.K, a.weights + (size_t)t * a.K, prob_s, sel_s, lane);
#ifdef ZMOE_GEMM_STATS
    rt[3] = now();
#endif
    __threadfence();
    __syncthreads();
    const unsigned n_tg = (unsigned)((a.T + ROUTER_TPB - 1) / ROUTER_TPB);
    if (tid == 0) {
        a.ticket[1 + tg] = 0u;
        s_ticket = atomicAdd(&a.ticket[0], 1u);
    }
    __syncthreads();
    if (s_ticket != n_tg - 1) return;
    __threadfence();
#ifdef ZMOE_GEMM_STATS
    rt[4] = now();
#endif
    PlanOut po{a.plan.hdr, a.plan.active, a.plan.offs, a.plan.slot, a.plan.item_offs_gu, a.plan.item_offs_dn,
               a.plan.freq, a.plan.aoffs, a.plan.antok, a.nrt_gu, a.nrt_dn, a.plan.pos, a.plan.mt_gu, a.plan.mt_dn};
    build_plan_cta(a.ids, a.T * a.K, a.E, po, cnt_s, pre_s, ids_s);
    if (tid == 0) a.ticket[0] = 0u;
#ifdef ZMOE_GEMM_STATS
    // phases of the CTA that ends the kernel, in ns: logits + quantise, ticket, routing, ticket, plan; calls
    __syncthreads();
    rt[5] = now();
    if (tid == 0 && a.stats) {
        for (int i = 0; i < 5; ++i) atomicAdd(&a.stats[8 + i], rt[i + 1] - rt[i]);
        atomicAdd(&a.stats[13], 1ull);
    }
#endif
}

int launch_router_decode(const RouterArgs &a, cudaStream_t st) {
    if (a.D / 4 > ROUTER_MAXV * ROUTER_THREADS) return ZMOE_ERR_SHAPE;
    if ((a.T + ROUTER_TPB - 1) / ROUTER_TPB > ROUTER_MAX_GROUPS) return ZMOE_ERR_CAPACITY;
    const size_t smem = (size_t)2 * (ROUTER_THREADS / 32) * a.E * sizeof(float) + (size_t)2 * (a.E + 1) * sizeof(int) +
                        (a.T * a.K <= ROUTER_IDS_SMEM ? (size_t)a.T * a.K * sizeof(int) : 0);
    if (smem > 200 * 1024) return ZMOE_ERR_SHAPE;
    if (raise_dynamic_smem(reinterpret_cast<const void *>(router_decode_kernel), 200 * 1024) != ZMOE_OK)
        return ZMOE_ERR_CUDA;
    const long grid = (long)a.E * ((a.T + ROUTER_TPB - 1) / ROUTER_TPB);
    if (grid > 0x7fffffffL) return ZMOE_ERR_SHAPE;
    return launch_pdl(router_decode_kernel, dim3((unsigned)grid), dim3(ROUTER_THREADS), smem, st, a) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------
// prefill-shaped router: logits[T, E] = x[T, D] . wr[E, D]^T as a tiled f32 GEMM (64 x 64 tile,
// 4 x 4 per thread), then one warp per token for gating / top-k, then the stand-alone planner.
// Replaces the per-token dense_proj + partial_sort loop of reference
// core/moe_router_service.cpp:1202-1214,1409-1474 for batches where one CTA per
// (expert, 4 tokens) would re-read the activations too often.
// ------------------------------------------------------------------------
__global__ void __launch_bounds__(256) router_logits_gemm_kernel(const float *__restrict__ x,
                                                                 const float *__restrict__ wr,
                                                                 float *__restrict__ logits, int T, int D, int E,
                                                                 int ksplit) {
    __shared__ float xs[16][64 + 4], ws[16][64 + 4];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int t0 = blockIdx.y * 64, e0 = blockIdx.x * 64;
    // blockIdx.z takes the z-th part of k and writes the z-th partial matrix (summed in a fixed order by
    // router_select_kernel): more CTAs in flight than one 64 x 64 tile per SM gives
    const int kper = D / ksplit, kbeg = blockIdx.z * kper, kend = kbeg + kper;
    float *out = logits + (size_t)blockIdx.z * T * E;
    const int lr = tid >> 2, lc = (tid & 3) * 4;       // loader: row 0..63, k offset 0,4,8,12
    const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;  // compute: 4 tokens x 4 experts
    float acc[4][4] = {};
    for (int k0 = kbeg; k0 < kend; k0 += 16) {
        float4 xv = make_float4(0.f, 0.f, 0.f, 0.f), wv = xv;
        if (t0 + lr < T) xv = *reinterpret_cast<const float4 *>(x + (size_t)(t0 + lr) * D + k0 + lc);
        if (e0 + lr < E) wv = *reinterpret_cast<const float4 *>(wr + (size_t)(e0 + lr) * D + k0 + lc);
        __syncthreads();
        xs[lc + 0][lr] = xv.x; xs[lc + 1][lr] = xv.y; xs[lc + 2][lr] = xv.z; xs[lc + 3][lr] = xv.w;
        ws[lc + 0][lr] = wv.x; ws[lc + 1][lr] = wv.y; ws[lc + 2][lr] = wv.z; ws[lc + 3][lr] = wv.w;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 a = *reinterpret_cast<const float4 *>(&xs[k][tm]);
            const float4 b = *reinterpret_cast<const float4 *>(&ws[k][tn]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (t0 + tm + i < T && e0 + tn + j < E) out[(size_t)(t0 + tm + i) * E + e0 + tn + j] = acc[i][j];
}

// part != nullptr: the logits are the sum of `ksplit` partial matrices part[z][T, E], added in the order z = 0, 1, ...
__global__ void __launch_bounds__(128) router_select_kernel(float *logits, const float *part, int ksplit,
                                                            const float *bias, int32_t *ids, float *weights, int T,
                                                            RouterSpec sp) {
    extern __shared__ float rsel[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float *row = logits + (size_t)t * sp.E;
    if (part) {
        for (int e = lane; e < sp.E; e += 32) {
            float v = part[(size_t)t * sp.E + e];
            for (int z = 1; z < ksplit; ++z) v = __fadd_rn(v, part[((size_t)z * T + t) * sp.E + e]);
            row[e] = v;
        }
        __syncwarp();
    }
    float *prob_s = rsel + (size_t)warp * 2 * sp.E;
    route_token_warp(sp, row, row, bias, ids + (size_t)t * sp.K, weights + (size_t)t * sp.K, prob_s, prob_s + sp.E, lane);
}

int launch_router_prefill(const RouterArgs &a, cudaStream_t st) {
    if (a.D % 16 || (size_t)8 * a.E * sizeof(float) > 48 * 1024) return ZMOE_ERR_SHAPE;
    // split k while the tiles alone leave most of the machine idle (a 64 x 64 tile per CTA, 8 warps)
    const int tiles = ((a.E + 63) / 64) * ((a.T + 63) / 64);
    int ksplit = 1;
    if (a.logits_part && a.n_sm > 0)
        while (ksplit < ROUTER_MAX_SPLIT && tiles * ksplit < 3 * a.n_sm && a.D % (32 * ksplit) == 0) ksplit *= 2;
    float *dst = ksplit > 1 ? a.logits_part : a.logits;
    int rc = launch_pdl(router_logits_gemm_kernel, dim3((a.E + 63) / 64, (a.T + 63) / 64, ksplit), dim3(256), 0, st, a.x,
                        a.wr, dst, a.T, a.D, a.E, ksplit) == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
    RouterSpec sp{a.E, a.K, a.gating, a.normalize, a.weight_scale, a.n_groups, a.n_groups_used};
    if (!rc)
        rc = launch_pdl(router_select_kernel, dim3((a.T + 3) / 4), dim3(128), (size_t)8 * a.E * sizeof(float), st,
                        a.logits, (const float *)(ksplit > 1 ? a.logits_part : nullptr), ksplit, a.bias, a.ids, a.weights,
                        a.T, sp) == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
    if (!rc && a.want_q8x) rc = launch_quantize_rows(a.x, a.D, a.q8x, a.T, a.D, a.q8_layout, st);
    if (!rc) rc = launch_plan_from_ids(a.ids, a.T * a.K, a.E, a.plan, a.nrt_gu, a.nrt_dn, st);
    return rc;
}

// ------------------------------------------------------------------------
// stand-alone planners
// ------------------------------------------------------------------------
// Routes that come from outside (src_ids / src_w, optional) are first copied into the context's own
// tables, expert numbers outside the window [first, first + E) becoming -1 (negative ones stay as they are).
struct RouteIngest {
    const int32_t *src_ids = nullptr;
    const float *src_w = nullptr;
    int32_t *dst_ids = nullptr;
    float *dst_w = nullptr;
    int first = 0;
    int window = 0;      // 0: ids are copied unchanged
    int topk = 0;        // > 0: the source rows are ids_ld / w_ld elements apart (a view of a wider table)
    int ids_ld = 0, w_ld = 0;
};

__global__ void __launch_bounds__(1024) plan_from_ids_kernel(const int32_t *ids, int P, int E, PlanOut po, RouteIngest in) {
    extern __shared__ int plan_s[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    if (in.src_ids) {
        for (int p = threadIdx.x; p < P; p += blockDim.x) {
            const int t = in.topk > 0 ? p / in.topk : 0, k = in.topk > 0 ? p - t * in.topk : p;
            const int e = in.src_ids[(size_t)t * in.ids_ld + k];
            in.dst_ids[p] = !in.window ? e : (e >= in.first && e < in.first + E) ? e - in.first : -1;
            in.dst_w[p] = in.src_w[(size_t)t * in.w_ld + k];
        }
        __syncthreads();
    }
    build_plan_cta(ids, P, E, po, plan_s, plan_s + E + 1, P <= ROUTER_IDS_SMEM ? plan_s + 2 * (E + 1) : nullptr);
}

static int launch_plan(const int32_t *ids, int P, int E, const PlanBuffers &plan, int nrt_gu, int nrt_dn,
                       const RouteIngest &in, cudaStream_t st) {
    PlanOut po{plan.hdr, plan.active, plan.offs, plan.slot, plan.item_offs_gu, plan.item_offs_dn, plan.freq,
               plan.aoffs, plan.antok, nrt_gu, nrt_dn, plan.pos, plan.mt_gu, plan.mt_dn};
    const size_t smem = (size_t)2 * (E + 1) * sizeof(int) + (P <= ROUTER_IDS_SMEM ? (size_t)P * sizeof(int) : 0);
    if (smem > 48 * 1024) return ZMOE_ERR_SHAPE;
    return launch_pdl(plan_from_ids_kernel, dim3(1), dim3(1024), smem, st, ids, P, E, po, in) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

int launch_plan_from_ids(const int32_t *ids, int P, int E, const PlanBuffers &plan, int nrt_gu, int nrt_dn,
                         cudaStream_t st) {
    return launch_plan(ids, P, E, plan, nrt_gu, nrt_dn, RouteIngest(), st);
}

int launch_plan_ingest(const int32_t *src_ids, const float *src_w, int32_t *ids, float *w, int P, int E, int first,
                       bool window, const PlanBuffers &plan, int nrt_gu, int nrt_dn, cudaStream_t st, int topk, int ids_ld,
                       int w_ld) {
    RouteIngest in;
    in.src_ids = src_ids; in.src_w = src_w; in.dst_ids = ids; in.dst_w = w; in.first = first; in.window = window ? 1 : 0;
    in.topk = topk; in.ids_ld = ids_ld; in.w_ld = w_ld;
    return launch_plan(ids, P, E, plan, nrt_gu, nrt_dn, in, st);
}

// dense matmul as a one-expert plan: every row of x is a pair of expert 0
__global__ void plan_dense_kernel(int S, PlanOut po) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S; i += gridDim.x * blockDim.x) po.slot[i] = i;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        const int items = ((S + po.mt_gu - 1) / po.mt_gu) * po.nrt_gu;
        po.active[0] = 0;
        po.aoffs[0] = 0; po.antok[0] = S;
        po.offs[0] = 0; po.offs[1] = S;
        po.item_offs_gu[0] = 0; po.item_offs_gu[1] = items;
        po.item_offs_dn[0] = 0; po.item_offs_dn[1] = items;
        po.hdr[0] = 1; po.hdr[1] = items; po.hdr[2] = items; po.hdr[3] = S;
    }
}

int launch_plan_dense(int S, const PlanBuffers &plan, int nrt, cudaStream_t st) {
    PlanOut po{plan.hdr, plan.active, plan.offs, plan.slot, plan.item_offs_gu, plan.item_offs_dn, nullptr,
               plan.aoffs, plan.antok, nrt, nrt, nullptr, plan.mt_gu, plan.mt_dn};
    const int grid = (S + 255) / 256 < 64 ? (S + 255) / 256 : 64;
    return launch_pdl(plan_dense_kernel, dim3(grid > 0 ? grid : 1), dim3(256), 0, st, S, po) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------
// Q8_K row quantiser (one warp per super-block) and the test-side repack to
// ggml's 292-byte blocks
// ------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float *x, int ldx, uint8_t *q8, int rows, int I,
                                                            int layout) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int nb = I / QK_K, stride = q8row_stride(I);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int idx = blockIdx.x * 8 + warp; idx < rows * nb; idx += gridDim.x * 8) {
        const int r = idx / nb, b = idx % nb;
        quantize_block_q8k(x + (size_t)r * ldx + QK_K * b, q8 + (size_t)r * stride, I, b, lane, layout);
    }
}

int launch_quantize_rows(const float *x, int ldx, uint8_t *q8, int rows, int I, int layout, cudaStream_t st) {
    if (rows <= 0) return ZMOE_OK;
    const long blocks = (long)rows * (I / QK_K);
    long grid = (blocks + 7) / 8;
    const long cap = 8L * device_sm_count();
    if (grid > cap) grid = cap;
    return launch_pdl(quantize_rows_kernel, dim3((unsigned)grid), dim3(256), 0, st, x, ldx, q8, rows, I, layout) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

__global__ void q8rows_to_blocks_kernel(const uint8_t *q8, uint8_t *blocks, int rows, int I, int layout) {
    const int nb = I / QK_K, stride = q8row_stride(I);
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nb) return;
    const int r = idx / nb, b = idx % nb;
    const uint8_t *row = q8 + (size_t)r * stride;
    uint8_t *o = blocks + (size_t)idx * 292;
    for (int i = 0; i < 4; ++i) o[i] = row[q8_d_off(b) + i];
    for (int i = 0; i < 256; ++i) o[4 + i] = row[q8row_elem_off(layout, b, i)];
    for (int i = 0; i < 32; ++i) o[260 + i] = row[q8_bs_off(b) + i];
}

int launch_q8rows_to_blocks(const uint8_t *q8, uint8_t *blocks, int rows, int I, int layout, cudaStream_t st) {
    const int n = rows * (I / QK_K);
    if (n <= 0) return ZMOE_OK;
    q8rows_to_blocks_kernel<<<(n + 127) / 128, 128, 0, st>>>(q8, blocks, rows, I, layout);
    return cudaPeekAtLastError() == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------
// weighted combine in k order (reference models/graph/moe_routed_ggml.hpp:198-215):
//   out[t,:] = ((w0*y0 + w1*y1) + w2*y2) + ...
// products and sums are separately rounded, as a MUL node followed by ADD nodes.
// Pairs with a negative id contribute a zero row, ids >= E a NaN row
// (reference kernels/quant/kquant_matmul.cu:659-662).
// ------------------------------------------------------------------------
// KMAX: routes per token whose rows are fetched before any is added (one trip to L2 instead of K in a
// row); 0: any K, row by row.
template <int KMAX>
__global__ void __launch_bounds__(256) combine_kernel(float *out, const float *y, const float *w, const int32_t *ids,
                                                      int T, int K, int D, int E, int accumulate) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int D4 = D / 4;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)T * D4; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / D4), d4 = (int)(i % D4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        auto row = [&](int k) -> float4 {
            const int id = ids[t * K + k];
            if (id < 0) return make_float4(0.f, 0.f, 0.f, 0.f);
            if (id >= E) return make_float4(nanf(""), nanf(""), nanf(""), nanf(""));
            return reinterpret_cast<const float4 *>(y + ((size_t)t * K + k) * D)[d4];
        };
        auto add = [&](int k, float4 v, float wk) {
            const float4 pr = make_float4(__fmul_rn(wk, v.x), __fmul_rn(wk, v.y), __fmul_rn(wk, v.z), __fmul_rn(wk, v.w));
            if (k == 0) acc = pr;
            else acc = make_float4(__fadd_rn(acc.x, pr.x), __fadd_rn(acc.y, pr.y), __fadd_rn(acc.z, pr.z), __fadd_rn(acc.w, pr.w));
        };
        if (KMAX > 0) {
            float4 v[KMAX > 0 ? KMAX : 1];
            float wk[KMAX > 0 ? KMAX : 1];
#pragma unroll
            for (int k = 0; k < KMAX; ++k)
                if (k < K) { v[k] = row(k); wk[k] = w[t * K + k]; }
#pragma unroll
            for (int k = 0; k < KMAX; ++k)
                if (k < K) add(k, v[k], wk[k]);
        } else {
            for (int k = 0; k < K; ++k) add(k, row(k), w[t * K + k]);
        }
        float4 *o = reinterpret_cast<float4 *>(out + (size_t)t * D) + d4;
        if (accumulate) {
            const float4 c = *o;
            acc = make_float4(__fadd_rn(c.x, acc.x), __fadd_rn(c.y, acc.y), __fadd_rn(c.z, acc.z), __fadd_rn(c.w, acc.w));
        }
        *o = acc;
    }
}

int launch_combine(float *out, const float *y, const float *w, const int32_t *ids, int T, int K, int D, int E,
                   int accumulate, cudaStream_t st) {
    const long n = (long)T * (D / 4);
    // one float4 per thread where that still fills the machine: a short batch is bound by the trip to L2
    long grid = (n + 255) / 256;
    int threads = 256;
    const int n_sm = device_sm_count();
    if (grid < n_sm) { threads = 64; grid = (n + 63) / 64; }
    if (grid > 8L * n_sm) grid = 8L * n_sm;
    auto fn = K <= 8 ? combine_kernel<8> : K <= 16 ? combine_kernel<16> : combine_kernel<0>;
    return launch_pdl(fn, dim3((unsigned)grid), dim3(threads), 0, st, out, y, w, ids, T, K, D, E, accumulate) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------
// test hook: per-super-block integer sums through the same unit functions the
// production kernels use.  grid = rows, 128 threads; weight row r against
// activation row r.
// ------------------------------------------------------------------------
template <int TYPE>
__global__ void __launch_bounds__(128) block_isums_kernel(const uint8_t *w, const uint8_t *q8, int32_t *isum,
                                                          int32_t *msum, int I) {
    extern __shared__ __align__(16) uint8_t sm[];
    __shared__ __align__(8) uint64_t g_s[TYPE == IQ2_XXS ? 256 : 1], s_s[TYPE == IQ2_XXS ? 128 : 1];
    constexpr int BB = QTraits<TYPE>::kBytes;
    const int nb = I / QK_K, rb = nb * BB, qstride = q8row_stride(I);
    const int r = blockIdx.x;
    const uint8_t *wrow = w + (size_t)r * rb;
    const int mis = (int)((size_t)wrow & 15);  // keep the global alignment of the row
    uint8_t *wdst = sm + mis;
    uint8_t *qdst = sm + ((rb + 15 + 32) & ~15);
    int *acc = reinterpret_cast<int *>(qdst + qstride);
    for (int i = threadIdx.x; i < rb; i += blockDim.x) wdst[i] = wrow[i];
    for (int i = threadIdx.x; i < qstride; i += blockDim.x) qdst[i] = q8[(size_t)r * qstride + i];
    for (int i = threadIdx.x; i < 2 * nb; i += blockDim.x) acc[i] = 0;
    if (TYPE == IQ2_XXS) iq2_fill_tables(g_s, s_s);
    __syncthreads();
    Iq2Tables tb{smem_u32(g_s), smem_u32(s_s)};
    for (int u = threadIdx.x; u < 4 * nb; u += blockDim.x) {
        UnitAct a;
        load_unit_act<TYPE>(smem_u32(qdst), I, u, a);
        int is, ms;
        float d, dm;
        unit_dot<TYPE>(smem_u32(wdst) + (u >> 2) * BB, u & 3, a, tb, is, ms, d, dm);
        atomicAdd(&acc[u >> 2], is);
        atomicAdd(&acc[nb + (u >> 2)], ms);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        isum[(size_t)r * nb + b] = acc[b];
        msum[(size_t)r * nb + b] = acc[nb + b];
    }
}

// ------------------------------------------------------------------------
// scalar gate of a shared expert: sigmoid(W_gi . x) per token (reference
// models/graph/ggml_moe_graph_builder.cpp:120-124), one warp per token
// ------------------------------------------------------------------------
__global__ void __launch_bounds__(128) token_gate_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                         float *__restrict__ g, int T, int D) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)t * D), *wr = reinterpret_cast<const float4 *>(w);
    float s = 0.f;
    for (int i = lane; i < D / 4; i += 32) {
        const float4 a = xr[i], b = __ldg(wr + i);
        s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) g[t] = 1.0f / (1.0f + expf(-s));
}

int launch_token_gate(const float *x, const float *w, float *g, int T, int D, cudaStream_t st) {
    if (D % 4 || (reinterpret_cast<size_t>(x) & 15) || (reinterpret_cast<size_t>(w) & 15)) return ZMOE_ERR_ALIGN;
    return launch_pdl(token_gate_kernel, dim3((T + 3) / 4), dim3(128), 0, st, x, w, g, T, D) == cudaSuccess ? ZMOE_OK
                                                                                                            : ZMOE_ERR_CUDA;
}

// bf16 -> f32, eight values per thread per step (the widening is exact)
__global__ void __launch_bounds__(256) widen_bf16_kernel(const uint4 *__restrict__ src, float4 *__restrict__ dst, long n8) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        float4 a, b;
        a.x = __uint_as_float(v.x << 16); a.y = __uint_as_float(v.x & 0xffff0000u);
        a.z = __uint_as_float(v.y << 16); a.w = __uint_as_float(v.y & 0xffff0000u);
        b.x = __uint_as_float(v.z << 16); b.y = __uint_as_float(v.z & 0xffff0000u);
        b.z = __uint_as_float(v.w << 16); b.w = __uint_as_float(v.w & 0xffff0000u);
        dst[2 * i] = a;
        dst[2 * i + 1] = b;
    }
}

int launch_widen_bf16(const void *src, float *dst, long n, int n_sm, cudaStream_t st) {
    if (n % 8 || (reinterpret_cast<size_t>(src) & 15) || (reinterpret_cast<size_t>(dst) & 15)) return ZMOE_ERR_ALIGN;
    const long n8 = n / 8;
    long grid = (n8 + 255) / 256;
    if (grid > 8L * n_sm) grid = 8L * n_sm;
    return launch_pdl(widen_bf16_kernel, dim3((unsigned)(grid > 0 ? grid : 1)), dim3(256), 0, st, static_cast<const uint4 *>(src),
                      reinterpret_cast<float4 *>(dst), n8) == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

int launch_block_isums(int type, const void *w, const uint8_t *q8, int32_t *isum, int32_t *msum, int rows, int I,
                       cudaStream_t st) {
    if (rows <= 0) return ZMOE_OK;
    const int nb = I / QK_K, rb = nb * block_bytes(type);
    const size_t smem = (size_t)((rb + 15 + 32) & ~15) + q8row_stride(I) + (size_t)2 * nb * sizeof(int) + 16;
    if (smem > 48 * 1024) return ZMOE_ERR_SHAPE;
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    switch (type) {
    case Q2_K: block_isums_kernel<Q2_K><<<rows, 128, smem, st>>>(wb, q8, isum, msum, I); break;
    case Q3_K: block_isums_kernel<Q3_K><<<rows, 128, smem, st>>>(wb, q8, isum, msum, I); break;
    case Q4_K: block_isums_kernel<Q4_K><<<rows, 128, smem, st>>>(wb, q8, isum, msum, I); break;
    case IQ2_XXS: block_isums_kernel<IQ2_XXS><<<rows, 128, smem, st>>>(wb, q8, isum, msum, I); break;
    default: return ZMOE_ERR_TYPE;
    }
    return cudaPeekAtLastError() == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

}  // namespace zmoe

// ------------------------------------------------------------------------
// reference kernel-launch ABI: element-wise and router entry points
// ------------------------------------------------------------------------
namespace {

// prod = SwiGLU(gate, up) over n elements, four per thread per step, grid-stride.  Same values as
// reference kernels/math/expert_activation.cu:46-58 (expf, the two clamp forms).  Non-finite inputs are
// counted like the reference does (bad[0]: an input is NaN, bad[1]: none is NaN and one is infinite),
// but a warp adds its counts with one atomic per counter instead of one per element.
__global__ void __launch_bounds__(256) swiglu_rows_kernel(float *__restrict__ prod, const float *__restrict__ gate,
                                                          const float *__restrict__ up, int n, float clamp, int fused,
                                                          int *__restrict__ bad, int vec_ok) {
    const int lane = threadIdx.x & 31;
    int n_nan = 0, n_inf = 0;
    auto one = [&](float g, float u) -> float {
        if (bad) {
            const bool isn = (g != g) || (u != u);
            n_nan += isn;
            n_inf += !isn && (isinf(g) || isinf(u));
        }
        return zmoe::swiglu_f(g, u, clamp, fused);
    };
    const long stride = (long)gridDim.x * blockDim.x;
    const long first = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int n4 = vec_ok ? n / 4 : 0;
    for (long i = first; i < n4; i += stride) {
        const float4 g = reinterpret_cast<const float4 *>(gate)[i], u = reinterpret_cast<const float4 *>(up)[i];
        float4 o;
        o.x = one(g.x, u.x); o.y = one(g.y, u.y); o.z = one(g.z, u.z); o.w = one(g.w, u.w);
        reinterpret_cast<float4 *>(prod)[i] = o;
    }
    for (long i = 4L * n4 + first; i < n; i += stride) prod[i] = one(gate[i], up[i]);
    if (bad) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            n_nan += __shfl_xor_sync(0xffffffffu, n_nan, off);
            n_inf += __shfl_xor_sync(0xffffffffu, n_inf, off);
        }
        if (lane == 0) {
            if (n_nan) atomicAdd(&bad[0], n_nan);
            if (n_inf) atomicAdd(&bad[1], n_inf);
        }
    }
}

// dst[tok[i], :] += w[i] * src[i, :] for the n rows of one call (w == nullptr: plain add).  Contract of
// reference kernels/math/expert_accum.cu:22-37: rows of one call name distinct tokens, calls are ordered
// by the stream, a token outside [0, S) is skipped, no atomics.  A warp walks a row four floats per lane;
// the grid covers rows x row chunks so that a short call still fills the machine.
__global__ void __launch_bounds__(256) scatter_rows_kernel(const float *__restrict__ src, const int *__restrict__ tok,
                                                           const float *__restrict__ w, float *__restrict__ dst, int n,
                                                           int D, int S, int chunks, int vec_ok) {
    const int row = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    if (row >= n) return;
    const int s = tok[row];
    if (s < 0 || s >= S) return;
    const float wt = w ? w[row] : 1.0f;
    const float *sr = src + (size_t)row * D;
    float *ds = dst + (size_t)s * D;
    const int per = (D + chunks - 1) / chunks;
    const int d0 = chunk * per, d1 = min(D, d0 + per);
    if (vec_ok && (per & 3) == 0) {
        for (int d = d0 + 4 * threadIdx.x; d + 3 < d1; d += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4 *>(sr + d);
            float4 o = *reinterpret_cast<float4 *>(ds + d);
            o.x = fmaf(wt, v.x, o.x); o.y = fmaf(wt, v.y, o.y); o.z = fmaf(wt, v.z, o.z); o.w = fmaf(wt, v.w, o.w);
            *reinterpret_cast<float4 *>(ds + d) = o;
        }
        const int tail = d0 + ((d1 - d0) & ~3);
        for (int d = tail + threadIdx.x; d < d1; d += blockDim.x) ds[d] = fmaf(wt, sr[d], ds[d]);
    } else {
        for (int d = d0 + threadIdx.x; d < d1; d += blockDim.x) ds[d] = fmaf(wt, sr[d], ds[d]);
    }
}

void scatter_rows(const float *src, const int *tok, const float *w, float *dst, int n, int D, int S, cudaStream_t st) {
    if (n <= 0 || D <= 0) return;
    const int n_sm = zmoe::device_sm_count();
    int chunks = 1;
    while (n * chunks < 2 * n_sm && D / (chunks * 2) >= 256) chunks *= 2;
    const int vec_ok = (D % 4 == 0) && ((reinterpret_cast<size_t>(src) | reinterpret_cast<size_t>(dst)) % 16 == 0);
    const int threads = D / chunks >= 1024 ? 256 : 64;
    scatter_rows_kernel<<<n * chunks, threads, 0, st>>>(src, tok, w, dst, n, D, S, chunks, vec_ok);
}

// reference kernels/models/glm5next_router.cu:33-93, one warp per token
__global__ void __launch_bounds__(128) router_topk_kernel(float *logits, const float *bias, int32_t *ids,
                                                          float *weights, int S, zmoe::RouterSpec sp) {
    extern __shared__ float rs[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= S) return;
    float *prob_s = rs + (size_t)warp * 2 * sp.E;
    zmoe::route_token_warp(sp, logits + (size_t)t * sp.E, logits + (size_t)t * sp.E, bias, ids + (size_t)t * sp.K,
                           weights + (size_t)t * sp.K, prob_s, prob_s + sp.E, lane);
}

}  // namespace

extern "C" {

void launch_expert_swiglu(float *prod, const float *gate, const float *up, int n, float clamp, int fused, int *d_bad,
                          void *stream) {
    if (n <= 0) return;
    const int n_sm = zmoe::device_sm_count();
    long grid = ((long)n / 4 + 255) / 256;
    if (grid < 1) grid = 1;
    if (grid > 8L * n_sm) grid = 8L * n_sm;
    const int vec_ok =
        ((reinterpret_cast<size_t>(prod) | reinterpret_cast<size_t>(gate) | reinterpret_cast<size_t>(up)) % 16) == 0;
    swiglu_rows_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(prod, gate, up, n, clamp, fused,
                                                                                     d_bad, vec_ok);
    zmoe::count_launches(1);
}

void launch_expert_scatter_accum(const float *src, const int *tok, const float *w, float *dst, int n, int D, int S,
                                 void *stream) {
    scatter_rows(src, tok, w, dst, n, D, S, static_cast<cudaStream_t>(stream));
    zmoe::count_launches(1);
}

void launch_expert_scatter_add(const float *src, const int *tok, float *dst, int n, int D, int S,
                               void *stream) {
    scatter_rows(src, tok, nullptr, dst, n, D, S, static_cast<cudaStream_t>(stream));
    zmoe::count_launches(1);
}

void launch_glm5next_router_topk(float *logits, const float *bias, int32_t *ids, float *weights, int S, int n_experts,
                                 int topk, int gating_func, int normalize, float weight_scale, void *stream) {
    if (!logits || !ids || !weights || S <= 0 || n_experts <= 0 || topk <= 0 || topk > n_experts) {
        zmoe::set_last_status(ZMOE_ERR_ARG);
        return;
    }
    zmoe::RouterSpec sp{n_experts, topk, gating_func, normalize, weight_scale, 0, 0};
    const size_t smem = (size_t)8 * n_experts * sizeof(float);
    if (smem > 200 * 1024) {
        zmoe::set_last_status(ZMOE_ERR_SHAPE);
        return;
    }
    if (smem > 48 * 1024 &&
        zmoe::raise_dynamic_smem(reinterpret_cast<const void *>(router_topk_kernel), smem) != ZMOE_OK) {
        zmoe::set_last_status(ZMOE_ERR_CUDA);
        return;
    }
    router_topk_kernel<<<(S + 3) / 4, 128, smem, static_cast<cudaStream_t>(stream)>>>(logits, bias, ids, weights, S, sp);
    zmoe::count_launches(1);
    zmoe::set_last_status(cudaPeekAtLastError() == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA);
}

}  // extern "C"
