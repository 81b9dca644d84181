// router.cuh -- router top-k, token-to-expert grouping and the device-side
// work plan.
//
// Follows reference core/moe_router.cpp:6-37 (gating), core/moe_router_service.cpp:1409-1474
// (selection bias, group-limited routing, top-k, unbiased weight gather,
// normalise with the 6.103515625e-5 clamp, scale) and
// kernels/models/glm5next_router.cu:60-92 (lowest index wins ties).
// Grouping follows reference core/batched_dispatch_pipeline.cpp:1185-1204
// (offs[e+1] = offs[e] + freq[e]; slot[] holds pair indices t*K+k in
// token-major order inside each expert).
#pragma once

#include <math_constants.h>

#include "mmid.cuh"

namespace zmoe {

struct RouterSpec {
    int E, K;
    int gating;        // 0 softmax, 1 sigmoid, 2 sqrt(softplus)
    int normalize;
    float weight_scale;
    int n_groups, n_groups_used;
};

struct PlanOut {
    int *hdr;          // [4]
    int *active;       // [E]
    int *offs;         // [E+1]
    int *slot;         // [P]
    int *item_offs_gu; // [E+1]
    int *item_offs_dn; // [E+1]
    int *freq;         // [E] expert histogram (reference scratch.expert_freq), may be null
    int *aoffs;        // [E] offs[active[a]]
    int *antok;        // [E] pairs of active[a]
    int nrt_gu, nrt_dn;  // row tiles per expert of the two projections
    int *pos = nullptr;  // [P] inverse of slot: position of pair p in expert order, -1 for an inactive route; may be null
    int mt_gu = 4, mt_dn = 4;  // pairs per item of the two projections
};

__device__ __forceinline__ float gate_scalar(float x, int gating) {
    if (gating == 1) return 1.0f / (1.0f + expf(-x));
    const float sp = x > 0.0f ? x + log1pf(expf(-x)) : log1pf(expf(x));
    return sqrtf(sp);
}

// (value, index) arg-max over a warp; ties go to the lower index
__device__ __forceinline__ void warp_argmax(float &v, int &i) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, i, off);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// One warp routes one token.  row: logits in (global), probs out (global, may
// alias row).  prob_s / sel_s: per-warp shared scratch of E floats each.
__device__ void route_token_warp(const RouterSpec &sp, const float *row_in, float *probs_out, const float *bias,
                                 int32_t *ids, float *weights, float *prob_s, float *sel_s, int lane) {
    const int E = sp.E, K = sp.K;
    if (sp.gating == 0) {
        float mx = -CUDART_INF_F;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row_in[e]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        for (int e = lane; e < E; e += 32) prob_s[e] = expf(row_in[e] - mx);
        __syncwarp();
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += prob_s[e];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) prob_s[e] *= inv;
    } else {
        for (int e = lane; e < E; e += 32) prob_s[e] = gate_scalar(row_in[e], sp.gating);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        const float pr = prob_s[e];
        if (probs_out) probs_out[e] = pr;
        sel_s[e] = pr + (bias ? bias[e] : 0.f);
    }
    __syncwarp();
    // group-limited routing: keep the n_groups_used groups with the largest top-2 sum
    if (sp.n_groups > 1 && sp.n_groups_used > 0 && sp.n_groups_used < sp.n_groups && E % sp.n_groups == 0 &&
        sp.n_groups <= 32) {
        const int G = sp.n_groups, gs = E / G;
        float score = -CUDART_INF_F;
        if (lane < G) {
            float first = -CUDART_INF_F, second = -CUDART_INF_F;
            for (int j = 0; j < gs; ++j) {
                const float s = sel_s[lane * gs + j];
                if (s > first) { second = first; first = s; }
                else if (s > second) second = s;
            }
            score = first + second;
        }
        unsigned keep = 0;
        bool taken = lane >= G;
        for (int u = 0; u < sp.n_groups_used; ++u) {
            // untaken groups compete, -inf scores included; ties go to the lower group
            float bv = taken ? -CUDART_INF_F : score;
            int bi = taken ? 0x7fffffff : lane;
            warp_argmax(bv, bi);
            if (bi == 0x7fffffff) break;
            keep |= 1u << bi;
            if (lane == bi) taken = true;
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32)
            if (!((keep >> (e / gs)) & 1u)) sel_s[e] = -CUDART_INF_F;
        __syncwarp();
    }
    float sum_w = 0.f;
    // lane k keeps the weight of route k: the normalisation below then needs no trip back to the
    // memory the weights were just stored to (K <= 32; more routes take the in-place path)
    float mine = 0.f;
    const bool in_regs = K <= 32;
    for (int k = 0; k < K; ++k) {
        float bv = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float s = sel_s[e];
            // taken entries are NaN; the first untaken entry is a candidate even at -inf
            if (!isnan(s) && (bi == 0x7fffffff || s > bv)) { bv = s; bi = e; }
        }
        warp_argmax(bv, bi);
        if (bi == 0x7fffffff) bi = 0;
        const float w = prob_s[bi];
        if (lane == 0) {
            ids[k] = bi;
            if (!in_regs) weights[k] = w;
            sel_s[bi] = CUDART_NAN_F;  // taken
        }
        if (lane == k) mine = w;
        sum_w += w;
        __syncwarp();
    }
    if (in_regs) {
        if (sp.normalize) mine *= 1.0f / fmaxf(sum_w, 6.103515625e-5f);
        if (sp.weight_scale != 0.0f) mine *= sp.weight_scale;
        if (lane < K) weights[lane] = mine;
    } else if (lane == 0) {
        if (sp.normalize) {
            const float inv = 1.0f / fmaxf(sum_w, 6.103515625e-5f);
            for (int k = 0; k < K; ++k) weights[k] *= inv;
        }
        if (sp.weight_scale != 0.0f)
            for (int k = 0; k < K; ++k) weights[k] *= sp.weight_scale;
    }
}

// CSR of pairs by expert plus the item spaces of the projections.  Called by
// all threads of ONE CTA; cnt_s/pre_s: shared scratch of E+1 ints each; ids_s:
// optional shared scratch of P ints (a copy of ids that the stable fill scans).
// ids: [T*K] (entries outside [0,E) are skipped: negative = inactive route,
// reference backends/ggml/mmid_route_skip.hpp:60-67).
__device__ void build_plan_cta(const int32_t *ids, int P, int E, const PlanOut &po, int *cnt_s, int *pre_s,
                               int *ids_s) {
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
    for (int e = tid; e <= E; e += nt) cnt_s[e] = 0;
    __syncthreads();
    for (int p = tid; p < P; p += nt) {
        const int e = ids[p];
        if (ids_s) ids_s[p] = e;
        if (e >= 0 && e < E) atomicAdd(&cnt_s[e], 1);
    }
    __syncthreads();
    if (tid < 32) {
        // warp scan over contiguous chunks of experts: pairs, active experts, items
        const int per = (E + 31) / 32, e0 = min(E, lane * per), e1 = min(E, e0 + per);
        int cs = 0, as = 0, gs = 0, ds = 0;
        for (int e = e0; e < e1; ++e) {
            const int c = cnt_s[e];
            cs += c;
            if (c > 0) {
                ++as;
                gs += ((c + po.mt_gu - 1) / po.mt_gu) * po.nrt_gu;
                ds += ((c + po.mt_dn - 1) / po.mt_dn) * po.nrt_dn;
            }
        }
        int xs[4] = {cs, as, gs, ds}, tot[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int v = xs[q];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, v, off);
                if (lane >= off) v += o;
            }
            tot[q] = __shfl_sync(0xffffffffu, v, 31);
            xs[q] = v - xs[q];  // exclusive
        }
        int run = xs[0], na = xs[1], igu = xs[2], idn = xs[3];
        for (int e = e0; e < e1; ++e) {
            const int c = cnt_s[e];
            pre_s[e] = run;
            po.offs[e] = run;
            if (po.freq) po.freq[e] = c;
            if (c > 0) {
                po.active[na] = e;
                po.aoffs[na] = run;
                po.antok[na] = c;
                igu += ((c + po.mt_gu - 1) / po.mt_gu) * po.nrt_gu;
                idn += ((c + po.mt_dn - 1) / po.mt_dn) * po.nrt_dn;
                ++na;
                po.item_offs_gu[na] = igu;
                po.item_offs_dn[na] = idn;
            }
            run += c;
        }
        if (lane == 0) {
            po.item_offs_gu[0] = 0;
            po.item_offs_dn[0] = 0;
            po.offs[E] = tot[0];
            po.hdr[0] = tot[1]; po.hdr[1] = tot[2]; po.hdr[2] = tot[3]; po.hdr[3] = tot[0];
        }
    }
    __syncthreads();
    if (P <= 8192) {
        // Stable fill by one warp, 32 pairs at a time: lanes that name the same expert find each other
        // (match), the first of them takes the expert's cursor and moves it on, each writes its pair at
        // cursor + its rank among them.  (A thread per expert walking all pairs costs P dependent steps:
        // 44 us at 1024 pairs.)
        const int *src = ids_s ? ids_s : ids;
        if (tid < 32) {
            for (int p0 = 0; p0 < P; p0 += 32) {
                const int p = p0 + lane;
                const int e = p < P ? src[p] : -1;
                const bool on = e >= 0 && e < E;
                const unsigned peers = __match_any_sync(0xffffffffu, on ? e : -1 - lane);
                const int leader = __ffs(peers) - 1;
                int base = 0;
                if (on && lane == leader) {
                    base = pre_s[e];
                    pre_s[e] = base + __popc(peers);
                }
                base = __shfl_sync(0xffffffffu, base, leader);
                const int at = base + __popc(peers & ((1u << lane) - 1u));
                if (on) po.slot[at] = p;
                if (po.pos && p < P) po.pos[p] = on ? at : -1;
                __syncwarp();
            }
        }
    } else {
        for (int p = tid; p < P; p += nt) {
            const int e = ids[p];
            const bool on = e >= 0 && e < E;
            const int at = on ? atomicAdd(&pre_s[e], 1) : -1;
            if (on) po.slot[at] = p;
            if (po.pos) po.pos[p] = at;
        }
    }
}

}  // namespace zmoe
