// mmid.cuh -- the decode-shaped MUL_MAT_ID kernel: quantised expert rows
// against Q8_K activations, one persistent CTA per SM.
//
// Replaces, for decode-shaped calls, the per-(expert, projection) launches of
// reference core/gpu_expert_executor.cpp:358-387,512-513 and the
// native_f32_matmul_id kernel of reference kernels/quant/kquant_matmul.cu:647-700.
//
// Structure (memory-bound, so everything serves keeping HBM requests in flight):
//   * work item = (expert, tile of R consecutive weight rows, chunk of <= MAXTOK
//     pairs routed to that expert).  Rows of one expert are contiguous, so a
//     tile is ONE contiguous byte range.
//   * a producer warp streams items through an NSTAGE ring in shared memory
//     with asynchronous copies on the TMA engine, completion on mbarriers: a
//     1-D bulk copy of the tile, or -- where the launch has a tiled map of the
//     tensor -- one tiled copy whose box is 16 bytes wider than a row, which pads
//     the rows in shared memory (bank-conflict-free fragment loads).  The packed
//     Q8_K rows of the item's pairs ride in the same stage.
//   * consumer warps decode from shared memory.  One pair: a row is split over
//     LPR lanes, each lane owns UPL "units" (64 elements) whose activation words
//     stay in registers across rows; dot products are dp4a, reduced by warp
//     shuffles.  Two to four pairs (MMA instantiations): mmid_mma.cuh.
//   * DUAL mode reads a gate tile and an up tile and writes SwiGLU(gate, up)
//     (reference kernels/math/expert_activation.cu:31-59).
// Every wait is bounded; on expiry the CTA raises an error flag and unwinds.
#pragma once

#include <cuda.h>
#include <math_constants.h>

#include "mmid_mma.cuh"
#include "quant_units.cuh"

namespace zmoe {

constexpr int MMID_MAXTOK = 4;   // pairs per item
constexpr int MMID_MAXSTAGE = 6;

// Routing plan produced on the device (router.cu): CSR of pairs by expert and
// the item index space of the two projections.
struct PlanView {
    const int *hdr;        // [0]=n_active [1]=items_gu [2]=items_dn [3]=n_pairs_valid
    const int *active;     // [n_active] expert ids, ascending
    const int *offs;       // [E+1]
    const int *slot;       // [P] pair index t*K+k grouped by expert
    const int *item_offs;  // [n_active+1] prefix of item counts for THIS projection
    const int *aoffs;      // [n_active] offs[active[a]]
    const int *antok;      // [n_active] pairs of active[a]
    int cap_e;             // capacity of the arrays above
};
constexpr int MMID_PLAN_SMEM = 512;  // active experts whose plan rows are mirrored in shared memory

struct MmidParams {
    const uint8_t *w0, *w1;     // weight tensors (w1: up, DUAL only)
    size_t stride0, stride1;    // bytes between experts
    size_t total0, total1;      // bytes addressable from w0 / w1
    int I, O;                   // elements per row, rows per expert
    int rb;                     // bytes per weight row
    int rbs;                    // bytes between rows of a tile in shared memory (>= rb; > rb: one copy per row)
    int q8s;                    // bytes between the item's activation rows in shared memory (>= q8_stride)
    int R;                      // rows per tile
    const uint8_t *q8;          // packed activation rows
    int q8_stride;              // bytes per packed row
    int xdiv;                   // activation row of pair p is p / xdiv
    float *y;                   // output [pair][ldy]
    int ldy;
    PlanView plan;
    int hdr_items;              // which hdr slot holds this projection's item count
    float clamp;
    int clamp_fused;
    int nstage;
    int stage_bytes;            // bytes per ring stage (multiple of 128)
    int wtile_bytes;            // bytes reserved per weight tile inside a stage (multiple of 128)
    int mma_ks_log2;            // multi-token path: log2 of the warps that share one 16-row piece of one matrix
    int mma_hpw;                // multi-token path: half super-blocks per warp
    int mma_rdiv;               // multi-token path: ceil(65536 / R), for dividing a thread index by R
    int *err;                   // device error flag
    int *bad;                   // DUAL: [2] counters of NaN / Inf gate or up values, or null
    int use_tmap;               // tiles come through tm0 / tm1 (rows padded to rbs = rb + 16 by the copy)
    alignas(64) CUtensorMap tm0, tm1;
};

// 3-D tiled copy (no multicast): box of the map at (0, row, expert)
__device__ __forceinline__ void tma_load_rows(void *dst_smem, const void *tmap, int row, int expert, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst_smem)), "l"(tmap), "r"(0), "r"(row), "r"(expert), "r"(smem_u32(bar))
        : "memory");
}

struct StageMeta {
    int expert, r0, nrows, ntok;
    int w0_off, w1_off;   // byte offset of the first row inside the stage
    int pair[MMID_MAXTOK];
    int xrow[MMID_MAXTOK];  // activation row of each pair
    int pad[2];
};
static_assert(sizeof(StageMeta) == 64, "meta");

__device__ __forceinline__ float swiglu_f(float g, float u, float clamp, int fused) {
    // reference kernels/math/expert_activation.cu:46-58 (expf, not the fast intrinsic)
    float out;
    if (fused) {
        if (clamp > 0.0f) {
            g = fminf(g, clamp);
            u = fmaxf(-clamp, fminf(clamp, u));
        }
        out = g / (1.0f + expf(-g)) * u;
    } else {
        g = g / (1.0f + expf(-g));
        out = g * u;
        if (clamp > 0.0f) out = fmaxf(-clamp, fminf(clamp, out));
    }
    return out;
}

// The same function for the tensor-core path's epilogue, where one warp per scheduler works through a whole
// accumulator tile while the tensor memory is held: the quotient comes from the reciprocal unit
// (__fdividef, at most 2 ulp from the correctly rounded one) so that no slow-path branch breaks up the
// interleaving of the columns' dependency chains.  The path's results are within 3e-4 of the CPU path anyway.
__device__ __forceinline__ float swiglu_fast(float g, float u, float clamp, int fused) {
    float out;
    if (fused) {
        if (clamp > 0.0f) {
            g = fminf(g, clamp);
            u = fmaxf(-clamp, fminf(clamp, u));
        }
        out = __fdividef(g, 1.0f + expf(-g)) * u;
    } else {
        g = __fdividef(g, 1.0f + expf(-g));
        out = g * u;
        if (clamp > 0.0f) out = fmaxf(-clamp, fminf(clamp, out));
    }
    return out;
}

// Non-finite inputs of the fused SwiGLU, counted as reference kernels/math/expert_activation.cu:42-44
// does (bad[0]: one of the two is NaN; bad[1]: none is NaN, one is infinite).  The test is one
// instruction on the common path; the atomics run only when something is wrong.
__device__ __forceinline__ void count_bad(int *bad, float g, float u) {
    if (bad && !(fabsf(g) < CUDART_INF_F && fabsf(u) < CUDART_INF_F)) {
        if (g != g || u != u) atomicAdd(&bad[0], 1);
        else atomicAdd(&bad[1], 1);
    }
}

// issue the copy of one weight tile; returns bytes that will complete on `bar`
__device__ __forceinline__ uint32_t issue_tile(uint8_t *dst, const uint8_t *w, size_t total, size_t g0, size_t g1,
                                               uint64_t *bar, int *off_out) {
    const size_t c0 = g0 & ~(size_t)15;
    size_t c1 = (g1 + 15) & ~(size_t)15;
    const size_t lim = total & ~(size_t)15;
    *off_out = (int)(g0 - c0);
    uint32_t bytes = 0;
    if (c1 > lim) {
        // ragged end of the tensor: the last <16 bytes come by plain loads
        for (size_t i = lim > c0 ? lim : c0; i < g1; ++i) dst[i - c0] = w[i];
        c1 = lim;
    }
    if (c1 > c0) {
        bytes = (uint32_t)(c1 - c0);
        bulk_g2s(dst, w + c0, bytes, bar);
    }
    return bytes;
}

// MMA: items with two or more pairs take the tensor-core path of mmid_mma.cuh; the activation
// registers of the scalar path are then not kept from one item to the next.
template <int TYPE, int LPR, int UPL, bool DUAL, int NCW, bool MMA>
__global__ void __launch_bounds__(32 * (NCW + 1), 1) mmid_kernel(const __grid_constant__ MmidParams p) {
    constexpr int BB = QTraits<TYPE>::kBytes;
    constexpr int RPW = 32 / LPR;  // rows a warp handles at once
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[MMID_MAXSTAGE], empty_bar[MMID_MAXSTAGE];
    __shared__ StageMeta meta[MMID_MAXSTAGE];
    __shared__ __align__(8) uint64_t iq2_grid[TYPE == IQ2_XXS ? 256 : 1], iq2_sign[TYPE == IQ2_XXS ? 128 : 1];

    // multi-token path: per-warp partial sums [buffer][warp][16 rows][MAXTOK pairs], double buffered
    constexpr int PART = 16 * MMID_MAXTOK;   // one matrix of one warp
    __shared__ __align__(16) float part[MMA ? 2 : 1][MMA ? NCW : 1][MMA ? PART : 1];
    __shared__ __align__(8) uint64_t part_bar;
    __shared__ int s_item_offs[MMID_PLAN_SMEM + 1], s_active[MMID_PLAN_SMEM], s_aoffs[MMID_PLAN_SMEM],
        s_antok[MMID_PLAN_SMEM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstage = p.nstage;
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], NCW);
        }
        mbar_init(&part_bar, NCW);
        mbar_init_fence();
    }
    if (TYPE == IQ2_XXS) iq2_fill_tables(iq2_grid, iq2_sign);
    __syncthreads();

    // everything below reads what earlier kernels of the stream wrote
    pdl_wait_prior_grid();
    pdl_launch_dependents();

    // one round trip for the whole plan: header and per-expert rows are fetched together
    const int n_items = p.plan.hdr[p.hdr_items];
    const int n_active = p.plan.hdr[0];
    for (int i = tid; i < MMID_PLAN_SMEM && i < p.plan.cap_e; i += blockDim.x) {
        s_item_offs[i + 1] = p.plan.item_offs[i + 1];
        s_active[i] = p.plan.active[i];
        s_aoffs[i] = p.plan.aoffs[i];
        s_antok[i] = p.plan.antok[i];
    }
    if (tid == 0) s_item_offs[0] = 0;
    __syncthreads();
    const bool plan_in_smem = n_active <= MMID_PLAN_SMEM;
    // items are dealt round-robin: an item's cost grows with the number of pairs of its
    // expert, and a strided deal gives every CTA the same mix of experts
    const int G = (int)gridDim.x;
    const int n_mine = n_items > (int)blockIdx.x ? (n_items - (int)blockIdx.x + G - 1) / G : 0;
    const int U = p.I / 64;  // units per row
    const int nrt = (p.O + p.R - 1) / p.R;

    if (warp == NCW) {
        // ------------------------------ producer ------------------------------
        // Item descriptors are resolved 32 at a time, one per lane, so the dependent
        // global loads of the plan overlap; issuing an item then touches no global
        // memory except the copies themselves.
        bool alive = true;
        for (int batch = 0; batch < n_mine && alive; batch += 32) {
            const int mine = (int)blockIdx.x + (batch + lane) * G;  // global item index
            int e = 0, r0 = 0, nrows = 0, ntok = 0, pr[MMID_MAXTOK];
#pragma unroll
            for (int t = 0; t < MMID_MAXTOK; ++t) pr[t] = 0;
            if (batch + lane < n_mine) {
                int lo = 0, hi = n_active - 1;  // last a with item_offs[a] <= mine
                int local, ebase, ecnt;
                if (plan_in_smem) {
                    while (lo < hi) {
                        const int mid = (lo + hi + 1) >> 1;
                        if (s_item_offs[mid] <= mine) lo = mid; else hi = mid - 1;
                    }
                    e = s_active[lo]; local = mine - s_item_offs[lo]; ebase = s_aoffs[lo]; ecnt = s_antok[lo];
                } else {
                    while (lo < hi) {
                        const int mid = (lo + hi + 1) >> 1;
                        if (p.plan.item_offs[mid] <= mine) lo = mid; else hi = mid - 1;
                    }
                    e = p.plan.active[lo]; local = mine - p.plan.item_offs[lo];
                    ebase = p.plan.aoffs[lo]; ecnt = p.plan.antok[lo];
                }
                const int tc = local / nrt, rt = local % nrt;
                r0 = rt * p.R;
                nrows = min(p.R, p.O - r0);
                const int s0 = ebase + tc * MMID_MAXTOK;
                ntok = min(MMID_MAXTOK, ecnt - tc * MMID_MAXTOK);
#pragma unroll
                for (int t = 0; t < MMID_MAXTOK; ++t)
                    if (t < ntok) pr[t] = p.plan.slot[s0 + t];
            }
            const int nb = min(32, n_mine - batch);
            for (int j = 0; j < nb; ++j) {
                const int k = batch + j, s = k % nstage;
                if (k >= nstage) {
                    if (!mbar_wait(&empty_bar[s], ((k / nstage) - 1) & 1)) {
                        if (lane == 0) atomicExch(p.err, 1);
                        alive = false;
                        break;
                    }
                }
                const int je = __shfl_sync(0xffffffffu, e, j), jr0 = __shfl_sync(0xffffffffu, r0, j);
                const int jnrows = __shfl_sync(0xffffffffu, nrows, j), jntok = __shfl_sync(0xffffffffu, ntok, j);
                int my_pair = 0;
#pragma unroll
                for (int t = 0; t < MMID_MAXTOK; ++t) {
                    const int v = __shfl_sync(0xffffffffu, pr[t], j);
                    if (lane == t) my_pair = v;
                }
                uint8_t *stage = smem + (size_t)s * p.stage_bytes;
                uint8_t *q8dst = stage + (DUAL ? 2 : 1) * p.wtile_bytes;
                uint32_t bytes = 0;
                if (p.use_tmap) {
                    // one tiled copy per tile; the box is always R full padded rows (rows past the
                    // expert's last arrive as zeros)
                    if (lane == 0) {
                        StageMeta &m = meta[s];
                        m.expert = je; m.r0 = jr0; m.nrows = jnrows; m.ntok = jntok;
                        m.w0_off = 0; m.w1_off = 0;
                        tma_load_rows(stage, &p.tm0, jr0, je, &full_bar[s]);
                        if (DUAL) tma_load_rows(stage + p.wtile_bytes, &p.tm1, jr0, je, &full_bar[s]);
                        bytes = (uint32_t)(p.R * p.rbs) * (DUAL ? 2u : 1u);
                    }
                } else if (lane == 0) {
                    StageMeta &m = meta[s];
                    m.expert = je; m.r0 = jr0; m.nrows = jnrows; m.ntok = jntok;
                    const size_t g0 = (size_t)je * p.stride0 + (size_t)jr0 * p.rb;
                    // the producer's own arrival (below, with the byte count) is what lets the
                    // phase complete, so copies issued before it cannot end the phase early
                    bytes += issue_tile(stage, p.w0, p.total0, g0, g0 + (size_t)jnrows * p.rb, &full_bar[s], &m.w0_off);
                    if (DUAL) {
                        const size_t h0 = (size_t)je * p.stride1 + (size_t)jr0 * p.rb;
                        bytes += issue_tile(stage + p.wtile_bytes, p.w1, p.total1, h0, h0 + (size_t)jnrows * p.rb,
                                            &full_bar[s], &m.w1_off);
                    }
                }
                // pairs and their activation rows: one lane per pair
                if (lane < jntok) {
                    const int xr = my_pair / p.xdiv;
                    meta[s].pair[lane] = my_pair;
                    meta[s].xrow[lane] = xr;
                    bulk_g2s(q8dst + (size_t)lane * p.q8s, p.q8 + (size_t)xr * p.q8_stride,
                             (uint32_t)p.q8_stride, &full_bar[s]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], bytes + (uint32_t)(jntok * p.q8_stride));
            }
        }
    } else {
        // ------------------------------ consumers -----------------------------
        Iq2Tables tb;
        tb.grid = smem_u32(iq2_grid);
        tb.signs = smem_u32(iq2_sign);
        const int sl = lane % LPR, grp = lane / LPR;
        UnitAct act[UPL];
        int cached_row = -1;
        bool ok = true;
        // finished outputs wait in lane registers (pass n of a row group parks in that group's lane n)
        // and are finalised LPR passes at a time, so the SwiGLU / store epilogue runs once per LPR passes
        float park0 = 0.f, park1 = 0.f;
        size_t park_idx = 0;
        int parked = 0;
        int n_mma = 0;   // multi-token items so far: the same in every consumer warp
        auto flush = [&]() {
            if (sl < parked) {
                float a0 = park0, a1 = park1;
                if (TYPE == IQ2_XXS) { a0 *= 0.125f; a1 *= 0.125f; }
                if (park_idx != (size_t)-1) {
                    if (DUAL) count_bad(p.bad, a0, a1);
                    p.y[park_idx] = DUAL ? swiglu_f(a0, a1, p.clamp, p.clamp_fused) : a0;
                }
            }
            parked = 0;
        };
        // output this thread owes for the last multi-token item (roles are recomputed where needed
        // rather than kept in registers through the scalar path)
        bool pend = false, pend_on = false;
        size_t pend_idx = 0;
        const int ks_n = 1 << p.mma_ks_log2;
        // final sums: thread t of the consumer warps owns output t of the tile (pair t / R, row t % R)
        auto out_role = [&](int &o_tok, int &o_row) {
            const int ot = warp * 32 + lane;
            o_tok = (ot * p.mma_rdiv) >> 16;   // ot / R for ot < 1024
            o_row = ot - o_tok * p.R;
        };
        auto finish_pending = [&]() -> bool {
            if (!pend) return true;
            pend = false;
            const int q = n_mma - 1;
            if (!mbar_wait(&part_bar, q & 1)) return false;
            if (pend_on) {
                int o_tok, o_row;
                out_role(o_tok, o_row);
                // the piece's warps: ks_n slices of the first matrix, then (DUAL) ks_n of the second
                const float *pr = &part[q & 1][0][0] + ((o_row >> 4) << (p.mma_ks_log2 + (DUAL ? 1 : 0))) * PART +
                                  (o_row & 15) * MMID_MAXTOK + o_tok;
                float a0 = 0.f, a1 = 0.f;
                for (int i = 0; i < ks_n; ++i) {
                    a0 += pr[i * PART];
                    if (DUAL) a1 += pr[(ks_n + i) * PART];
                }
                if (DUAL) count_bad(p.bad, a0, a1);
                p.y[pend_idx] = DUAL ? swiglu_f(a0, a1, p.clamp, p.clamp_fused) : a0;
            }
            return true;
        };
        for (int k = 0; k < n_mine && ok; ++k) {
            const int s = k % nstage;
            if (!mbar_wait(&full_bar[s], (k / nstage) & 1)) {
                if (lane == 0) atomicExch(p.err, 2);
                ok = false;
                break;
            }
            const StageMeta &m = meta[s];
            const int m_nrows = m.nrows, m_ntok = m.ntok, m_r0 = m.r0;
            const uint32_t stage = smem_u32(smem + (size_t)s * p.stage_bytes);
            const uint32_t t0 = stage + m.w0_off;
            const uint32_t t1 = stage + p.wtile_bytes + m.w1_off;
            const uint32_t q8base = stage + (DUAL ? 2 : 1) * p.wtile_bytes;
            if (MMA && m_ntok >= 2 && ((t0 | (DUAL ? t1 : 0u)) & (QTraits<TYPE>::kAlign >= 4 ? 3u : 1u)) == 0) {
                // ---- multi-token item: warp = (16-row piece ti, matrix, slice [hb0, hb1) of the row) ----
                const int wsh = p.mma_ks_log2 + (DUAL ? 1 : 0);
                const int ti = warp >> wsh, mat = DUAL ? (warp >> p.mma_ks_log2) & 1 : 0;
                const int hb0 = (warp & (ks_n - 1)) * p.mma_hpw, hb1 = min(hb0 + p.mma_hpw, p.I / 128);
                // role in the final reduction, read before the stage is released
                int o_tok, o_row;
                out_role(o_tok, o_row);
                const bool o_on = o_tok < m_ntok && o_row < m_nrows;
                const size_t o_idx = o_on ? (size_t)m.pair[o_tok] * p.ldy + m_r0 + o_row : 0;
                float f0[4] = {0.f, 0.f, 0.f, 0.f};
                if (ti * 16 < m_nrows && hb0 < hb1)
                    mma_rows<TYPE, false>((mat ? t1 : t0) + (uint32_t)(ti * 16) * p.rbs, 0, p.rbs, q8base, p.q8s, p.I, hb0, hb1,
                                          lane, f0, f0);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
                // the previous multi-token item is finished first: its phase of part_bar must be over
                // before this warp arrives for the next one
                if (!finish_pending()) {
                    if (lane == 0) atomicExch(p.err, 3);
                    ok = false;
                    break;
                }
                // partial sums of this warp: lanes with c < 2 hold pairs 2c, 2c+1 of rows g and g+8
                float *pw = part[n_mma & 1][warp];
                {
                    const int g = lane >> 2, c = lane & 3;
                    if (c < MMID_MAXTOK / 2) {
                        *reinterpret_cast<float2 *>(pw + g * MMID_MAXTOK + 2 * c) = make_float2(f0[0], f0[1]);
                        *reinterpret_cast<float2 *>(pw + (g + 8) * MMID_MAXTOK + 2 * c) = make_float2(f0[2], f0[3]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&part_bar);
                // the sums are added up one item later (finish_pending), when every warp's slice has long
                // arrived.  The buffer written two items ago is free: a warp gets here only after the wait
                // for the previous item's phase, which every warp joins after its reads of the one before.
                pend = true; pend_on = o_on; pend_idx = o_idx;
                ++n_mma;
                continue;
            }
            for (int tk = 0; tk < m_ntok; ++tk) {
                const int pair = m.pair[tk];
                const int xrow = m.xrow[tk];
                if (MMA || xrow != cached_row) {
#pragma unroll
                    for (int i = 0; i < UPL; ++i) {
                        const int u = sl + LPR * i;
                        if (u < U) load_unit_act<TYPE>(q8base + tk * p.q8s, p.I, u, act[i]);
                    }
                    cached_row = xrow;
                }
                for (int base = warp * RPW; base < m_nrows; base += NCW * RPW) {
                    const int rr = base + grp;
                    const bool valid = rr < m_nrows;
                    float acc0 = 0.f, acc1 = 0.f;
                    if (valid) {
#pragma unroll
                        for (int i = 0; i < UPL; ++i) {
                            const int u = sl + LPR * i;
                            if (u < U) {
                                int is, ms;
                                float d, dm;
                                const uint32_t boff = (uint32_t)rr * p.rbs + (uint32_t)(u >> 2) * BB;
                                unit_dot<TYPE>(t0 + boff, u & 3, act[i], tb, is, ms, d, dm);
                                acc0 = fmaf(d * act[i].d, (float)is, acc0);
                                if (QTraits<TYPE>::kHasMin) acc0 = fmaf(-(dm * act[i].d), (float)ms, acc0);
                                if (DUAL) {
                                    unit_dot<TYPE>(t1 + boff, u & 3, act[i], tb, is, ms, d, dm);
                                    acc1 = fmaf(d * act[i].d, (float)is, acc1);
                                    if (QTraits<TYPE>::kHasMin) acc1 = fmaf(-(dm * act[i].d), (float)ms, acc1);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int off = LPR / 2; off > 0; off >>= 1) {
                        acc0 += __shfl_xor_sync(0xffffffffu, acc0, off);
                        if (DUAL) acc1 += __shfl_xor_sync(0xffffffffu, acc1, off);
                    }
                    // every lane of a row group now holds the row's sums: the group's lane `parked` keeps them
                    if (sl == parked) {
                        park0 = acc0; park1 = acc1;
                        park_idx = valid ? (size_t)pair * p.ldy + m_r0 + rr : (size_t)-1;
                    }
                    if (++parked == LPR) flush();
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
        flush();
        if (MMA && ok && !finish_pending() && lane == 0) atomicExch(p.err, 3);
    }
}

}  // namespace zmoe
