// mmid2.cuh -- the decode-shaped MUL_MAT_ID kernel with K-chunked stages and independent warp sets.
//
// Same job and same arithmetic as mmid.cuh (quantised expert rows against Q8_K activations, one persistent
// CTA per SM, replaces reference core/gpu_expert_executor.cpp:358-387,512-513 and
// kernels/quant/kquant_matmul.cu:647-700), restructured around what limited that kernel: every consumer warp
// paid the fixed cost of a pipeline stage (barrier wait, descriptor, activation reload, reduction) for one or
// two rows' worth of work.
//   * An item is (expert, 32 consecutive rows, up to `maxtok` pairs: 4 to 8, what the stages have room for).  It is
//     streamed as chunks of CB super-blocks of all 32 rows: a stage holds [32 rows x CB blocks] of the tile (two
//     tiles in DUAL mode) and the matching slice of the pairs' packed activation rows.  Where the tensor's rows
//     are multiples of 16 bytes the chunk is one tiled copy (box = chunk width x 32 rows); short rows of any
//     length that is a multiple of 4 bytes are copied whole (one chunk) as a contiguous run.
//   * The 12 consumer warps form three sets of four.  Each set has its own ring of two stages, its own producer
//     warp and works on its own item: a warp's share of a stage is 8 rows x CB blocks (x 2 matrices),
//     accumulated in registers across the item's chunks, so the per-stage fixed cost is spread over 8 to 16
//     times more arithmetic and no reduction runs until the item ends.  A producer takes the CTA's next item
//     from a shared counter, so sets with light items simply take more of them.  (One producer warp for all
//     three sets was measured to be the bottleneck: it shares a scheduler with three busy consumer warps.)
//   * One pair per item: a lane owns a run of units of one row (and of its partner row in the other matrix);
//     Q2_K decodes a super-block at a time.  Two or more pairs: mma.sync on 16-row pieces (mmid_mma.cuh) with all
//     eight fragment columns in use; the set's warps split pieces and matrices (DUAL) or pieces and halves of
//     the chunk, and meet through shared memory once per item.
// Every wait is bounded; on expiry the warp raises the error flag and leaves.
#pragma once

#include "mmid.cuh"

namespace zmoe {

constexpr int M2_NSET = 3;             // independent warp sets
constexpr int M2_WPS = 4;              // warps per set
constexpr int M2_NSTG = 2;             // stages per set
constexpr int M2_NCW = M2_NSET * M2_WPS;
constexpr int M2_R = 32;               // rows per item
constexpr int M2_MAXTOK = 8;           // most pairs per item (the launch's maxtok is 4 or 8)

struct M2Params {
    const uint8_t *w0, *w1;
    size_t stride0, stride1, total0, total1;
    int I, O, rb;
    int cb;          // super-blocks per chunk
    int nch;         // chunks per row
    int cbytes;      // bytes of one row's chunk in global memory
    int pitch;       // bytes between rows of a tile in shared memory
    int lb_log2;     // one-pair path: log2 of the lanes that share a row (one super-block each)
    int acb;         // super-blocks of the activation slice a stage holds: cb, or 4 where cb is 2 (the slice then
                     // covers two consecutive chunks)
    int I_l;         // elements of that slice
    int maxtok;      // pairs per item the plan was built with
    int q8s_l;       // bytes between the pairs' activation slices in shared memory
    int tiled;       // chunks come through tm0 / tm1
    const uint8_t *q8;
    int q8_stride, xdiv;
    float *y;
    int ldy;
    PlanView plan;
    int hdr_items;
    float clamp;
    int clamp_fused;
    int stage_bytes, wtile_bytes;
    int *err, *bad;
    int *queue;      // [2] ticket counter and finished-producer counter, both zero between launches; or null
    unsigned long long *stats;   // cycle counters (builds with ZMOE_GEMM_STATS only), or null
    alignas(64) CUtensorMap tm0, tm1;
};

// Cycle accounting, compiled in with -DZMOE_GEMM_STATS: every warp adds its clock64() differences to
//   [0] consumers waiting for a stage  [1] consumers working  [2] producer with nothing to issue
//   [3] producer issuing  [4] stages filled  [5] stages consumed (per warp)
#ifdef ZMOE_GEMM_STATS
#define M2STAT_NOW() clock64()
#define M2STAT_ADD(slot, v) do { if (p.stats && lane == 0) atomicAdd(&p.stats[slot], (unsigned long long)(v)); } while (0)
#else
#define M2STAT_NOW() 0ll
#define M2STAT_ADD(slot, v) do { } while (0)
#endif

struct alignas(16) M2Meta {
    int expert, r0, nrows, ntok;
    int chunk, flags;          // flags: 1 = last chunk of the item, 2 = no more items for this set
    int w0_off, w1_off;
    int pair[M2_MAXTOK];
};
static_assert(sizeof(M2Meta) == 64, "meta");

// 3-D tiled copy (no multicast): box of the map at (x, row, expert)
__device__ __forceinline__ void tma_load_chunk(void *dst_smem, const void *tmap, int x, int row, int expert, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst_smem)), "l"(tmap), "r"(x), "r"(row), "r"(expert), "r"(smem_u32(bar))
        : "memory");
}

template <int TYPE, bool DUAL, bool MMA>
__global__ void __launch_bounds__(32 * (M2_NCW + 4), 1) mmid2_kernel(const __grid_constant__ M2Params p) {
    constexpr int BB = QTraits<TYPE>::kBytes;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[M2_NSET][M2_NSTG], empty_bar[M2_NSET][M2_NSTG], x_bar[M2_NSET][2];
    __shared__ M2Meta meta[M2_NSET][M2_NSTG];
    __shared__ __align__(16) float exch[MMA ? M2_NSET : 1][2][2][32][4];   // [set][item parity][piece][lane]
    __shared__ __align__(8) uint64_t iq2_grid[TYPE == IQ2_XXS ? 256 : 1], iq2_sign[TYPE == IQ2_XXS ? 128 : 1];
    __shared__ int s_item_offs[MMID_PLAN_SMEM + 1], s_active[MMID_PLAN_SMEM], s_aoffs[MMID_PLAN_SMEM],
        s_antok[MMID_PLAN_SMEM];
    __shared__ int s_next;   // the CTA's next item
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        s_next = 0;
        for (int s = 0; s < M2_NSET; ++s) {
            for (int g = 0; g < M2_NSTG; ++g) {
                mbar_init(&full_bar[s][g], 1);
                mbar_init(&empty_bar[s][g], M2_WPS);
            }
            mbar_init(&x_bar[s][0], 2);
            mbar_init(&x_bar[s][1], 2);
        }
        mbar_init_fence();
    }
    if (TYPE == IQ2_XXS) iq2_fill_tables(iq2_grid, iq2_sign);
    __syncthreads();

    // everything below reads what earlier kernels of the stream wrote
    pdl_wait_prior_grid();
    pdl_launch_dependents();

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
    const int G = (int)gridDim.x;
    const int n_mine = n_items > (int)blockIdx.x ? (n_items - (int)blockIdx.x + G - 1) / G : 0;
    const int nrt = (p.O + M2_R - 1) / M2_R;

    if (warp >= M2_NCW) {
        // ------------------------------ producers -----------------------------
        // One warp per set (a spare warp rounds the CTA to 16 and leaves at once).  A producer takes the CTA's
        // next item from a shared counter -- sets with light items simply take more of them -- resolves it
        // while the previous item's chunks are still being issued, and feeds its set's two stages.
        const int s = warp - M2_NCW;
        if (s >= M2_NSET) return;
        // a pair's activations for one stage: the whole packed row, or the slice of acb blocks the chunk meets (the
        // packed row is stored block by block, so a slice is one run of bytes)
        const uint32_t act_bytes = p.nch == 1 ? (uint32_t)p.q8_stride : (uint32_t)(p.acb * Q8_BLOCK_STRIDE);
        const int cpa = p.acb / p.cb;
        // what a fill needs and what does not change from fill to fill, computed once: the producer shares its
        // scheduler with three consumer warps and every instruction of a fill delays the stage
        const uint32_t wbytes = (uint32_t)(M2_R * p.pitch) * (DUAL ? 2u : 1u);
        const uint32_t q8_lane = (uint32_t)((DUAL ? 2 : 1) * p.wtile_bytes) + (uint32_t)lane * (uint32_t)p.q8s_l;
        const int xstep = p.cbytes >> 3;   // the maps count in 8-byte elements
        long long st_idle = 0, st_busy = 0, st_fills = 0;
        // item descriptor: e, r0, nrows, ntok and, in lane t < ntok, pair t
        struct Item { int e, r0, nrows, ntok, pair; const uint8_t *src; };   // src: the pair's packed activation row
        auto take = [&](Item &it) -> bool {
            // with a ticket counter the next item goes to whichever set of the grid is free first (items differ in
            // cost by their path); without one, items are dealt round-robin over the grid and a CTA's sets share them
            int j = 0;
            if (lane == 0) j = p.queue ? atomicAdd(p.queue, 1) : atomicAdd(&s_next, 1);
            j = __shfl_sync(0xffffffffu, j, 0);
            if (j >= (p.queue ? n_items : n_mine)) return false;
            const int mine = p.queue ? j : (int)blockIdx.x + j * G;
            // last a with item_offs[a] <= mine: the lanes probe 32 points of the range at once
            int lo = 0, hi = n_active - 1;
            while (lo < hi) {
                const int span = hi - lo, step = (span + 31) >> 5;
                const int probe = min(hi, lo + (lane + 1) * step);
                const int v = plan_in_smem ? s_item_offs[probe] : p.plan.item_offs[probe];
                const unsigned le = __ballot_sync(0xffffffffu, v <= mine);
                // probes are increasing: the lanes that satisfy the test form a prefix
                const int k = __popc(le);
                const int nlo = k == 0 ? lo : min(hi, lo + k * step);
                const int nhi = k == 32 ? hi : min(hi, lo + (k + 1) * step) - 1;
                lo = nlo;
                hi = max(nlo, nhi);
            }
            int e, local, ebase, ecnt;
            if (plan_in_smem) {
                e = s_active[lo]; local = mine - s_item_offs[lo]; ebase = s_aoffs[lo]; ecnt = s_antok[lo];
            } else {
                e = p.plan.active[lo]; local = mine - p.plan.item_offs[lo]; ebase = p.plan.aoffs[lo]; ecnt = p.plan.antok[lo];
            }
            const int tc = local / nrt, rt = local % nrt;
            it.e = e;
            it.r0 = rt * M2_R;
            it.nrows = min(M2_R, p.O - it.r0);
            it.ntok = min(p.maxtok, ecnt - tc * p.maxtok);
            it.pair = lane < it.ntok ? p.plan.slot[ebase + tc * p.maxtok + lane] : 0;
            it.src = p.q8 + (size_t)(it.pair / p.xdiv) * p.q8_stride;
            return true;
        };
        Item cur, nxt;
        bool have = take(cur);
        int f = 0;
        bool alive = true;
        while (have && alive) {
            bool have_next = false;
            // this item's activation slices, walked chunk by chunk
            const uint8_t *su = cur.src;
            int x = 0, cc = 0;
            for (int c = 0; c < p.nch; ++c, ++f) {
                const int slot = f % M2_NSTG;
                const long long st_t0 = M2STAT_NOW();
                if (f >= M2_NSTG && !mbar_wait(&empty_bar[s][slot], ((f / M2_NSTG) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.err, 1);
                    alive = false;
                    break;
                }
                const long long st_t1 = M2STAT_NOW();
                M2Meta &m = meta[s][slot];
                uint8_t *stage = smem + (size_t)(s * M2_NSTG + slot) * p.stage_bytes;
                uint64_t *bar = &full_bar[s][slot];
                uint32_t bytes = 0;
                if (lane == 0) {
                    int w0_off = 0, w1_off = 0;
                    if (p.tiled) {
                        // the box is always 32 full rows of `pitch` bytes: rows past the expert's last and bytes past
                        // the row's end arrive as zeros
                        tma_load_chunk(stage, &p.tm0, x, cur.r0, cur.e, bar);
                        if (DUAL) tma_load_chunk(stage + p.wtile_bytes, &p.tm1, x, cur.r0, cur.e, bar);
                        bytes = wbytes;
                    } else {
                        const size_t g0 = (size_t)cur.e * p.stride0 + (size_t)cur.r0 * p.rb;
                        bytes += issue_tile(stage, p.w0, p.total0, g0, g0 + (size_t)cur.nrows * p.rb, bar, &w0_off);
                        if (DUAL) {
                            const size_t h0 = (size_t)cur.e * p.stride1 + (size_t)cur.r0 * p.rb;
                            bytes += issue_tile(stage + p.wtile_bytes, p.w1, p.total1, h0, h0 + (size_t)cur.nrows * p.rb, bar, &w1_off);
                        }
                    }
                    *reinterpret_cast<int4 *>(&m.expert) = make_int4(cur.e, cur.r0, cur.nrows, cur.ntok);
                    *reinterpret_cast<int4 *>(&m.chunk) = make_int4(c, c + 1 == p.nch ? 1 : 0, w0_off, w1_off);
                }
                if (lane < cur.ntok) {
                    // this chunk's slice of the pair's packed activation row, laid out as a row of I_l elements
                    m.pair[lane] = cur.pair;
                    uint8_t *dst = stage + q8_lane;
                    bulk_g2s(dst, su, act_bytes, bar);
                }
                __syncwarp();
                // the producer's own arrival, with the byte count, is what lets the phase complete
                if (lane == 0) mbar_arrive_expect_tx(bar, bytes + (uint32_t)cur.ntok * act_bytes);
                x += xstep;
                if (++cc == cpa) { cc = 0; su += act_bytes; }
                st_idle += st_t1 - st_t0;
                st_busy += M2STAT_NOW() - st_t1;
                ++st_fills;
                // the next item is resolved once this item's first chunk is on its way
                if (c == 0) have_next = take(nxt);
            }
            cur = nxt;
            have = have_next;
        }
        // nothing left: tell the set to stop
        if (alive) {
            const int slot = f % M2_NSTG;
            if (f >= M2_NSTG && !mbar_wait(&empty_bar[s][slot], ((f / M2_NSTG) - 1) & 1)) {
                if (lane == 0) atomicExch(p.err, 1);
            } else if (lane == 0) {
                meta[s][slot].flags = 2;
                mbar_arrive(&full_bar[s][slot]);
            }
        }
        // the last producer of the grid to finish leaves the counters zero for the next launch
        if (p.queue && lane == 0) {
            if (atomicAdd(p.queue + 1, 1) == M2_NSET * G - 1) {
                p.queue[0] = 0;
                p.queue[1] = 0;
            }
        }
        M2STAT_ADD(2, st_idle); M2STAT_ADD(3, st_busy); M2STAT_ADD(4, st_fills);
    } else {
        // ------------------------------ consumers -----------------------------
        const int set = warp / M2_WPS, ws = warp % M2_WPS;
        Iq2Tables tb;
        tb.grid = smem_u32(iq2_grid);
        tb.signs = smem_u32(iq2_sign);
        // one-pair path: lane = (row rl of the warp's rows, run bl of upl consecutive 64-element units of the chunk)
        const int LB = 1 << p.lb_log2, bl = lane & (LB - 1), rl = lane >> p.lb_log2, rpp = 32 >> p.lb_log2;
        const int np = M2_R / (M2_WPS * rpp);   // passes over the tile: 1 (four lanes per row) or 2 (eight)
        const int n_units = 4 * p.cb, upl = (n_units + LB - 1) >> p.lb_log2;
        const int cpa = p.acb / p.cb;
        // [pass][matrix][pair]; builds with the tensor-core path send every item of two or more pairs there
        constexpr int SC = MMA ? 1 : M2_MAXTOK;
        constexpr int UNIT_UNROLL = (TYPE == Q3_K || TYPE == IQ2_XXS) ? 1 : 4;
        float acc[2][2][SC];
        float f0[4] = {0.f, 0.f, 0.f, 0.f};     // tensor-core path: (row g | g+8) x (pair 2c | 2c+1)
        // tensor-core path: warp = (16-row piece, matrix) in DUAL mode, (piece, half of the chunk) otherwise
        const int piece = ws >> 1, half = ws & 1;
        int hb0 = 0, hb1 = 2 * p.cb;
        if (!DUAL) {
            int mid = p.cb;                                          // in half super-blocks
            if (MmaPath<TYPE>::kGrain == 2) mid = (mid + 1) & ~1;
            if (half == 0) hb1 = mid; else hb0 = mid;
        }
        int fcount = 0, n_mma = 0;
        long long st_wait = 0, st_work = 0;
        for (;;) {
            const int slot = fcount % M2_NSTG;
            const long long st_t0 = M2STAT_NOW();
            if (!mbar_wait(&full_bar[set][slot], (fcount / M2_NSTG) & 1)) {
                if (lane == 0) atomicExch(p.err, 2);
                break;
            }
            const long long st_t1 = M2STAT_NOW();
            st_wait += st_t1 - st_t0;
            const M2Meta &m = meta[set][slot];
            const int flags = m.flags;
            if (flags & 2) break;
            const int m_nrows = m.nrows, m_ntok = m.ntok, m_r0 = m.r0;
            const uint32_t stage = smem_u32(smem + (size_t)(set * M2_NSTG + slot) * p.stage_bytes);
            const uint32_t t0 = stage + m.w0_off;
            const uint32_t t1 = stage + p.wtile_bytes + m.w1_off;
            const uint32_t q8base = stage + (DUAL ? 2 : 1) * p.wtile_bytes;
            const bool mma_item = MMA && m_ntok >= 2;
            const int ab = (m.chunk & (cpa - 1)) * p.cb;   // where the chunk's blocks sit inside the activation slice (cpa is 1 or 2)
            if (m.chunk == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) f0[i] = 0.f;
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b)
#pragma unroll
                        for (int t = 0; t < SC; ++t) acc[a][b][t] = 0.f;
            }
            if (mma_item) {
                // block b of the activation slice meets block b - ab of the chunk: shift the tile instead of the index
                if (piece * 16 < m_nrows && hb0 < hb1)
                    mma_rows<TYPE, false, false, M2_MAXTOK>((DUAL && half ? t1 : t0) + (uint32_t)(piece * 16) * p.pitch - (uint32_t)(ab * BB),
                                                            0, p.pitch, q8base, p.q8s_l, p.I_l, hb0 + 2 * ab, hb1 + 2 * ab, lane, f0, f0, nullptr,
                                                            p.maxtok - 1);
            } else if (TYPE == Q2_K && upl == 4) {
                // a lane's four units are one super-block: the block-at-a-time form
                if (bl < p.cb) {
#pragma unroll
                    for (int tk = 0; tk < SC; ++tk) {
                        if (tk < m_ntok) {
#pragma unroll
                            for (int pp = 0; pp < 2; ++pp) {
                                if (pp < np) {
                                    const uint32_t roff = (uint32_t)(pp * M2_WPS * rpp + ws * rpp + rl) * p.pitch + (uint32_t)bl * BB;
                                    if (DUAL) {
                                        const uint32_t blk[2] = {t0 + roff, t1 + roff};
                                        float a[2] = {acc[pp][0][tk], acc[pp][1][tk]};
                                        q2k_block_dot<2>(blk, q8base + tk * p.q8s_l, p.I_l, ab + bl, a);
                                        acc[pp][0][tk] = a[0]; acc[pp][1][tk] = a[1];
                                    } else {
                                        const uint32_t blk[1] = {t0 + roff};
                                        float a[1] = {acc[pp][0][tk]};
                                        q2k_block_dot<1>(blk, q8base + tk * p.q8s_l, p.I_l, ab + bl, a);
                                        acc[pp][0][tk] = a[0];
                                    }
                                }
                            }
                        }
                    }
                }
            } else if (TYPE == Q3_K && SC == 1) {
                // four lanes per row (the geometry gives Q3_K lb_log2 == 2, so np == 1: a warp's lanes cover eight rows),
                // each takes a run of half super-blocks
                const int n_half = 2 * p.cb, hpl = (n_half + 3) >> 2;
                if (m_ntok > 0) {
#pragma unroll 1
                    for (int i = 0; i < hpl; ++i) {
                        const int hb = bl * hpl + i;
                        if (hb >= n_half) break;
                        const uint32_t roff = (uint32_t)(ws * rpp + rl) * p.pitch + (uint32_t)(hb >> 1) * BB;
                        if (DUAL) {
                            const uint32_t blk[2] = {t0 + roff, t1 + roff};
                            float a[2] = {acc[0][0][0], acc[0][1][0]};
                            q3k_half_dot<2>(blk, hb & 1, q8base, p.I_l, ab + (hb >> 1), a);
                            acc[0][0][0] = a[0]; acc[0][1][0] = a[1];
                        } else {
                            const uint32_t blk[1] = {t0 + roff};
                            float a[1] = {acc[0][0][0]};
                            q3k_half_dot<1>(blk, hb & 1, q8base, p.I_l, ab + (hb >> 1), a);
                            acc[0][0][0] = a[0];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int tk = 0; tk < SC; ++tk) {
                    if (tk < m_ntok) {
                        // the unit loop stays rolled for the formats whose unit dot is long (Q3_K, IQ2_XXS): unrolled, the
                        // consumer loop outgrew the instruction cache (84 % hit rate, "no instruction" the top stall)
#pragma unroll(UNIT_UNROLL)
                        for (int i = 0; i < upl; ++i) {
                            const int u = bl * upl + i;
                            if (u >= n_units) continue;
                            const int sub = u & 3;
                            const uint32_t boff = (uint32_t)(u >> 2) * BB;
                            UnitAct ua;
                            load_unit_act<TYPE>(q8base + tk * p.q8s_l, p.I_l, 4 * ab + u, ua);
#pragma unroll
                            for (int pp = 0; pp < 2; ++pp) {
                                if (pp < np) {
                                    const uint32_t roff = (uint32_t)(pp * M2_WPS * rpp + ws * rpp + rl) * p.pitch + boff;
                                    int is, ms;
                                    float d, dm;
                                    unit_dot<TYPE>(t0 + roff, sub, ua, tb, is, ms, d, dm);
                                    acc[pp][0][tk] = fmaf(d * ua.d, (float)is, acc[pp][0][tk]);
                                    if (QTraits<TYPE>::kHasMin) acc[pp][0][tk] = fmaf(-(dm * ua.d), (float)ms, acc[pp][0][tk]);
                                    if (DUAL) {
                                        unit_dot<TYPE>(t1 + roff, sub, ua, tb, is, ms, d, dm);
                                        acc[pp][1][tk] = fmaf(d * ua.d, (float)is, acc[pp][1][tk]);
                                        if (QTraits<TYPE>::kHasMin) acc[pp][1][tk] = fmaf(-(dm * ua.d), (float)ms, acc[pp][1][tk]);
                                    }
                                }
                            }
                        }
                    }
                }
            }
            if (flags & 1) {
                // ---- the item is complete: reduce, activate, store (before the stage is released, which orders
                // this item's use of the exchange buffer before the use two items later) ----
                if (mma_item) {
                    const int par = n_mma & 1;
                    float *mine = &exch[MMA ? set : 0][par][piece][lane][0];
                    if (half == 1) {
                        *reinterpret_cast<float4 *>(mine) = make_float4(f0[0], f0[1], f0[2], f0[3]);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&x_bar[set][par]);
                    } else {
                        if (!mbar_wait(&x_bar[set][par], (n_mma >> 1) & 1)) {
                            if (lane == 0) atomicExch(p.err, 3);
                            break;
                        }
                        const float4 o = *reinterpret_cast<const float4 *>(mine);
                        const float other[4] = {o.x, o.y, o.z, o.w};
                        const int g = lane >> 2, c = lane & 3;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int row = piece * 16 + g + (i >> 1) * 8, tk = 2 * c + (i & 1);
                            if (tk < m_ntok && row < m_nrows) {
                                float v;
                                if (DUAL) {
                                    count_bad(p.bad, f0[i], other[i]);
                                    v = swiglu_f(f0[i], other[i], p.clamp, p.clamp_fused);
                                } else {
                                    v = f0[i] + other[i];
                                }
                                p.y[(size_t)m.pair[tk] * p.ldy + m_r0 + row] = v;
                            }
                        }
                    }
                    ++n_mma;
                } else {
#pragma unroll
                    for (int pp = 0; pp < 2; ++pp) {
                        if (pp < np) {
                            const int row = pp * M2_WPS * rpp + ws * rpp + rl;
#pragma unroll
                            for (int tk = 0; tk < SC; ++tk) {
                                if (tk < m_ntok) {
                                    float a0 = acc[pp][0][tk], a1 = DUAL ? acc[pp][1][tk] : 0.f;
                                    for (int off = LB >> 1; off > 0; off >>= 1) {
                                        a0 += __shfl_xor_sync(0xffffffffu, a0, off);
                                        if (DUAL) a1 += __shfl_xor_sync(0xffffffffu, a1, off);
                                    }
                                    if (TYPE == IQ2_XXS) { a0 *= 0.125f; a1 *= 0.125f; }
                                    if (bl == 0 && row < m_nrows) {
                                        if (DUAL) count_bad(p.bad, a0, a1);
                                        p.y[(size_t)m.pair[tk] * p.ldy + m_r0 + row] = DUAL ? swiglu_f(a0, a1, p.clamp, p.clamp_fused) : a0;
                                    }
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[set][slot]);
            ++fcount;
            st_work += M2STAT_NOW() - st_t1;
        }
        M2STAT_ADD(0, st_wait); M2STAT_ADD(1, st_work); M2STAT_ADD(5, fcount);
    }
}

}  // namespace zmoe
