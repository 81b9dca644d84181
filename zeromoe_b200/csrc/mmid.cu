// mmid.cu -- geometry selection and dispatch for the decode-shaped expert matmul.
#include <map>
#include <mutex>
#include <utility>

#include "mmid.cuh"
#include "mmid2.cuh"
#include "zmoe_internal.h"

namespace zmoe {

// Geometry of the K-chunked kernel, where one exists for the shape: chunks of cb super-blocks whose bytes are a
// multiple of 16 (tiled copies; the tensor's rows must be multiples of 16 bytes too), or -- rows of at most eight
// super-blocks -- the whole row as one chunk, copied as a contiguous run.
static bool mmid2_geometry(int type, int I, int O, bool dual, MmidGeom *g) {
    const int bb = block_bytes(type), nb = I / QK_K, rb = nb * bb;
    if (nb < 2 || rb % 4 != 0) return false;
    const int ntile = dual ? 2 : 1;
    const int budget = 208 * 1024;   // with the kernel's static arrays (about 15 KB) under the 227 KB a CTA may hold
    int cands[5], nc = 0;
    if (rb % 16 == 0) {
        cands[nc++] = dual ? 4 : 8;
        cands[nc++] = dual ? 8 : 4;
        cands[nc++] = 2;
    }
    if (nb <= 8) cands[nc++] = nb;   // the whole row
    for (int i = 0; i < nc; ++i) {
        const int cb = cands[i];
        if (cb > nb || nb % cb != 0) continue;
        const bool whole = cb == nb;
        const bool tiled = rb % 16 == 0 && (cb * bb) % 16 == 0;
        if (!tiled && !whole) continue;
        // a chunk that is not the whole row rides with a slice of the packed activation row (stored block by block,
        // so any run of blocks is one 16-byte-aligned piece): four super-blocks, which then cover two chunks of two
        const int acb = whole ? cb : (cb == 2 ? 4 : cb);
        if (!whole && (acb % 4 != 0 || nb % acb != 0)) continue;
        int pitch = rb;
        if (tiled) {
            pitch = (cb * bb + 15) & ~15;
            while ((pitch / 4) % 8 != 4) pitch += 16;   // fragment loads of eight rows fall into distinct banks
            if (pitch / 8 > 256) continue;
        }
        const int I_l = acb * QK_K;
        int q8s_l = q8row_stride(I_l);
        while ((q8s_l / 4) % 16 == 0) q8s_l += 16;
        const int wtile = (M2_R * pitch + 32 + 127) & ~127;
        // eight pairs per item where the tensor-core consumer path serves the type (its cost does not depend on
        // the pairs) and the wider activation area still fits; else four
        int maxtok = (type == Q2_K || type == Q3_K || type == Q4_K) ? M2_MAXTOK : 4;
        int stage = (ntile * wtile + maxtok * q8s_l + 127) & ~127;
        while (maxtok > 4 && (size_t)stage * M2_NSET * M2_NSTG > (size_t)budget) {
            --maxtok;
            stage = (ntile * wtile + maxtok * q8s_l + 127) & ~127;
        }
        if ((size_t)stage * M2_NSET * M2_NSTG > (size_t)budget) continue;
        g->v2 = 1; g->maxtok = maxtok; g->cb = cb; g->acb = acb; g->nch = nb / cb; g->pitch = pitch; g->tiled = tiled ? 1 : 0;
        g->lb_log2 = cb * 4 > 16 ? 3 : 2;   // up to four units per lane
        if (type == Q3_K) g->lb_log2 = 2;   // its one-pair path works on half super-blocks, four lanes to a row
        g->q8s_l = q8s_l;
        g->R = M2_R; g->wtile_bytes = wtile; g->stage_bytes = stage; g->nstage = M2_NSTG;
        g->smem_bytes = (size_t)stage * M2_NSET * M2_NSTG;
        g->rbs = pitch; g->q8s = q8s_l; g->ncw = M2_NCW; g->lpr = 1 << g->lb_log2; g->upl = (cb * 4 + g->lpr - 1) / g->lpr;
        return true;
    }
    return false;
}

int mmid_geometry(int type, int I, int O, bool dual, MmidGeom *g, bool allow_v2) {
    const int bb = block_bytes(type);
    if (bb == 0) return ZMOE_ERR_TYPE;
    if (I <= 0 || O <= 0 || I % QK_K != 0) return ZMOE_ERR_SHAPE;
    *g = MmidGeom();
    if (allow_v2 && mmid2_geometry(type, I, O, dual, g)) return ZMOE_OK;
    const int U = I / 64;
    if (U > 128) return ZMOE_ERR_SHAPE;  // rows longer than 8192 elements: no kernel yet
    if (U <= 32) {
        g->lpr = 8;
        g->upl = (U + 7) / 8;
    } else {
        g->lpr = 32;
        g->upl = (U + 31) / 32;
    }
    // must match the instantiations in pick(): consumer warps per (lanes per row, units per lane)
    g->ncw = g->upl <= 2 ? 16 : g->upl == 3 ? 12 : 8;
    const int rb = (I / QK_K) * bb;
    const int rpw = 32 / g->lpr;
    int unit = rpw * g->ncw;  // rows of one full pass of the consumer warps
    // tiles must start and end on 16-byte boundaries of the tensor
    int ralign = 1;
    while ((ralign * rb) % 16 != 0) ralign *= 2;
    while (unit % ralign != 0) unit *= 2;
    const int ntile = dual ? 2 : 1;
    // Shared-memory strides.  The multi-token path reads 8 rows x 4 consecutive words per load and
    // 4 activation rows x 4 words: a row stride of 4 (mod 8) words and an activation stride that is not
    // a multiple of 16 words keep those loads free of bank conflicts.  Padding weight rows needs one
    // copy per row, so rows must be multiples of 16 bytes.
    int rbs = rb, q8s = q8row_stride(I);
    if ((type == Q2_K || type == Q3_K || type == Q4_K) && rb % 16 == 0)
        while ((rbs / 4) % 8 != 4) rbs += 16;   // at most one step: rb + 16, what make_rows_map delivers
    while ((q8s / 4) % 16 == 0) q8s += 16;
    g->rbs = rbs; g->q8s = q8s;
    const int budget = 200 * 1024;
    int R = unit;
    // grow towards ~40 KB of weights per stage while at least three stages fit
    while ((size_t)ntile * (R + unit) * rbs <= 40 * 1024 && R + unit <= O + unit - 1) R += unit;
    for (;;) {
        g->R = R;
        g->wtile_bytes = (R * rbs + 16 + 16 + 127) & ~127;
        g->stage_bytes = (ntile * g->wtile_bytes + MMID_MAXTOK * q8s + 127) & ~127;
        g->nstage = budget / g->stage_bytes;
        if (g->nstage > MMID_MAXSTAGE) g->nstage = MMID_MAXSTAGE;
        if (g->nstage >= 2 || R <= ralign) break;
        R = (R / 2 / ralign) * ralign;
        if (R < ralign) R = ralign;
    }
    if (g->nstage < 2) return ZMOE_ERR_SHAPE;
    g->smem_bytes = (size_t)g->nstage * g->stage_bytes;
    return ZMOE_OK;
}

using KernelFn = void (*)(const MmidParams);

template <int TYPE, bool DUAL, bool MMA>
static KernelFn pick(int lpr, int upl) {
    if (lpr == 8) {
        switch (upl) {
        case 1: return mmid_kernel<TYPE, 8, 1, DUAL, 16, MMA>;
        case 2: return mmid_kernel<TYPE, 8, 2, DUAL, 16, MMA>;
        case 3: return mmid_kernel<TYPE, 8, 3, DUAL, 12, MMA>;
        case 4: return mmid_kernel<TYPE, 8, 4, DUAL, 8, MMA>;
        }
    } else {
        switch (upl) {
        case 1: return mmid_kernel<TYPE, 32, 1, DUAL, 16, MMA>;
        case 2: return mmid_kernel<TYPE, 32, 2, DUAL, 16, MMA>;
        case 3: return mmid_kernel<TYPE, 32, 3, DUAL, 12, MMA>;
        case 4: return mmid_kernel<TYPE, 32, 4, DUAL, 8, MMA>;
        }
    }
    return nullptr;
}

template <bool DUAL>
static KernelFn pick_type(int type, int lpr, int upl, bool mma) {
    switch (type) {
    case Q2_K: return mma ? pick<Q2_K, DUAL, true>(lpr, upl) : pick<Q2_K, DUAL, false>(lpr, upl);
    case Q3_K: return mma ? pick<Q3_K, DUAL, true>(lpr, upl) : pick<Q3_K, DUAL, false>(lpr, upl);
    case Q4_K: return mma ? pick<Q4_K, DUAL, true>(lpr, upl) : pick<Q4_K, DUAL, false>(lpr, upl);
    case IQ2_XXS: return pick<IQ2_XXS, DUAL, false>(lpr, upl);
    }
    return nullptr;
}

// The multi-token path splits a tile into 16-row pieces and each piece's row into slices of whole
// half super-blocks, one slice per warp; it needs every output of a tile to find a thread.
static bool mma_split(int type, const MmidGeom &g, int I, bool dual, int *ks, int *hpw) {
    if (type != Q2_K && type != Q3_K && type != Q4_K) return false;
    if (g.R % 16 != 0) return false;
    // rows must start on word boundaries, the same for every lane of a fragment load
    if (((I / QK_K) * block_bytes(type)) % 4 != 0) return false;
    const int pieces = (g.R / 16) * (dual ? 2 : 1);   // (piece, matrix) units that need a warp each
    if (pieces > g.ncw || MMID_MAXTOK * g.R > 32 * g.ncw) return false;
    const int nhb = I / 128;
    *ks = 1;   // a power of two
    while (*ks * 2 * pieces <= g.ncw && *ks * 2 <= nhb) *ks *= 2;
    *hpw = (nhb + *ks - 1) / *ks;
    if (type != Q3_K) *hpw = (*hpw + 1) & ~1;   // whole super-blocks per warp (MmaPath<TYPE>::kGrain)
    return true;
}

using Kernel2Fn = void (*)(const M2Params);

template <bool DUAL>
static Kernel2Fn pick2(int type, bool mma) {
    switch (type) {
    case Q2_K: return mma ? mmid2_kernel<Q2_K, DUAL, true> : mmid2_kernel<Q2_K, DUAL, false>;
    case Q3_K: return mma ? mmid2_kernel<Q3_K, DUAL, true> : mmid2_kernel<Q3_K, DUAL, false>;
    case Q4_K: return mma ? mmid2_kernel<Q4_K, DUAL, true> : mmid2_kernel<Q4_K, DUAL, false>;
    case IQ2_XXS: return mmid2_kernel<IQ2_XXS, DUAL, false>;
    }
    return nullptr;
}

static int launch_mmid2(const MmidLaunch &L, const MmidGeom &g, cudaStream_t st) {
    const bool mma = L.multi && (L.type == Q2_K || L.type == Q3_K || L.type == Q4_K);
    Kernel2Fn fn = L.dual ? pick2<true>(L.type, mma) : pick2<false>(L.type, mma);
    if (!fn) return ZMOE_ERR_TYPE;
    if ((reinterpret_cast<size_t>(L.w0) & 15) || (L.dual && (reinterpret_cast<size_t>(L.w1) & 15))) return ZMOE_ERR_ALIGN;
    if (g.tiled && (!L.tm0 || (L.dual && !L.tm1))) return ZMOE_ERR_ARG;
    if (raise_dynamic_smem(reinterpret_cast<const void *>(fn), 208 * 1024) != ZMOE_OK) return ZMOE_ERR_CUDA;
    M2Params p;
    p.w0 = static_cast<const uint8_t *>(L.w0);
    p.w1 = static_cast<const uint8_t *>(L.w1);
    p.stride0 = L.stride0; p.stride1 = L.stride1;
    p.total0 = L.total0; p.total1 = L.total1;
    p.I = L.I; p.O = L.O;
    p.rb = (L.I / QK_K) * block_bytes(L.type);
    p.cb = g.cb; p.nch = g.nch; p.cbytes = g.cb * block_bytes(L.type);
    p.acb = g.acb;
    p.maxtok = g.maxtok;
    p.pitch = g.pitch; p.lb_log2 = g.lb_log2; p.I_l = g.acb * QK_K; p.q8s_l = g.q8s_l; p.tiled = g.tiled;
    if (g.tiled) {
        p.tm0 = *L.tm0;
        if (L.dual) p.tm1 = *L.tm1;
    }
    p.q8 = L.q8;
    p.q8_stride = q8row_stride(L.I);
    p.xdiv = L.xdiv;
    p.y = L.y; p.ldy = L.ldy;
    p.plan.hdr = L.plan.hdr; p.plan.active = L.plan.active; p.plan.offs = L.plan.offs; p.plan.slot = L.plan.slot;
    p.plan.item_offs = L.down ? L.plan.item_offs_dn : L.plan.item_offs_gu;
    p.plan.aoffs = L.plan.aoffs; p.plan.antok = L.plan.antok; p.plan.cap_e = L.plan.cap_e;
    p.hdr_items = L.down ? 2 : 1;
    p.clamp = L.clamp; p.clamp_fused = L.clamp_fused;
    p.stage_bytes = g.stage_bytes; p.wtile_bytes = g.wtile_bytes;
    p.err = L.err;
    p.bad = L.dual ? L.bad : nullptr;
    p.queue = L.queue ? L.queue + (L.down ? 2 : 0) : nullptr;
    p.stats = gemm_stats_buffer(L.down ? 1 : 0);
    return launch_pdl(fn, dim3(L.n_sm), dim3(32 * (M2_NCW + 4)), g.smem_bytes, st, p) == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

// Parity hook of the tensor-core consumer path: one warp runs mma_rows on 16 weight rows against up to MMA_NTOK
// packed activation rows and writes the per-super-block s32 sums.
template <int TYPE>
__global__ void __launch_bounds__(32) mma_isums_kernel(const uint8_t *w, const uint8_t *q8, int *out, int I, int pairs, int q8s) {
    extern __shared__ __align__(128) uint8_t sm[];
    constexpr int BB = QTraits<TYPE>::kBytes;
    const int nb = I / QK_K, rb = nb * BB, qstride = q8row_stride(I);
    uint8_t *wdst = sm, *qdst = sm + ((16 * rb + 127) & ~127);
    for (int i = threadIdx.x; i < 16 * rb; i += 32) wdst[i] = w[i];
    // slots past `pairs` repeat row 0: their sums are computed and never read
    for (int t = 0; t < MMA_NTOK; ++t)
        for (int i = threadIdx.x; i < qstride; i += 32) qdst[(size_t)t * q8s + i] = q8[(size_t)(t < pairs ? t : 0) * qstride + i];
    __syncwarp();
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    mma_rows<TYPE, false, true>(smem_u32(wdst), 0, rb, smem_u32(qdst), q8s, I, 0, 2 * nb, (int)threadIdx.x, f, f, out);
}

int launch_mma_isums(int type, const void *w, const uint8_t *q8, int *out, int I, int pairs, cudaStream_t st) {
    if (pairs < 1 || pairs > MMA_NTOK) return ZMOE_ERR_ARG;
    const int nb = I / QK_K, rb = nb * block_bytes(type);
    if (rb % 4 != 0) return ZMOE_ERR_SHAPE;
    int q8s = q8row_stride(I);
    while ((q8s / 4) % 16 == 0) q8s += 16;
    const size_t smem = (size_t)((16 * rb + 127) & ~127) + (size_t)MMA_NTOK * q8s;
    if (smem > 200 * 1024) return ZMOE_ERR_SHAPE;
    void (*fn)(const uint8_t *, const uint8_t *, int *, int, int, int) = nullptr;
    switch (type) {
    case Q2_K: fn = mma_isums_kernel<Q2_K>; break;
    case Q3_K: fn = mma_isums_kernel<Q3_K>; break;
    case Q4_K: fn = mma_isums_kernel<Q4_K>; break;
    default: return ZMOE_ERR_TYPE;   // no tensor-core consumer path for the type
    }
    if (raise_dynamic_smem(reinterpret_cast<const void *>(fn), 200 * 1024) != ZMOE_OK) return ZMOE_ERR_CUDA;
    fn<<<1, 32, smem, st>>>(static_cast<const uint8_t *>(w), q8, out, I, pairs, q8s);
    return cudaPeekAtLastError() == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

int launch_mmid(const MmidLaunch &L, const MmidGeom &g, cudaStream_t st) {
    if (g.v2) return launch_mmid2(L, g, st);
    int mma_ks = 0, mma_hpw = 0;
    const bool mma = L.multi && mma_split(L.type, g, L.I, L.dual, &mma_ks, &mma_hpw);
    KernelFn fn = L.dual ? pick_type<true>(L.type, g.lpr, g.upl, mma) : pick_type<false>(L.type, g.lpr, g.upl, mma);
    if (!fn) return ZMOE_ERR_TYPE;
    if ((reinterpret_cast<size_t>(L.w0) & 15) || (L.dual && (reinterpret_cast<size_t>(L.w1) & 15))) return ZMOE_ERR_ALIGN;
    // the opt-in shared-memory limit is a per-function, per-device attribute: raise it once
    {
        static std::mutex mu;
        static std::map<std::pair<const void *, int>, size_t> done;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        size_t &have = done[std::make_pair(reinterpret_cast<const void *>(fn), dev)];
        if (have < g.smem_bytes) {
            // the budget of mmid_geometry (200 KB) plus the kernel's static arrays stays under 227 KB
            if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                return ZMOE_ERR_CUDA;
            have = 200 * 1024;
        }
    }
    MmidParams p;
    p.w0 = static_cast<const uint8_t *>(L.w0);
    p.w1 = static_cast<const uint8_t *>(L.w1);
    p.stride0 = L.stride0; p.stride1 = L.stride1;
    p.total0 = L.total0; p.total1 = L.total1;
    p.I = L.I; p.O = L.O;
    p.rb = (L.I / QK_K) * block_bytes(L.type);
    // padded rows need the tiled maps; without them tiles are dense
    p.use_tmap = g.rbs != p.rb && L.tm0 && (!L.dual || L.tm1);
    p.rbs = p.use_tmap ? g.rbs : p.rb;
    p.q8s = g.q8s;
    if (p.use_tmap) {
        p.tm0 = *L.tm0;
        if (L.dual) p.tm1 = *L.tm1;
    }
    p.R = g.R;
    p.q8 = L.q8;
    p.q8_stride = q8row_stride(L.I);
    p.xdiv = L.xdiv;
    p.y = L.y; p.ldy = L.ldy;
    p.plan.hdr = L.plan.hdr; p.plan.active = L.plan.active; p.plan.offs = L.plan.offs; p.plan.slot = L.plan.slot;
    p.plan.item_offs = L.down ? L.plan.item_offs_dn : L.plan.item_offs_gu;
    p.plan.aoffs = L.plan.aoffs; p.plan.antok = L.plan.antok; p.plan.cap_e = L.plan.cap_e;
    p.hdr_items = L.down ? 2 : 1;
    p.clamp = L.clamp; p.clamp_fused = L.clamp_fused;
    p.nstage = g.nstage; p.stage_bytes = g.stage_bytes; p.wtile_bytes = g.wtile_bytes;
    p.mma_ks_log2 = 0;
    while ((1 << p.mma_ks_log2) < mma_ks) ++p.mma_ks_log2;
    p.mma_hpw = mma_hpw;
    p.mma_rdiv = (65536 + g.R - 1) / g.R;
    p.err = L.err;
    p.bad = L.dual ? L.bad : nullptr;
    return launch_pdl(fn, dim3(L.n_sm), dim3(32 * (g.ncw + 1)), g.smem_bytes, st, p) == cudaSuccess ? ZMOE_OK
                                                                                                   : ZMOE_ERR_CUDA;
}

}  // namespace zmoe
