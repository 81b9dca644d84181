// mmid.cu -- geometry selection and dispatch for the decode-shaped expert matmul.
#include <map>
#include <mutex>
#include <utility>

#include "mmid.cuh"
#include "zmoe_internal.h"

namespace zmoe {

int mmid_geometry(int type, int I, int O, bool dual, MmidGeom *g) {
    const int bb = block_bytes(type);
    if (bb == 0) return ZMOE_ERR_TYPE;
    if (I <= 0 || O <= 0 || I % QK_K != 0) return ZMOE_ERR_SHAPE;
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
    g->ncw = g->lpr == 16 ? 12 : g->upl <= 2 ? 16 : g->upl == 3 ? 12 : 8;
    const int rb = (I / QK_K) * bb;
    const int rpw = 32 / g->lpr;
    int unit = rpw * g->ncw;  // rows of one full pass of the consumer warps
    // tiles must start and end on 16-byte boundaries of the tensor
    int ralign = 1;
    while ((ralign * rb) % 16 != 0) ralign *= 2;
    while (unit % ralign != 0) unit *= 2;
    const int ntile = dual ? 2 : 1;
    const int q8s = q8row_stride(I);
    const int budget = 200 * 1024;
    int R = unit;
    // grow towards ~40 KB of weights per stage while at least three stages fit
    while ((size_t)ntile * (R + unit) * rb <= 40 * 1024 && R + unit <= O + unit - 1) R += unit;
    for (;;) {
        g->R = R;
        g->wtile_bytes = (R * rb + 16 + 16 + 127) & ~127;
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

template <int TYPE, bool DUAL>
static KernelFn pick(int lpr, int upl) {
    if (lpr == 8) {
        switch (upl) {
        case 1: return mmid_kernel<TYPE, 8, 1, DUAL, 16>;
        case 2: return mmid_kernel<TYPE, 8, 2, DUAL, 16>;
        case 3: return mmid_kernel<TYPE, 8, 3, DUAL, 12>;
        case 4: return mmid_kernel<TYPE, 8, 4, DUAL, 8>;
        }
    } else if (lpr == 16) {
        switch (upl) {
        case 3: return mmid_kernel<TYPE, 16, 3, DUAL, 12>;
        case 4: return mmid_kernel<TYPE, 16, 4, DUAL, 12>;
        }
    } else {
        switch (upl) {
        case 1: return mmid_kernel<TYPE, 32, 1, DUAL, 16>;
        case 2: return mmid_kernel<TYPE, 32, 2, DUAL, 16>;
        case 3: return mmid_kernel<TYPE, 32, 3, DUAL, 12>;
        case 4: return mmid_kernel<TYPE, 32, 4, DUAL, 8>;
        }
    }
    return nullptr;
}

template <bool DUAL>
static KernelFn pick_type(int type, int lpr, int upl) {
    switch (type) {
    case Q2_K: return pick<Q2_K, DUAL>(lpr, upl);
    case Q3_K: return pick<Q3_K, DUAL>(lpr, upl);
    case Q4_K: return pick<Q4_K, DUAL>(lpr, upl);
    case IQ2_XXS: return pick<IQ2_XXS, DUAL>(lpr, upl);
    }
    return nullptr;
}

int launch_mmid(const MmidLaunch &L, const MmidGeom &g, cudaStream_t st) {
    KernelFn fn = L.dual ? pick_type<true>(L.type, g.lpr, g.upl) : pick_type<false>(L.type, g.lpr, g.upl);
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
    p.err = L.err;
    return launch_pdl(fn, dim3(L.n_sm), dim3(32 * (g.ncw + 1)), g.smem_bytes, st, p) == cudaSuccess ? ZMOE_OK
                                                                                                   : ZMOE_ERR_CUDA;
}

}  // namespace zmoe
