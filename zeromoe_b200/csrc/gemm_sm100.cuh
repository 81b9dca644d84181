// gemm_sm100.cuh -- prefill-shaped grouped expert GEMM on the 5th-generation tensor
// cores: C[f, p] = sum_k W_e[f, k] * X[p, k] for the pairs p routed to expert e.
//
// Replaces, for calls with many tokens per expert, the GEMV-shaped per-expert loop of
// reference core/batched_dispatch_pipeline.cpp:1833-1921 and the dequantise-to-bf16 +
// cublasGemmEx escape hatch of reference backends/cuda/cuda_kernel_dispatcher.cpp:58-124.
//
// One persistent CTA per SM, warp-specialised:
//   warps 0-15 producers: dequantise a 128-row x 64-k weight tile (two in DUAL mode: gate and
//              up) from the quantised blocks in global memory into shared memory as fp16 in
//              the 128-byte-swizzled K-major layout tcgen05 reads; one of them issues the TMA
//              tile load (cp.async.bulk.tensor, no multicast) of the matching 64-k slice of up
//              to 256 activation rows, which were gathered into expert order beforehand.
//   warp 16    issues tcgen05.mma (M = 128 weight rows, N = pairs, K = 16 per instruction),
//              accumulators in tensor memory; tcgen05.commit releases the stage.
//   warps 17-20 epilogue: tcgen05.ld the accumulators, apply SwiGLU in DUAL mode, store f32.
// Activations arrive already rounded through Q8_K (value = d * q) as fp16, each row divided by a
// power of two that brings its largest value near 2^13 (undone exactly in the epilogue), so the
// result follows the reference CPU path's activation quantisation and cannot overflow fp16;
// weights are rounded to fp16 after the reference dequantiser's f32 arithmetic.
// Every wait is bounded; on expiry the CTA raises the error flag and unwinds, and the
// tensor memory is always released.
#pragma once

#include <cuda.h>

#include "dequant_f16.cuh"
#include "mmid.cuh"

namespace zmoe {

constexpr int GEMM_BM = 128;        // weight rows per tile
constexpr int GEMM_BN = 256;        // pairs per tile (tensor-memory columns per accumulator)
constexpr int GEMM_BK = 64;         // k per stage: one 128-byte swizzle row of bf16
constexpr int GEMM_PRODUCERS = 512;   // 16 warps: the conversion is latency-bound, more warps raise its issue rate
constexpr int GEMM_PWARPS = GEMM_PRODUCERS / 32;
constexpr int GEMM_THREADS = GEMM_PRODUCERS + 32 + 128;
constexpr int GEMM_MAX_ACTIVE = 512;

struct GemmParams {
    const uint8_t *w0, *w1;      // quantised weights (w1: up, DUAL only)
    size_t stride0, stride1;     // bytes between experts
    int I, O;                    // k extent, weight rows per expert (multiple of 128)
    int rb;                      // bytes per weight row
    const float *xscale;         // per SORTED activation row: the power of two the row was divided by
    float *y;                    // output [pair][ldy]
    int ldy;
    const int *hdr, *active, *aoffs, *antok, *slot;   // plan (see router.cuh)
    float clamp;
    int clamp_fused;
    int nstage;
    int *err;
    int *bad;                    // DUAL: [2] counters of NaN / Inf gate or up values, or null
};

// Activation tile maps with boxes of 32, 64, 128 and 256 rows: a tile loads the smallest box that covers
// its pairs, so an expert with few pairs does not pull 256 rows through L2 for every k-step.
struct GemmMaps {
    alignas(64) CUtensorMap box[4];
};

template <int TYPE, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_sm100_kernel(const GemmParams p, const __grid_constant__ GemmMaps maps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_tile_offs[GEMM_MAX_ACTIVE + 1];
    __shared__ __align__(16) uint64_t grid_s[TYPE == IQ2_XXS ? 256 : 2];
    __shared__ __align__(16) uint4 sign_s[TYPE == IQ2_XXS ? 128 : 1];

    // 1024-byte alignment of the operand tiles (required by the 128-byte swizzle)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;           // 16 KB
    constexpr int B_BYTES = GEMM_BN * GEMM_BK * 2;           // 32 KB
    constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
    // DUAL: gate and up accumulators of 256 columns fill the tensor memory; otherwise two
    // 256-column accumulators alternate between tiles so the epilogue overlaps the next tile
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int NACC = DUAL ? 1 : 2;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstage = p.nstage;
    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(&full_bar[s], GEMM_PWARPS + 1);   // one arrival per producer warp + the TMA issuer's expect_tx
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        mbar_init_fence();
    }
    if (warp == GEMM_PWARPS) tmem_alloc(&tmem_slot, TMEM_COLS);
    if (TYPE == IQ2_XXS) dequant_fill_tables(grid_s, sign_s);
    const DequantTables tb{grid_s, sign_s};

    pdl_wait_prior_grid();
    pdl_launch_dependents();

    // tiles: for each active expert, (O / 128) row blocks x ceil(pairs / 256) pair blocks
    const int n_active = min(p.hdr[0], GEMM_MAX_ACTIVE);
    const int mblocks = p.O / GEMM_BM;
    if (tid == 0) {
        int run = 0;
        s_tile_offs[0] = 0;
        for (int a = 0; a < n_active; ++a) {
            run += mblocks * ((p.antok[a] + GEMM_BN - 1) / GEMM_BN);
            s_tile_offs[a + 1] = run;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    const int n_tiles = s_tile_offs[n_active];
    const int ksteps = p.I / GEMM_BK;
    bool alive = true;

    auto tile_info = [&](int tile, int &e, int &m0, int &p0, int &np) {
        int lo = 0, hi = n_active - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_tile_offs[mid] <= tile) lo = mid; else hi = mid - 1;
        }
        const int local = tile - s_tile_offs[lo];
        e = p.active[lo];
        // pair block outermost: the row blocks of one pair block run back to back and reuse
        // the same activation rows from L2
        const int nb = local / mblocks;
        m0 = (local % mblocks) * GEMM_BM;
        // an expert's pairs are split evenly over its pair blocks (300 pairs: 2 x 160, not 256 + 44)
        const int cnt = p.antok[lo], nblk = (cnt + GEMM_BN - 1) / GEMM_BN;
        const int bsz = ((cnt + nblk - 1) / nblk + 15) & ~15;
        p0 = p.aoffs[lo] + nb * bsz;
        np = max(0, min(bsz, cnt - nb * bsz));
    };

    if (warp < GEMM_PWARPS) {
        // ------------------------------- producers -------------------------------------
        int it = 0;  // stage use counter
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            // weights: thread -> (tensor, row r, 32-k half) of the 128 x 64 tile(s); without a second
            // tensor the upper half of the producer threads only takes part in the barriers
            const int which = tid >> 8, r = (tid & 255) >> 1, half = tid & 1;
            const bool worker = DUAL || which == 0;
            const uint8_t *wrow0 = (DUAL && which) ? p.w1 + (size_t)e * p.stride1 + (size_t)(m0 + r) * p.rb
                                                   : p.w0 + (size_t)e * p.stride0 + (size_t)(m0 + r) * p.rb;
            // the loads of k-step ks+1 are issued before k-step ks is converted, so global latency
            // hides behind the conversion work
            RawW<TYPE> r0, n0;
            auto fetch = [&](int ks, RawW<TYPE> &a0) {
                if (worker) load_raw<TYPE>(wrow0, ks * GEMM_BK + 32 * half, a0);
            };
            fetch(0, r0);
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int s = it % nstage;
                if (ks + 1 < ksteps) fetch(ks + 1, n0);
                if (it >= nstage && !mbar_wait(&empty_bar[s], ((it / nstage) - 1) & 1)) {
                    atomicExch(p.err, 3);
                    alive = false;
                    break;
                }
                uint8_t *stage = smem + (size_t)s * STAGE_BYTES;
                const int k0 = ks * GEMM_BK;
                if (tid == 0) {
                    // the activation tile: rows p0 .. p0 + box - 1 of the sorted activations, columns
                    // k0 .. k0+63; rows past the end of the buffer arrive as zeros
                    const int bi = ncols <= 32 ? 0 : ncols <= 64 ? 1 : ncols <= 128 ? 2 : 3;
                    mbar_arrive_expect_tx(&full_bar[s], (uint32_t)((32 << bi) * GEMM_BK * 2));
                    tma_load_2d(stage + (DUAL ? 2 : 1) * A_BYTES, &maps.box[bi], k0, p0, &full_bar[s]);
                }
                if (worker) {
                    uint4 a[4];
                    convert_raw<TYPE>(r0, k0 + 32 * half, tb, a);
                    uint8_t *tile = stage + which * A_BYTES;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4 *>(tile + swz128_offset(r, 32 * half + 8 * c)) = a[c];
                }
                fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_bar[s]);   // one arrival per warp: 512 serialised arrivals would dominate
                r0 = n0;
            }
        }
    } else if (warp == GEMM_PWARPS) {
        // ------------------------------- MMA issuer ------------------------------------
        int it = 0, nt = 0;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++nt) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            const uint32_t idesc = umma_idesc_f16(GEMM_BM, ncols);
            // the epilogue must have drained the previous tile's accumulators
            const int ab = nt % NACC;                       // accumulator buffer of this tile
            const uint32_t acc = tmem_base + (DUAL ? 0 : ab * GEMM_BN);
            if (nt >= NACC && !mbar_wait_sleep(&acc_empty[ab], ((nt / NACC) - 1) & 1, 64)) {
                if (lane == 0) atomicExch(p.err, 4);
                alive = false;
                break;
            }
            tc_fence_after_sync();
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int s = it % nstage;
                if (!mbar_wait_sleep(&full_bar[s], (it / nstage) & 1, 32)) {
                    if (lane == 0) atomicExch(p.err, 5);
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
                if (lane == 0) {
                    fence_proxy_async_smem();
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + (DUAL ? 2 : 1) * A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < GEMM_BK / 16; ++k4) {
                        const uint64_t bd = umma_desc_sw128(sb + 32 * k4);
                        umma_f16(acc, umma_desc_sw128(sa + 32 * k4), bd, idesc, (ks | k4) != 0);
                        if (DUAL) umma_f16(acc + GEMM_BN, umma_desc_sw128(sa + A_BYTES + 32 * k4), bd, idesc, (ks | k4) != 0);
                    }
                    umma_commit(&empty_bar[s]);                 // stage free once these MMAs have read it
                    if (ks == ksteps - 1) umma_commit(&acc_full[ab]);  // accumulators complete
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------- epilogue --------------------------------------
        const int q = warp & 3;              // the warp's quarter of the 128 tensor-memory lanes
        int nt = 0;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++nt) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ab = nt % NACC;
            const uint32_t acc = tmem_base + (DUAL ? 0 : ab * GEMM_BN);
            if (!mbar_wait_sleep(&acc_full[ab], (nt / NACC) & 1, 256)) {
                if (lane == 0) atomicExch(p.err, 6);
                alive = false;
                break;
            }
            tc_fence_after_sync();
            const int f = m0 + 32 * q + lane;   // this thread's weight row
            for (int c0 = 0; c0 < np; c0 += 32) {
                uint32_t g[32], u[32];
                tmem_ld_32x32(acc + ((uint32_t)(32 * q) << 16) + c0, g);
                if (DUAL) tmem_ld_32x32(acc + ((uint32_t)(32 * q) << 16) + GEMM_BN + c0, u);
                // column metadata: lane j fetches pair id and scale of column c0 + j once, the loop
                // below broadcasts them (32 dependent scalar loads per chunk would serialise on latency)
                const int my_pair = c0 + lane < np ? p.slot[p0 + c0 + lane] : 0;
                const float my_sc = c0 + lane < np ? p.xscale[p0 + c0 + lane] : 0.f;
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int pair = __shfl_sync(0xffffffffu, my_pair, j);
                    const float sc = __shfl_sync(0xffffffffu, my_sc, j);
                    if (c0 + j < np) {
                        float v = __uint_as_float(g[j]) * sc;
                        if (DUAL) {
                            const float uv = __uint_as_float(u[j]) * sc;
                            count_bad(p.bad, v, uv);
                            v = swiglu_f(v, uv, p.clamp, p.clamp_fused);
                        }
                        p.y[(size_t)pair * p.ldy + f] = v;
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[ab]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == GEMM_PWARPS) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zmoe
