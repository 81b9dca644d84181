// gemm_sm100.cuh -- prefill-shaped grouped expert GEMM on the 5th-generation tensor
// cores: C[f, p] = sum_k W_e[f, k] * X[p, k] for the pairs p routed to expert e.
//
// Replaces, for calls with many tokens per expert, the GEMV-shaped per-expert loop of
// reference core/batched_dispatch_pipeline.cpp:1833-1921 and the dequantise-to-bf16 +
// cublasGemmEx escape hatch of reference backends/cuda/cuda_kernel_dispatcher.cpp:58-124.
//
// One persistent CTA per SM, warp-specialised.  A tile is 2 x 128 weight rows (DUAL: 128 gate
// rows and the same 128 up rows; otherwise rows m0..m0+127 and m0+128..m0+255 of one matrix)
// against up to 256 pairs; both halves multiply the same activation tile, which halves the
// activation traffic per flop.
//   warp 17    loader: copies the raw quantised super-blocks of the tile's 256 rows, one
//              super-block column (256 k) at a time, into a two-slot ring in shared memory with the
//              TMA engine (one tiled copy per 128 rows where rows are multiples of 16 bytes, else
//              one bulk copy per row; no multicast), completion on mbarriers.
//   warps 0-15 converters: read the raw blocks from shared memory and write them as fp16 in the
//              128-byte-swizzled K-major layout tcgen05 reads, 64 k per pipeline stage; one of
//              them issues the tiled copy of the matching 64-k slice of the activation rows,
//              which were gathered into expert order beforehand.
//   warp 16    issues tcgen05.mma (M = 128 weight rows, N = pairs, K = 16 per instruction) for
//              both halves, accumulators in tensor memory; tcgen05.commit releases the stage.
//   warps 18-21 epilogue: tcgen05.ld the accumulators, apply SwiGLU in DUAL mode, store f32.
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

constexpr int GEMM_BM = 128;        // weight rows per half tile
constexpr int GEMM_BN = 256;        // pairs per tile (tensor-memory columns per accumulator)
constexpr int GEMM_BK = 64;         // k per stage: one 128-byte swizzle row of fp16
constexpr int GEMM_NSTAGE = 2;      // fp16 operand stages
constexpr int GEMM_NRAW = 2;        // raw super-block slots
constexpr int GEMM_CWARPS = 16;     // converter warps
constexpr int GEMM_CONVERTERS = 32 * GEMM_CWARPS;
constexpr int GEMM_THREADS = GEMM_CONVERTERS + 32 + 32 + 128;
constexpr int GEMM_MAX_ACTIVE = 512;

// bytes between the raw copies of consecutive rows in shared memory: room for one super-block plus its
// offset from the 16-byte boundary the copy starts on, and a multiple of 16 that is 16 or 48 modulo 128
// so that the converters' loads (one row per lane pair) spread over the banks
template <int TYPE> struct RawGeom;
template <> struct RawGeom<IQ2_XXS> { static constexpr int kPitch = 80; };    // 66 + 14
template <> struct RawGeom<Q2_K> { static constexpr int kPitch = 112; };      // 84 + 12
template <> struct RawGeom<Q3_K> { static constexpr int kPitch = 144; };      // 110 + 14
template <> struct RawGeom<Q4_K> { static constexpr int kPitch = 144; };      // 144 + 0
__host__ __device__ constexpr int gemm_raw_pitch(int type) {
    return type == IQ2_XXS ? 80 : type == Q2_K ? 112 : 144;
}

struct GemmParams {
    const uint8_t *w0, *w1;      // quantised weights (w1: up, DUAL only)
    size_t stride0, stride1;     // bytes between experts
    int I, O;                    // k extent, weight rows per expert (multiple of 128)
    int rb;                      // bytes per weight row
    int raw_tiled;               // raw blocks come through the tiled maps wmap[] (rows are multiples of 16 bytes)
    const float *xscale;         // per SORTED activation row: the power of two the row was divided by
    float *y;                    // output [pair][ldy]
    int ldy;
    const int *hdr, *active, *aoffs, *antok, *slot;   // plan (see router.cuh)
    float clamp;
    int clamp_fused;
    int *err;
    int *bad;                    // DUAL: [2] counters of NaN / Inf gate or up values, or null
};

// Activation tile maps with boxes of 32, 64, 128 and 256 rows (a tile loads the smallest box that covers
// its pairs, so an expert with few pairs does not pull 256 rows through L2 for every k-step) and the
// byte maps [E][O][rb] of the weight tensors with a box of 128 rows x one raw row pitch.
struct GemmMaps {
    alignas(64) CUtensorMap box[4];
    alignas(64) CUtensorMap wmap[2];
};

// 3-D tiled copy (no multicast): box of the map at (x, row, expert); x must be a multiple of 16 bytes
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void *tmap, int x, int row, int expert, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(row), "r"(expert), "r"(smem_u32(bar))
        : "memory");
}

template <int TYPE, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_sm100_kernel(const GemmParams p, const __grid_constant__ GemmMaps maps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[GEMM_NSTAGE], empty_bar[GEMM_NSTAGE], raw_full[GEMM_NRAW],
        raw_empty[GEMM_NRAW], acc_full, acc_empty;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_tile_offs[GEMM_MAX_ACTIVE + 1];
    __shared__ __align__(16) uint64_t grid_s[TYPE == IQ2_XXS ? 256 : 2];

    // 1024-byte alignment of the operand tiles (required by the 128-byte swizzle)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int BB = QTraits<TYPE>::kBytes;
    constexpr int PITCH = RawGeom<TYPE>::kPitch;
    constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;           // 16 KB per half tile
    constexpr int B_BYTES = GEMM_BN * GEMM_BK * 2;           // 32 KB
    constexpr int STAGE_BYTES = 2 * A_BYTES + B_BYTES;       // 64 KB
    constexpr int RAW_HALF = GEMM_BM * PITCH;                // raw blocks of one half tile
    constexpr int RAW_SLOT = 2 * RAW_HALF;
    constexpr uint32_t TMEM_COLS = 512;                      // two accumulators of 256 columns
    uint8_t *raw_base = smem + GEMM_NSTAGE * STAGE_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < GEMM_NSTAGE; ++s) {
            mbar_init(&full_bar[s], GEMM_CWARPS + 1);   // one arrival per converter warp + the TMA issuer's expect_tx
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < GEMM_NRAW; ++s) {
            mbar_init(&raw_full[s], 1);                 // the loader's expect_tx arrival
            mbar_init(&raw_empty[s], GEMM_CWARPS);
        }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, 128);
        mbar_init_fence();
    }
    if (warp == GEMM_CWARPS) tmem_alloc(&tmem_slot, TMEM_COLS);
    if (TYPE == IQ2_XXS) dequant_fill_tables(grid_s);
    const DequantTables tb{grid_s};

    pdl_wait_prior_grid();
    pdl_launch_dependents();

    // tiles: for each active expert, row blocks x ceil(pairs / 256) pair blocks
    const int n_active = min(p.hdr[0], GEMM_MAX_ACTIVE);
    const int mstep = DUAL ? GEMM_BM : 2 * GEMM_BM;          // rows of one matrix a tile covers
    const int mblocks = (p.O + mstep - 1) / mstep;
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
    const int nblk = p.I / QK_K;
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
        m0 = (local % mblocks) * mstep;
        // an expert's pairs are split evenly over its pair blocks (300 pairs: 2 x 160, not 256 + 44)
        const int cnt = p.antok[lo], npb = (cnt + GEMM_BN - 1) / GEMM_BN;
        const int bsz = ((cnt + npb - 1) / npb + 15) & ~15;
        p0 = p.aoffs[lo] + nb * bsz;
        np = max(0, min(bsz, cnt - nb * bsz));
    };
    // first byte of row r (0..127) of half h of the tile in global memory
    auto half_row = [&](int h, int e, int m0, int r) -> const uint8_t * {
        if (DUAL) return (h ? p.w1 + (size_t)e * p.stride1 : p.w0 + (size_t)e * p.stride0) + (size_t)(m0 + r) * p.rb;
        return p.w0 + (size_t)e * p.stride0 + (size_t)(m0 + GEMM_BM * h + r) * p.rb;
    };
    // the second half of a tile exists unless the matrix ends after the first (rows a multiple of 128, not 256)
    auto has_half1 = [&](int m0) -> bool { return DUAL || m0 + GEMM_BM < p.O; };

    if (warp < GEMM_CWARPS) {
        // ------------------------------- converters ------------------------------------
        int it = 0;   // fp16 stage use counter
        int rc = 0;   // raw slot use counter
        // thread -> (half tile, row r, 32-k half of the stage)
        const int which = tid >> 8, r = (tid & 255) >> 1, half = tid & 1;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            const bool worker = which == 0 || has_half1(m0);
            const uint8_t *grow = half_row(which, e, m0, r);
            uint32_t blk = 0;
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int s = it % GEMM_NSTAGE;
                const int rs = rc % GEMM_NRAW;
                if ((ks & 3) == 0) {
                    // a new super-block column: its raw copy must have landed
                    if (!mbar_wait(&raw_full[rs], (rc / GEMM_NRAW) & 1)) {
                        atomicExch(p.err, 7);
                        alive = false;
                        break;
                    }
                    const uint32_t off = (uint32_t)(reinterpret_cast<uintptr_t>(grow + (size_t)(ks >> 2) * BB) & 15u);
                    blk = smem_u32(raw_base) + rs * RAW_SLOT + which * RAW_HALF + r * PITCH + off;
                }
                if (it >= GEMM_NSTAGE && !mbar_wait(&empty_bar[s], ((it / GEMM_NSTAGE) - 1) & 1)) {
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
                    tma_load_2d(stage + 2 * A_BYTES, &maps.box[bi], k0, p0, &full_bar[s]);
                }
                if (worker) {
                    RawW<TYPE> raw;
                    load_raw_s<TYPE>(blk, (k0 & 255) + 32 * half, raw);
                    uint4 a[4];
                    convert_raw<TYPE>(raw, k0 + 32 * half, tb, a);
                    uint8_t *tile_s = stage + which * A_BYTES;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4 *>(tile_s + swz128_offset(r, 32 * half + 8 * c)) = a[c];
                }
                fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full_bar[s]);   // one arrival per warp
                    if ((ks & 3) == 3) mbar_arrive(&raw_empty[rs]);   // this warp is done with the raw slot
                }
                if ((ks & 3) == 3) ++rc;
            }
        }
    } else if (warp == GEMM_CWARPS) {
        // ------------------------------- MMA issuer ------------------------------------
        int it = 0, nt = 0;
        // operand descriptors of the two stages; a k-step of 16 elements advances the start address by 32 bytes
        static_assert(GEMM_NSTAGE == 2, "descriptor registers are laid out for two stages");
        const uint32_t sa0 = smem_u32(smem), sa1 = sa0 + STAGE_BYTES;
        const uint64_t d0a0 = umma_desc_sw128(sa0), d0a1 = umma_desc_sw128(sa0 + A_BYTES), d0b = umma_desc_sw128(sa0 + 2 * A_BYTES);
        const uint64_t d1a0 = umma_desc_sw128(sa1), d1a1 = umma_desc_sw128(sa1 + A_BYTES), d1b = umma_desc_sw128(sa1 + 2 * A_BYTES);
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++nt) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            const uint32_t idesc = umma_idesc_f16(GEMM_BM, ncols);
            const bool two = has_half1(m0);
            // the epilogue must have drained the previous tile's accumulators
            if (nt >= 1 && !mbar_wait_sleep(&acc_empty, (nt - 1) & 1, 64)) {
                if (lane == 0) atomicExch(p.err, 4);
                alive = false;
                break;
            }
            tc_fence_after_sync();
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int s = it % GEMM_NSTAGE;
                if (!mbar_wait(&full_bar[s], (it / GEMM_NSTAGE) & 1, 1u << 22)) {
                    if (lane == 0) atomicExch(p.err, 5);
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint64_t a0 = s ? d1a0 : d0a0, a1 = s ? d1a1 : d0a1, b0 = s ? d1b : d0b;
#pragma unroll
                    for (int k4 = 0; k4 < GEMM_BK / 16; ++k4) {
                        umma_f16(tmem_base, a0 + 2 * k4, b0 + 2 * k4, idesc, (ks | k4) != 0);
                        if (two) umma_f16(tmem_base + GEMM_BN, a1 + 2 * k4, b0 + 2 * k4, idesc, (ks | k4) != 0);
                    }
                    umma_commit(&empty_bar[s]);                 // stage free once these MMAs have read it
                    if (ks == ksteps - 1) umma_commit(&acc_full);  // accumulators complete
                }
                __syncwarp();
            }
        }
    } else if (warp == GEMM_CWARPS + 1) {
        // ------------------------------- raw loader ------------------------------------
        int rc = 0;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const bool two = has_half1(m0);
            for (int b = 0; b < nblk; ++b, ++rc) {
                const int rs = rc % GEMM_NRAW;
                if (rc >= GEMM_NRAW && !mbar_wait_sleep(&raw_empty[rs], ((rc / GEMM_NRAW) - 1) & 1, 32, 1u << 20)) {
                    if (lane == 0) atomicExch(p.err, 8);
                    alive = false;
                    break;
                }
                const uint32_t dst = smem_u32(raw_base) + rs * RAW_SLOT;
                if (p.raw_tiled) {
                    // rows are multiples of 16 bytes: every row's block starts at the same offset from a
                    // 16-byte boundary; one box of 128 rows x PITCH bytes per half tile (bytes past the
                    // end of a row arrive as zeros and are never read)
                    if (lane == 0) {
                        const int x = (b * BB) & ~15;
                        mbar_arrive_expect_tx(&raw_full[rs], (uint32_t)((two ? 2 : 1) * RAW_HALF));
                        tma_load_3d(dst, &maps.wmap[0], x, m0, e, &raw_full[rs]);
                        if (two) tma_load_3d(dst + RAW_HALF, &maps.wmap[DUAL ? 1 : 0], x, DUAL ? m0 : m0 + GEMM_BM, e, &raw_full[rs]);
                    }
                } else {
                    // one bulk copy per row, from the 16-byte boundary at or below the block's first byte
                    // to the one at or above its last (the tensor ends on such a boundary)
                    uint32_t bytes = 0;
#pragma unroll 4
                    for (int i = 0; i < 8; ++i) {
                        const int idx = lane + 32 * i, h = idx >> 7, r = idx & 127;
                        if (h == 0 || two) {
                            const uint8_t *src = half_row(h, e, m0, r) + (size_t)b * BB;
                            const uint32_t off = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15u);
                            const uint32_t sz = (off + BB + 15u) & ~15u;
                            bulk_g2s_addr(dst + h * RAW_HALF + r * PITCH, src - off, sz, &raw_full[rs]);
                            bytes += sz;
                        }
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
                    // the copies above cannot complete the phase before this arrival registers their bytes
                    if (lane == 0) mbar_arrive_expect_tx(&raw_full[rs], bytes);
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
            const bool two = has_half1(m0);
            if (!mbar_wait_sleep(&acc_full, nt & 1, 256)) {
                if (lane == 0) atomicExch(p.err, 6);
                alive = false;
                break;
            }
            tc_fence_after_sync();
            const int f = m0 + 32 * q + lane;   // this thread's weight row (first half)
            const uint32_t tl = tmem_base + ((uint32_t)(32 * q) << 16);
            for (int c0 = 0; c0 < np; c0 += 32) {
                uint32_t g[32], u[32];
                tmem_ld_32x32(tl + c0, g);
                if (two) tmem_ld_32x32(tl + GEMM_BN + c0, u);
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
                        const float v = __uint_as_float(g[j]) * sc;
                        float *row = p.y + (size_t)pair * p.ldy;
                        if (DUAL) {
                            const float uv = __uint_as_float(u[j]) * sc;
                            count_bad(p.bad, v, uv);
                            row[f] = swiglu_f(v, uv, p.clamp, p.clamp_fused);
                        } else {
                            row[f] = v;
                            if (two) row[f + GEMM_BM] = __uint_as_float(u[j]) * sc;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == GEMM_CWARPS) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zmoe
