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
//              super-block column (256 k) at a time, into a two-slot ring in shared memory with
//              tiled copies on the TMA engine (no multicast), completion on mbarriers.  Rows that are
//              not multiples of 16 bytes are addressed G rows at a time (G * row bytes is one): G
//              copies per 128 rows, one per position of a row inside its group.
//   warps 0-15 converters: read the raw blocks from shared memory and write them as fp16 in the
//              128-byte-swizzled K-major layout tcgen05 reads, 64 k per pipeline stage; one of
//              them issues the tiled copy of the matching 64-k slice of the activation rows,
//              which were gathered into expert order beforehand.  The same warps drain the
//              accumulators of a finished tile (tcgen05.ld, SwiGLU in DUAL mode, f32 stores): both
//              accumulators fill the tensor memory, so the next tile's MMAs wait for the drain, and
//              sixteen warps (four per quarter of the tensor-memory lanes, two 32-column chunks each)
//              finish it in a quarter of the time four dedicated warps need.  The drain of tile t runs
//              after the first stage of tile t+1 has been converted, when tile t's last MMAs are done.
//   warp 16    issues tcgen05.mma (M = 128 weight rows, N = pairs, K = 16 per instruction) for
//              both halves, accumulators in tensor memory; tcgen05.commit releases the stage.
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
constexpr int GEMM_THREADS = GEMM_CONVERTERS + 32 + 32;
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
    int g_log2;                  // log2 of G, the rows per group whose bytes are a multiple of 16 (1, 2, 4 or 8 rows)
    const float *xscale;         // per SORTED activation row: the power of two the row was divided by
    float *y;                    // output [pair][ldy]
    int ldy;
    const int *hdr, *active, *aoffs, *antok, *slot;   // plan (see router.cuh)
    float clamp;
    int clamp_fused;
    int *err;
    int *bad;                    // DUAL: [2] counters of NaN / Inf gate or up values, or null
    unsigned long long *stats;   // cycle counters of CTA 0's roles (builds with ZMOE_GEMM_STATS only), or null
};

// Cycle accounting of one CTA's roles, compiled in with -DZMOE_GEMM_STATS (python -m zeromoe_b200.build with
// ZMOE_GEMM_STATS=1 in the environment): one thread per role of CTA 0 adds up clock64() differences around
// its waits and its work and stores the sums when the kernel ends.  Slots: 0 stages converted, 1 converter
// wait for raw blocks, 2 converter wait for a free stage, 3 load + convert + store, 4 fence + arrive,
// 5 MMA wait for a full stage, 6 MMA issue + commit, 7 MMA wait for the accumulators, 8 epilogue wait,
// 9 epilogue work, 10 loader wait for a free slot, 11 loader issue, 12 tiles.
#ifdef ZMOE_GEMM_STATS
#define GSTAT_DECL unsigned long long gs_t0 = 0, gs_acc[4] = {0, 0, 0, 0}; const bool gs_on = blockIdx.x == 0 && p.stats != nullptr
#define GSTAT_BEGIN() do { if (gs_on) gs_t0 = clock64(); } while (0)
#define GSTAT_END(i) do { if (gs_on) { const unsigned long long gs_t1 = clock64(); gs_acc[i] += gs_t1 - gs_t0; gs_t0 = gs_t1; } } while (0)
#define GSTAT_STORE(i, slot) do { if (gs_on) p.stats[slot] += gs_acc[i]; } while (0)
#else
#define GSTAT_DECL do { } while (0)
#define GSTAT_BEGIN() do { } while (0)
#define GSTAT_END(i) do { } while (0)
#define GSTAT_STORE(i, slot) do { } while (0)
#endif

// Activation tile maps with boxes of 32, 64, 128 and 256 rows (a tile loads the smallest box that covers
// its pairs, so an expert with few pairs does not pull 256 rows through L2 for every k-step) and the
// byte maps [E][O / G][G * rb] of the weight tensors with a box of 128 / G row groups x one raw row pitch.
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
    __shared__ __align__(16) uint2 grid_s[TYPE == IQ2_XXS ? 256 * IQ2_TABLE_COPIES : 2];

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
        mbar_init(&acc_empty, GEMM_CWARPS);
        mbar_init_fence();
    }
    if (warp == GEMM_CWARPS) tmem_alloc(&tmem_slot, TMEM_COLS);
    if (TYPE == IQ2_XXS) dequant_fill_tables(grid_s);
    const DequantTables tb{smem_u32(grid_s)};

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
    // the second half of a tile exists unless the matrix ends after the first (rows a multiple of 128, not 256)
    auto has_half1 = [&](int m0) -> bool { return DUAL || m0 + GEMM_BM < p.O; };

    if (warp < GEMM_CWARPS) {
        // ------------------------------- converters ------------------------------------
        int it = 0;   // fp16 stage use counter
        int rc = 0;   // raw slot use counter
        // thread -> (half tile, row r, 32-k half of the stage)
        const int which = tid >> 8, r = (tid & 255) >> 1, half = tid & 1;
        // where this thread's four 16-byte chunks go inside a stage (fixed for the whole kernel)
        const uint32_t stage0 = smem_u32(smem);
        uint32_t st_off[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) st_off[c] = which * A_BYTES + swz128_offset(r, 32 * half + 8 * c);
        GSTAT_DECL;
        // ---- drain of a finished tile's accumulators (all converter warps) ----
        // warp w reads its quarter q = w % 4 of the tensor-memory lanes (rows) and the 32-column chunks
        // w / 4 and w / 4 + 4 of the tile's pairs; lane j of a chunk's metadata holds column 32 c + j
        const int q = warp & 3, cset = warp >> 2;
        const uint32_t tl = tmem_base + ((uint32_t)(32 * q) << 16);
        int nt = 0;                      // tiles converted so far
        int d_m0 = 0, d_np = 0;          // the tile waiting for its drain
        bool d_two = false;
        int d_pair[2] = {-1, -1};
        float d_sc[2] = {0.f, 0.f};
        auto drain = [&]() -> bool {
#ifdef ZMOE_GEMM_STATS
            unsigned long long e_t0 = 0;
            if (gs_on) e_t0 = clock64();
#endif
            if (!mbar_wait_suspend(&acc_full, (nt - 1) & 1)) return false;
            tc_fence_after_sync();
#ifdef ZMOE_GEMM_STATS
            if (gs_on && tid == 32) { const unsigned long long t1 = clock64(); p.stats[8] += t1 - e_t0; e_t0 = t1; }
#endif
            const int f = d_m0 + 32 * q + lane;   // this thread's weight row (first half)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int c0 = 32 * (cset + 4 * i);
                if (c0 >= d_np) break;
                uint32_t g[32], u[32];
                tmem_ld_32x32(tl + c0, g);
                if (d_two) tmem_ld_32x32(tl + GEMM_BN + c0, u);
                const int my_pair = d_pair[i];
                const float my_sc = d_sc[i];
                tmem_ld_wait();
                // the arithmetic of all 32 columns first, without branches, so that the columns' dependency
                // chains interleave; x - x is 0 for a finite x and NaN otherwise: the sum flags a non-finite
                // gate / up value
                float probe = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float sc = __shfl_sync(0xffffffffu, my_sc, j);
                    const float gv = __uint_as_float(g[j]) * sc;
                    if (DUAL) {
                        const float uv = __uint_as_float(u[j]) * sc;
                        probe += (gv - gv) + (uv - uv);
                        g[j] = __float_as_uint(swiglu_fast(gv, uv, p.clamp, p.clamp_fused));
                    } else {
                        g[j] = __float_as_uint(gv);
                        if (d_two) u[j] = __float_as_uint(__uint_as_float(u[j]) * sc);
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int pair = __shfl_sync(0xffffffffu, my_pair, j);
                    if (pair >= 0) {
                        float *row = p.y + (size_t)pair * p.ldy;
                        row[f] = __uint_as_float(g[j]);
                        if (!DUAL && d_two) row[f + GEMM_BM] = __uint_as_float(u[j]);
                    }
                }
                // warp-uniform decision: the loads and shuffles below are warp-collective
                if (DUAL && p.bad && __any_sync(0xffffffffu, probe != probe)) {
                    // rare: recount this chunk's non-finite inputs exactly
                    for (int j = 0; j < 32; ++j) {
                        const float sc = __shfl_sync(0xffffffffu, my_sc, j);
                        uint32_t gj, uj;
                        tmem_ld_1(tl + c0 + j, gj);
                        tmem_ld_1(tl + GEMM_BN + c0 + j, uj);
                        tmem_ld_wait();
                        if (c0 + j < d_np) count_bad(p.bad, __uint_as_float(gj) * sc, __uint_as_float(uj) * sc);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
#ifdef ZMOE_GEMM_STATS
            if (gs_on && tid == 32) p.stats[9] += clock64() - e_t0;
#endif
            return true;
        };
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++nt) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            const bool worker = which == 0 || has_half1(m0);
            // pair ids and scales of this warp's two column chunks: fetched now, used by the drain much later
            int n_pair[2];
            float n_sc[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int col = 32 * (cset + 4 * i) + lane;
                n_pair[i] = col < np ? p.slot[p0 + col] : -1;
                n_sc[i] = col < np ? p.xscale[p0 + col] : 0.f;
            }
            uint32_t blk = 0;
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                // the previous tile's accumulators: its last MMAs finish while this tile's first stage is converted
                if (ks == 1 && nt > 0 && !drain()) {
                    atomicExch(p.err, 6);
                    alive = false;
                    break;
                }
                const int s = it % GEMM_NSTAGE;
                const int rs = rc % GEMM_NRAW;
                GSTAT_BEGIN();
                if ((ks & 3) == 0) {
                    // a new super-block column: its raw copy must have landed
                    if (!mbar_wait_suspend(&raw_full[rs], (rc / GEMM_NRAW) & 1)) {
                        atomicExch(p.err, 7);
                        alive = false;
                        break;
                    }
                    // row r = G * sr + j sits in sub-array j (the copy of position j of every group) at sr
                    const int G = 1 << p.g_log2, j = r & (G - 1), sr = r >> p.g_log2;
                    const uint32_t off = (uint32_t)(j * p.rb + (ks >> 2) * BB) & 15u;
                    blk = smem_u32(raw_base) + rs * RAW_SLOT + which * RAW_HALF + (j * (GEMM_BM >> p.g_log2) + sr) * PITCH + off;
                }
                GSTAT_END(0);
                if (it >= GEMM_NSTAGE && !mbar_wait_suspend(&empty_bar[s], ((it / GEMM_NSTAGE) - 1) & 1)) {
                    atomicExch(p.err, 3);
                    alive = false;
                    break;
                }
                GSTAT_END(1);
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
                    const uint32_t sbase = stage0 + s * STAGE_BYTES;
#pragma unroll
                    for (int c = 0; c < 4; ++c) sts128(sbase + st_off[c], a[c]);
                }
                GSTAT_END(2);
                fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full_bar[s]);   // one arrival per warp
                    if ((ks & 3) == 3) mbar_arrive(&raw_empty[rs]);   // this warp is done with the raw slot
                }
                if ((ks & 3) == 3) ++rc;
                GSTAT_END(3);
            }
            d_m0 = m0; d_np = np; d_two = has_half1(m0);
            d_pair[0] = n_pair[0]; d_pair[1] = n_pair[1];
            d_sc[0] = n_sc[0]; d_sc[1] = n_sc[1];
        }
        if (alive && nt > 0 && !drain()) atomicExch(p.err, 6);
#ifdef ZMOE_GEMM_STATS
        if (tid == 32) {
            if (gs_on) p.stats[0] += (unsigned long long)it;
            GSTAT_STORE(0, 1); GSTAT_STORE(1, 2); GSTAT_STORE(2, 3); GSTAT_STORE(3, 4);
        }
#endif
    } else if (warp == GEMM_CWARPS) {
        // ------------------------------- MMA issuer ------------------------------------
        int it = 0, nt = 0;
        // operand descriptors of the two stages; a k-step of 16 elements advances the start address by 32 bytes
        static_assert(GEMM_NSTAGE == 2, "descriptor registers are laid out for two stages");
        const uint32_t sa0 = smem_u32(smem), sa1 = sa0 + STAGE_BYTES;
        const uint64_t d0a0 = umma_desc_sw128(sa0), d0a1 = umma_desc_sw128(sa0 + A_BYTES), d0b = umma_desc_sw128(sa0 + 2 * A_BYTES);
        const uint64_t d1a0 = umma_desc_sw128(sa1), d1a1 = umma_desc_sw128(sa1 + A_BYTES), d1b = umma_desc_sw128(sa1 + 2 * A_BYTES);
        GSTAT_DECL;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++nt) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const int ncols = (np + 15) & ~15;
            const uint32_t idesc = umma_idesc_f16(GEMM_BM, ncols);
            const bool two = has_half1(m0);
            GSTAT_BEGIN();
            // the epilogue must have drained the previous tile's accumulators
            if (nt >= 1 && !mbar_wait_suspend(&acc_empty, (nt - 1) & 1)) {
                if (lane == 0) atomicExch(p.err, 4);
                alive = false;
                break;
            }
            GSTAT_END(2);
            tc_fence_after_sync();
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int s = it % GEMM_NSTAGE;
                GSTAT_BEGIN();
                if (!mbar_wait_suspend(&full_bar[s], (it / GEMM_NSTAGE) & 1)) {
                    if (lane == 0) atomicExch(p.err, 5);
                    alive = false;
                    break;
                }
                GSTAT_END(0);
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
                GSTAT_END(1);
            }
        }
#ifdef ZMOE_GEMM_STATS
        if (lane == 0) { GSTAT_STORE(0, 5); GSTAT_STORE(1, 6); GSTAT_STORE(2, 7); if (gs_on) p.stats[12] += (unsigned long long)nt; }
#endif
    } else if (warp == GEMM_CWARPS + 1) {
        // ------------------------------- raw loader ------------------------------------
        int rc = 0;
        GSTAT_DECL;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
            int e, m0, p0, np;
            tile_info(tile, e, m0, p0, np);
            const bool two = has_half1(m0);
            for (int b = 0; b < nblk; ++b, ++rc) {
                const int rs = rc % GEMM_NRAW;
                GSTAT_BEGIN();
                if (rc >= GEMM_NRAW && !mbar_wait_suspend(&raw_empty[rs], ((rc / GEMM_NRAW) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.err, 8);
                    alive = false;
                    break;
                }
                GSTAT_END(0);
                const uint32_t dst = smem_u32(raw_base) + rs * RAW_SLOT;
                // G tiled copies per half tile: copy j brings, for each of the 128 / G row groups, the window
                // of PITCH bytes that holds block b of the group's row j (it starts on the 16-byte boundary at or
                // below the block; bytes past the end of a group arrive as zeros and are never read)
                const int G = 1 << p.g_log2;
                if (lane == 0) mbar_arrive_expect_tx(&raw_full[rs], (uint32_t)((two ? 2 : 1) * RAW_HALF));
                __syncwarp();
                if (lane < 2 * G && (lane < G || two)) {
                    const int h = lane >= G, j = lane & (G - 1);
                    const int x = (j * p.rb + b * BB) & ~15;
                    const int row0 = (DUAL || h == 0) ? m0 : m0 + GEMM_BM;
                    tma_load_3d(dst + h * RAW_HALF + j * (GEMM_BM >> p.g_log2) * PITCH, &maps.wmap[DUAL ? h : 0], x,
                                row0 >> p.g_log2, e, &raw_full[rs]);
                }
                __syncwarp();
                GSTAT_END(1);
            }
        }
#ifdef ZMOE_GEMM_STATS
        if (lane == 0) { GSTAT_STORE(0, 10); GSTAT_STORE(1, 11); }
#endif
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == GEMM_CWARPS) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zmoe
