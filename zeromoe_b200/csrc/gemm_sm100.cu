// gemm_sm100.cu -- launchers of the prefill path: Q8_K round trip of activations to fp16 and
// the tcgen05 grouped GEMM.
#include <map>
#include <mutex>
#include <utility>

#include "gemm_sm100.cuh"
#include "zmoe_internal.h"

namespace zmoe {

// Sorted row s of the output is source row slot[s] / xdiv of x, passed through the Q8_K round
// trip: fp16(d * q / scale[s]) with (d, q) the Q8_K quantisation of each 256-block (same rule as
// q8k.cuh: the value the reference CPU path multiplies with) and scale[s] the power of two that
// puts the row's largest magnitude in [2^13, 2^14).  This is the token-to-expert gather of
// reference core/batched_dispatch_pipeline.cpp:1661-1671 done on the device: afterwards every
// expert's activation rows are contiguous.  One CTA per row, one warp per block.
constexpr int RT_MAXB = 4;   // blocks per warp: rows up to 8192 elements
__global__ void __launch_bounds__(256) q8_roundtrip_f16_kernel(const float *__restrict__ x, int ldx,
                                                               __half *__restrict__ out, float *__restrict__ scale,
                                                               const int *__restrict__ hdr,
                                                               const int *__restrict__ slot, int xdiv, int I) {
    __shared__ float s_max[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int nb = I / QK_K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = hdr[3];   // pairs with a valid expert
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const int srow = slot[r] / xdiv;
        float o[RT_MAXB][8];
        float wmax = 0.f;
#pragma unroll
        for (int i = 0; i < RT_MAXB; ++i) {
            const int b = warp + 8 * i;
            if (b >= nb) break;
            const float *src = x + (size_t)srow * ldx + QK_K * b + 8 * lane;
            const float4 v0 = *reinterpret_cast<const float4 *>(src), v1 = *reinterpret_cast<const float4 *>(src + 4);
            const float xv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            float amax = 0.f, mx = 0.f;
            int id = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float ax = fabsf(xv[j]);
                if (ax > amax) { amax = ax; mx = xv[j]; id = 8 * lane + j; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, amax, off), om = __shfl_xor_sync(0xffffffffu, mx, off);
                const int oi = __shfl_xor_sync(0xffffffffu, id, off);
                if (oa > amax || (oa == amax && oi < id)) { amax = oa; mx = om; id = oi; }
            }
            if (amax == 0.f) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[i][j] = 0.f;
            } else {
                const float iscale = __fdiv_rn(-127.f, mx), d = __fdiv_rn(1.f, iscale);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    o[i][j] = __fmul_rn(d, (float)min(127, __float2int_rn(__fmul_rn(iscale, xv[j]))));
            }
            wmax = fmaxf(wmax, amax);   // |d*q| <= amax up to rounding
        }
        __syncthreads();
        if (lane == 0) s_max[warp] = wmax;
        __syncthreads();
        float rmax = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) rmax = fmaxf(rmax, s_max[w]);
        // power of two sc with rmax / sc in [2^13, 2^14); 1 for an all-zero or non-finite row
        float sc = 1.f;
        if (rmax > 0.f && rmax < 3.0e38f) {
            int ex;
            frexpf(rmax, &ex);              // rmax = m * 2^ex, m in [0.5, 1)
            sc = ldexpf(1.f, ex - 14);
        }
        const float inv = 1.f / sc;
        if (threadIdx.x == 0) scale[r] = sc;
#pragma unroll
        for (int i = 0; i < RT_MAXB; ++i) {
            const int b = warp + 8 * i;
            if (b >= nb) break;
            uint4 pk;
            pk.x = pack_f16x2(o[i][0] * inv, o[i][1] * inv); pk.y = pack_f16x2(o[i][2] * inv, o[i][3] * inv);
            pk.z = pack_f16x2(o[i][4] * inv, o[i][5] * inv); pk.w = pack_f16x2(o[i][6] * inv, o[i][7] * inv);
            *reinterpret_cast<uint4 *>(out + (size_t)r * I + QK_K * b + 8 * lane) = pk;
        }
    }
}

// The same for the layer input, where the K pairs of a token share one source row: one CTA per token
// passes the row through Q8_K once and writes it to the K positions of the token's pairs in expert order
// (pos[t * K + k], -1 for an inactive route).
__global__ void __launch_bounds__(256) q8_roundtrip_tokens_kernel(const float *__restrict__ x, int ldx,
                                                                  __half *__restrict__ out, float *__restrict__ scale,
                                                                  const int *__restrict__ pos, int T, int K, int I) {
    __shared__ float s_max[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int nb = I / QK_K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        float o[RT_MAXB][8];
        float wmax = 0.f;
#pragma unroll
        for (int i = 0; i < RT_MAXB; ++i) {
            const int b = warp + 8 * i;
            if (b >= nb) break;
            const float *src = x + (size_t)t * ldx + QK_K * b + 8 * lane;
            const float4 v0 = *reinterpret_cast<const float4 *>(src), v1 = *reinterpret_cast<const float4 *>(src + 4);
            const float xv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            float amax = 0.f, mx = 0.f;
            int id = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float ax = fabsf(xv[j]);
                if (ax > amax) { amax = ax; mx = xv[j]; id = 8 * lane + j; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, amax, off), om = __shfl_xor_sync(0xffffffffu, mx, off);
                const int oi = __shfl_xor_sync(0xffffffffu, id, off);
                if (oa > amax || (oa == amax && oi < id)) { amax = oa; mx = om; id = oi; }
            }
            if (amax == 0.f) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[i][j] = 0.f;
            } else {
                const float iscale = __fdiv_rn(-127.f, mx), d = __fdiv_rn(1.f, iscale);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    o[i][j] = __fmul_rn(d, (float)min(127, __float2int_rn(__fmul_rn(iscale, xv[j]))));
            }
            wmax = fmaxf(wmax, amax);
        }
        __syncthreads();
        if (lane == 0) s_max[warp] = wmax;
        __syncthreads();
        float rmax = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) rmax = fmaxf(rmax, s_max[w]);
        float sc = 1.f;
        if (rmax > 0.f && rmax < 3.0e38f) {
            int ex;
            frexpf(rmax, &ex);
            sc = ldexpf(1.f, ex - 14);
        }
        const float inv = 1.f / sc;
        uint4 pk[RT_MAXB];
#pragma unroll
        for (int i = 0; i < RT_MAXB; ++i) {
            pk[i].x = pack_f16x2(o[i][0] * inv, o[i][1] * inv); pk[i].y = pack_f16x2(o[i][2] * inv, o[i][3] * inv);
            pk[i].z = pack_f16x2(o[i][4] * inv, o[i][5] * inv); pk[i].w = pack_f16x2(o[i][6] * inv, o[i][7] * inv);
        }
        for (int k = 0; k < K; ++k) {
            const int r = pos[(size_t)t * K + k];
            if (r < 0) continue;
            if (threadIdx.x == 0) scale[r] = sc;
#pragma unroll
            for (int i = 0; i < RT_MAXB; ++i) {
                const int b = warp + 8 * i;
                if (b >= nb) break;
                *reinterpret_cast<uint4 *>(out + (size_t)r * I + QK_K * b + 8 * lane) = pk[i];
            }
        }
    }
}

int launch_q8_roundtrip_tokens_f16(const float *x, int ldx, void *out_f16, float *scale, const PlanBuffers &plan,
                                   int T, int K, int I, cudaStream_t st) {
    if (T <= 0) return ZMOE_OK;
    if (I / QK_K > 8 * RT_MAXB || !plan.pos) return ZMOE_ERR_SHAPE;
    const int cap = 8 * device_sm_count();
    const int grid = T < cap ? T : cap;
    return launch_pdl(q8_roundtrip_tokens_kernel, dim3((unsigned)grid), dim3(256), 0, st, x, ldx,
                      static_cast<__half *>(out_f16), scale, (const int *)plan.pos, T, K, I) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

int launch_q8_roundtrip_f16(const float *x, int ldx, void *out_f16, float *scale, const PlanBuffers &plan,
                            int max_rows, int xdiv, int I, cudaStream_t st) {
    if (max_rows <= 0) return ZMOE_OK;
    if (I / QK_K > 8 * RT_MAXB) return ZMOE_ERR_SHAPE;
    const int cap = 8 * device_sm_count();
    const int grid = max_rows < cap ? max_rows : cap;
    return launch_pdl(q8_roundtrip_f16_kernel, dim3((unsigned)grid), dim3(256), 0, st, x, ldx,
                      static_cast<__half *>(out_f16), scale, (const int *)plan.hdr, (const int *)plan.slot, xdiv,
                      I) == cudaSuccess
               ? ZMOE_OK
               : ZMOE_ERR_CUDA;
}

bool gemm_sm100_supported(int type, int I, int O) {
    return block_bytes(type) != 0 && I > 0 && O > 0 && I % QK_K == 0 && O % GEMM_BM == 0;
}

using GemmFn = void (*)(const GemmParams, const GemmMaps);

// Cycle counters of the instrumented build (see GSTAT_* in gemm_sm100.cuh): two sets of 16 counters on the
// current device, the first for gate / up launches, the second for down launches; null in normal builds.
#ifdef ZMOE_GEMM_STATS
static unsigned long long *g_stats_dev[64] = {};
unsigned long long *gemm_stats_buffer(int which) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_stats_dev[dev]) {
        if (cudaMalloc(reinterpret_cast<void **>(&g_stats_dev[dev]), 32 * sizeof(unsigned long long)) != cudaSuccess) return nullptr;
        cudaMemset(g_stats_dev[dev], 0, 32 * sizeof(unsigned long long));
    }
    return g_stats_dev[dev] + 16 * which;
}
int gemm_stats_read(unsigned long long *out32) {
    unsigned long long *b = gemm_stats_buffer(0);
    if (!b) return ZMOE_ERR_CUDA;
    if (cudaMemcpy(out32, b, 32 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return ZMOE_ERR_CUDA;
    cudaMemset(b, 0, 32 * sizeof(unsigned long long));
    return ZMOE_OK;
}
#else
unsigned long long *gemm_stats_buffer(int) { return nullptr; }
int gemm_stats_read(unsigned long long *out32) {
    for (int i = 0; i < 32; ++i) out32[i] = 0;
    return ZMOE_ERR_STATE;
}
#endif

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link against libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// fp16 matrix [rows, cols] row-major, box 64 columns x box_rows rows, 128-byte swizzle
static int make_x_map(CUtensorMap *m, const void *base, int rows, int cols, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ZMOE_ERR_CUDA;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ZMOE_OK : ZMOE_ERR_CUDA;
}

// Quantised weights as bytes, G rows at a time so that a "row" of the map (G * rb bytes) is a multiple of
// 16: dims [E][O / G][G * rb], box = 128 / G row groups x `pitch` bytes of one expert.
static int make_w_map(CUtensorMap *m, const void *base, int E, int O, int rb, size_t expert_stride, int pitch, int G) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ZMOE_ERR_CUDA;
    if ((G * rb) % 16 || expert_stride % 16 || pitch % 16 || pitch > 256 || O % G || GEMM_BM % G) return ZMOE_ERR_SHAPE;
    const cuuint64_t dims[3] = {(cuuint64_t)G * rb, (cuuint64_t)(O / G), (cuuint64_t)E};
    const cuuint64_t strides[2] = {(cuuint64_t)G * rb, (cuuint64_t)expert_stride};
    const cuuint32_t box[3] = {(cuuint32_t)pitch, (cuuint32_t)(GEMM_BM / G), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ZMOE_OK : ZMOE_ERR_CUDA;
}

int make_rows_map(CUtensorMap *m, const void *base, int E, int O, int rb, size_t expert_stride, int R) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ZMOE_ERR_CUDA;
    // rows as 8-byte elements: a box row is one contiguous run, two elements longer than the row
    if (rb % 16 || expert_stride % 16 || rb / 8 + 2 > 256 || R > 256) return ZMOE_ERR_SHAPE;
    const cuuint64_t dims[3] = {(cuuint64_t)(rb / 8), (cuuint64_t)O, (cuuint64_t)E};
    const cuuint64_t strides[2] = {(cuuint64_t)rb, (cuuint64_t)expert_stride};
    const cuuint32_t box[3] = {(cuuint32_t)(rb / 8 + 2), (cuuint32_t)R, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ZMOE_OK : ZMOE_ERR_CUDA;
}

int make_chunk_map(CUtensorMap *m, const void *base, int E, int O, int rb, size_t expert_stride, int pitch) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ZMOE_ERR_CUDA;
    if (rb % 16 || expert_stride % 16 || pitch % 16 || pitch / 8 > 256) return ZMOE_ERR_SHAPE;
    const cuuint64_t dims[3] = {(cuuint64_t)(rb / 8), (cuuint64_t)O, (cuuint64_t)E};
    const cuuint64_t strides[2] = {(cuuint64_t)rb, (cuuint64_t)expert_stride};
    const cuuint32_t box[3] = {(cuuint32_t)(pitch / 8), 32, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ZMOE_OK : ZMOE_ERR_CUDA;
}

int launch_gemm_sm100(const GemmLaunch &L, cudaStream_t st) {
    if (!gemm_sm100_supported(L.type, L.I, L.O)) return ZMOE_ERR_SHAPE;
    GemmFn fn = nullptr;
    switch (L.type) {
    case Q2_K: fn = L.dual ? gemm_sm100_kernel<Q2_K, true> : gemm_sm100_kernel<Q2_K, false>; break;
    case Q3_K: fn = L.dual ? gemm_sm100_kernel<Q3_K, true> : gemm_sm100_kernel<Q3_K, false>; break;
    case Q4_K: fn = L.dual ? gemm_sm100_kernel<Q4_K, true> : gemm_sm100_kernel<Q4_K, false>; break;
    case IQ2_XXS: fn = L.dual ? gemm_sm100_kernel<IQ2_XXS, true> : gemm_sm100_kernel<IQ2_XXS, false>; break;
    default: return ZMOE_ERR_TYPE;
    }
    const int stage = 2 * GEMM_BM * GEMM_BK * 2 + GEMM_BN * GEMM_BK * 2;
    const int pitch = gemm_raw_pitch(L.type);
    const size_t smem = (size_t)GEMM_NSTAGE * stage + (size_t)GEMM_NRAW * 2 * GEMM_BM * pitch + 1024;
    if (raise_dynamic_smem(reinterpret_cast<const void *>(fn), smem) != ZMOE_OK) return ZMOE_ERR_CUDA;
    GemmParams p;
    p.w0 = static_cast<const uint8_t *>(L.w0);
    p.w1 = static_cast<const uint8_t *>(L.w1);
    p.stride0 = L.stride0; p.stride1 = L.stride1;
    p.I = L.I; p.O = L.O;
    p.rb = (L.I / QK_K) * block_bytes(L.type);
    p.xscale = L.xscale;
    GemmMaps maps;
    for (int i = 0; i < 4; ++i)
        if (make_x_map(&maps.box[i], L.x_f16, L.x_rows, L.I, 32 << i)) return ZMOE_ERR_CUDA;
    // raw super-blocks come through tiled maps over groups of G rows (G * rb a multiple of 16 bytes)
    int G = 1;
    while ((G * p.rb) % 16) G *= 2;           // rb is even: G <= 8
    p.g_log2 = G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3;
    if (L.n_experts <= 0 || (reinterpret_cast<size_t>(L.w0) & 15) || (L.dual && (reinterpret_cast<size_t>(L.w1) & 15)))
        return ZMOE_ERR_ALIGN;
    if (make_w_map(&maps.wmap[0], L.w0, L.n_experts, L.O, p.rb, L.stride0, pitch, G)) return ZMOE_ERR_CUDA;
    if (make_w_map(&maps.wmap[1], L.dual ? L.w1 : L.w0, L.n_experts, L.O, p.rb, L.dual ? L.stride1 : L.stride0, pitch, G))
        return ZMOE_ERR_CUDA;
    p.y = L.y; p.ldy = L.ldy;
    p.hdr = L.plan.hdr; p.active = L.plan.active; p.aoffs = L.plan.aoffs; p.antok = L.plan.antok; p.slot = L.plan.slot;
    p.clamp = L.clamp; p.clamp_fused = L.clamp_fused;
    p.err = L.err;
    p.bad = L.dual ? L.bad : nullptr;
    p.stats = gemm_stats_buffer(L.dual ? 0 : 1);
    return launch_pdl(fn, dim3(L.n_sm), dim3(GEMM_THREADS), smem, st, p, maps) == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA;
}

}  // namespace zmoe
