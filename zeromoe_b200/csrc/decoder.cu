// decoder.cu -- the dense kernels around the MoE block and a decoder step built from them: RMSNorm, dense
// Q8_0 matmul (attention projections, output head), RoPE, grouped-query attention over an f16 KV cache,
// greedy sampling.  With these the fifth benchmark configuration (a full random-init MoE decoder) runs end to
// end on the device.
//
// What each piece follows in the reference:
//   RMSNorm     y = x * rsqrt(mean(x^2) + eps) * w            kernels/math/rmsnorm.cu:6-78 (launch_rmsnorm)
//   Q8_0        34-byte blocks {fp16 d; int8 q[32]}, w = d*q  kernels/quant/q8_0_matmul.cu:20-60,189-221
//   RoPE        interleaved pairs (2j, 2j+1), angle pos * theta^(-2j/dim) built by repeated multiplication
//                                                             models/base/rope.hpp:52-118 (no YaRN: ext_factor 0)
//   attention   scores q.k / sqrt(head_dim), max-subtracted softmax, sum p*v; q head h reads kv head
//               h / (n_heads / n_kv_heads)                     core/attention_layer.cpp:2633-2690
// As everywhere in this library the matmul follows the reference's CPU arithmetic (ggml MUL_MAT): the
// activation row is quantised too (Q8_0 per 32 values) and blocks are multiplied in integers; the
// reference's own CUDA kernel multiplies f32 activations by dequantised weights.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <cmath>
#include <mutex>
#include <new>
#include <vector>

#include "quant_units.cuh"
#include "zmoe_internal.h"

using namespace zmoe;

namespace {

inline int cu(cudaError_t e) { return e == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA; }

// ---------------------------------------------------------------------------
// RMSNorm: one CTA per row
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(float *__restrict__ y, const float *__restrict__ x,
                                                      const float *__restrict__ w, int D, float eps) {
    __shared__ float s_part[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float4 *xv = reinterpret_cast<const float4 *>(x + (size_t)row * D);
    const float4 *wv = reinterpret_cast<const float4 *>(w);
    float4 *yv = reinterpret_cast<float4 *>(y + (size_t)row * D);
    float ss = 0.f;
    for (int i = tid; i < D / 4; i += 256) {
        const float4 v = xv[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float inv = rsqrtf(tot / (float)D + eps);
    for (int i = tid; i < D / 4; i += 256) {
        const float4 v = xv[i], g = wv[i];
        yv[i] = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
    }
}

// RMSNorm followed by the Q8_0 quantiser in one launch (the normed row only feeds a Q8_0 matmul): one CTA per
// row, a thread owns four consecutive elements, the eight threads of a 32-element block share its maximum.
// Same arithmetic, in the same order, as rmsnorm_kernel followed by quantize_q8_0_kernel.
__global__ void __launch_bounds__(256) rmsnorm_q8_0_kernel(int8_t *__restrict__ q, float *__restrict__ d,
                                                           const float *__restrict__ x, const float *__restrict__ w, int D,
                                                           float eps) {
    __shared__ float s_part[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float4 *xv = reinterpret_cast<const float4 *>(x + (size_t)row * D);
    const float4 *wv = reinterpret_cast<const float4 *>(w);
    float ss = 0.f;
    for (int i = tid; i < D / 4; i += 256) {
        const float4 v = xv[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    const float inv = rsqrtf(tot / (float)D + eps);
    const int nb = D / 32;
    // D is a multiple of 32: whole groups of eight threads run each iteration together
    for (int i = tid; i < D / 4; i += 256) {
        const float4 v = xv[i], g = wv[i];
        const float y0 = v.x * inv * g.x, y1 = v.y * inv * g.y, y2 = v.z * inv * g.z, y3 = v.w * inv * g.w;
        float amax = fmaxf(fmaxf(fabsf(y0), fabsf(y1)), fmaxf(fabsf(y2), fabsf(y3)));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float dd = __fdiv_rn(amax, 127.f);
        const float id = dd != 0.f ? __fdiv_rn(1.0f, dd) : 0.f;
        char4 o4;
        o4.x = (signed char)roundf(__fmul_rn(y0, id)); o4.y = (signed char)roundf(__fmul_rn(y1, id));
        o4.z = (signed char)roundf(__fmul_rn(y2, id)); o4.w = (signed char)roundf(__fmul_rn(y3, id));
        reinterpret_cast<char4 *>(q + (size_t)row * D)[i] = o4;
        if ((tid & 7) == 0) d[(size_t)row * nb + (i >> 3)] = __half2float(__float2half_rn(dd));
    }
}

// ---------------------------------------------------------------------------
// Q8_0 activation quantiser: one warp per block of 32 values.  q int8 [rows, I], d f32 [rows, I / 32] holds
// the fp16-rounded scale (what the dot multiplies with).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, int ldx, int8_t *__restrict__ q,
                                                            float *__restrict__ d, int rows, int I) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int nb = I / 32, lane = threadIdx.x & 31;
    for (long blk = (long)blockIdx.x * 8 + (threadIdx.x >> 5); blk < (long)rows * nb; blk += (long)gridDim.x * 8) {
        const int r = (int)(blk / nb), b = (int)(blk % nb);
        const float v = x[(size_t)r * ldx + 32 * b + lane];
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float dd = __fdiv_rn(amax, 127.f);
        const float id = dd != 0.f ? __fdiv_rn(1.0f, dd) : 0.f;
        q[(size_t)r * I + 32 * b + lane] = (int8_t)roundf(__fmul_rn(v, id));
        if (lane == 0) d[(size_t)r * nb + b] = __half2float(__float2half_rn(dd));
    }
}

// ---------------------------------------------------------------------------
// Dense Q8_0 matmul: y[s, o] (+)= sum over blocks of (q_w . q_x) * d_w * d_x.  A warp owns an output row: it
// stages the row's bytes in shared memory with coalesced 16-byte loads, lanes take blocks, the activation
// chunk (up to SC rows) sits in shared memory for the whole CTA, so a weight row is read once per SC rows.
// ---------------------------------------------------------------------------
constexpr int MM_WARPS = 8;
template <int SC>
__global__ void __launch_bounds__(32 * MM_WARPS) q8_0_matmul_kernel(float *__restrict__ y, int ldy,
                                                                    const uint8_t *__restrict__ w, size_t w_bytes,
                                                                    const int8_t *__restrict__ xq,
                                                                    const float *__restrict__ xd, int S, int I, int O,
                                                                    int accumulate) {
    extern __shared__ __align__(16) uint8_t sm[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = I / 32, rb = nb * 34;
    const int rbs = (rb + 32 + 15) & ~15;                   // row buffer: room for the offset from a 16-byte boundary
    int8_t *aq = reinterpret_cast<int8_t *>(sm);            // [SC][I]
    float *ad = reinterpret_cast<float *>(sm + (size_t)SC * I);   // [SC][nb]
    uint8_t *wrow = sm + (size_t)SC * I + (size_t)SC * nb * 4 + (size_t)warp * rbs;
    const uint32_t wrow_s = smem_u32(wrow);
    const size_t w_end16 = w_bytes & ~(size_t)15;           // 16-byte loads stay below this offset
    for (int s0 = 0; s0 < S; s0 += SC) {
        const int ns = min(SC, S - s0);
        __syncthreads();
        for (int i = tid; i < ns * I / 16; i += blockDim.x)
            reinterpret_cast<uint4 *>(aq)[i] = reinterpret_cast<const uint4 *>(xq + (size_t)s0 * I)[i];
        for (int i = tid; i < ns * nb; i += blockDim.x) ad[i] = xd[(size_t)s0 * nb + i];
        __syncthreads();
        for (int o = blockIdx.x * MM_WARPS + warp; o < O; o += gridDim.x * MM_WARPS) {
            const size_t g = (size_t)o * rb;
            const int off = (int)(g & 15);
            const size_t g0 = g - off;
            const int nchunk = (off + rb + 15) / 16;
            for (int c = lane; c < nchunk; c += 32) {
                const size_t at = g0 + 16 * (size_t)c;
                uint4 v;
                if (at + 16 <= w_end16) {
                    v = *reinterpret_cast<const uint4 *>(w + at);
                } else {   // the last bytes of the tensor
                    uint8_t tmp[16];
                    for (int i = 0; i < 16; ++i) tmp[i] = at + i < w_bytes ? w[at + i] : 0;
                    v = *reinterpret_cast<uint4 *>(tmp);
                }
                reinterpret_cast<uint4 *>(wrow)[c] = v;
            }
            __syncwarp();
            float acc[SC];
#pragma unroll
            for (int s = 0; s < SC; ++s) acc[s] = 0.f;
            for (int b = lane; b < nb; b += 32) {
                const uint32_t blk = wrow_s + off + 34 * b;
                const float dw = half_bits_to_float(lds16(blk));
                uint32_t qw[8];
                lds32xN_any<2, 8>(blk + 2, qw);
#pragma unroll
                for (int s = 0; s < SC; ++s) {
                    if (s < ns) {
                        const uint4 a0 = *reinterpret_cast<const uint4 *>(aq + (size_t)s * I + 32 * b);
                        const uint4 a1 = *reinterpret_cast<const uint4 *>(aq + (size_t)s * I + 32 * b + 16);
                        int sum = __dp4a((int)qw[0], (int)a0.x, 0);
                        sum = __dp4a((int)qw[1], (int)a0.y, sum);
                        sum = __dp4a((int)qw[2], (int)a0.z, sum);
                        sum = __dp4a((int)qw[3], (int)a0.w, sum);
                        sum = __dp4a((int)qw[4], (int)a1.x, sum);
                        sum = __dp4a((int)qw[5], (int)a1.y, sum);
                        sum = __dp4a((int)qw[6], (int)a1.z, sum);
                        sum = __dp4a((int)qw[7], (int)a1.w, sum);
                        acc[s] = __fadd_rn(acc[s], __fmul_rn((float)sum, __fmul_rn(dw, ad[s * nb + b])));
                    }
                }
            }
#pragma unroll
            for (int s = 0; s < SC; ++s) {
#pragma unroll
                for (int o2 = 16; o2 > 0; o2 >>= 1) acc[s] += __shfl_xor_sync(0xffffffffu, acc[s], o2);
            }
            if (lane == 0) {
#pragma unroll
                for (int s = 0; s < SC; ++s)
                    if (s < ns) {
                        float *dst = y + (size_t)(s0 + s) * ldy + o;
                        *dst = accumulate ? *dst + acc[s] : acc[s];
                    }
            }
            __syncwarp();
        }
    }
}

// dequantised rows of a Q8_0 table for a list of row numbers (token embedding): one CTA per token
__global__ void __launch_bounds__(256) embed_q8_0_kernel(const int32_t *__restrict__ tokens, const uint8_t *__restrict__ w,
                                                         float *__restrict__ h, int D, int vocab) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : tok >= vocab ? vocab - 1 : tok;
    const uint8_t *row = w + (size_t)tok * (D / 32) * 34;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const uint8_t *blk = row + (i >> 5) * 34;
        const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
        h[(size_t)t * D + i] = d * (float)(int8_t)blk[2 + (i & 31)];
    }
}

// ---------------------------------------------------------------------------
// RoPE on q and k (in place, interleaved pairs) and append of k, v to the f16 cache.  qkv: [T, (H + 2 KV) * hd]
// rows of q | k | v.  Token t sits at position *pos + t.  grid (T, H + KV), hd / 2 threads.
// ---------------------------------------------------------------------------
__global__ void rope_kv_kernel(float *__restrict__ qkv, __half *__restrict__ kc, __half *__restrict__ vc,
                               const int *__restrict__ pos, int H, int KV, int hd, float theta_scale, int max_ctx) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int p = *pos + t;
    if (p >= max_ctx) return;
    const int ld = (H + 2 * KV) * hd;
    float *v = qkv + (size_t)t * ld + (size_t)head * hd;      // q heads, then k heads
    // the angle as the reference builds it: pos * scale * scale * ... (j factors), all in f32, with
    // scale = theta_base^(-2 / head_dim) computed once on the host (as the reference's host code does)
    float ang = (float)p;
    for (int i = 0; i < j; ++i) ang = __fmul_rn(ang, theta_scale);
    const float c = cosf(ang), s = sinf(ang);
    const float a = v[2 * j], b = v[2 * j + 1];
    const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    v[2 * j] = ra;
    v[2 * j + 1] = rb;
    if (head >= H) {
        const int kvh = head - H;
        const size_t at = ((size_t)p * KV + kvh) * hd;
        kc[at + 2 * j] = __float2half_rn(ra);
        kc[at + 2 * j + 1] = __float2half_rn(rb);
        const float *vv = qkv + (size_t)t * ld + (size_t)(H + KV + kvh) * hd;
        vc[at + 2 * j] = __float2half_rn(vv[2 * j]);
        vc[at + 2 * j + 1] = __float2half_rn(vv[2 * j + 1]);
    }
}

// ---------------------------------------------------------------------------
// Grouped-query attention over the f16 cache, causal, keys split over CTAs.  grid (T, KV, NS); one warp per
// query head of the group.  Split z of a token takes the z-th share of its keys and leaves a partial
// (running maximum, sum of weights, weighted sum of V) in scratch; attention_merge_kernel combines the shares.
// A lane owns one key of a 32-key chunk for the scores (the whole head_dim dot product, K row read as 16-byte
// pieces) and DPL output dimensions for the weighted sum of V; the softmax is the running-maximum form.
// ---------------------------------------------------------------------------
constexpr int ATTN_SPLITS = 16;
template <int HD>
__global__ void __launch_bounds__(1024) attention_kernel(const float *__restrict__ qkv, const __half *__restrict__ kc,
                                                         const __half *__restrict__ vc, float *__restrict__ part,
                                                         const int *__restrict__ pos, int H, int KV, float scale,
                                                         int max_ctx) {
    constexpr int DPL = HD / 32;
    extern __shared__ float q_s[];          // [warps][HD]
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = H / KV, h = kvh * G + warp;
    const int n_keys = min(*pos + t + 1, max_ctx);
    // this split's keys: whole chunks of 32, shared out evenly
    const int chunks = (n_keys + 31) / 32, per = (chunks + ATTN_SPLITS - 1) / ATTN_SPLITS;
    const int key_lo = min(n_keys, z * per * 32), key_hi = min(n_keys, (z + 1) * per * 32);
    const int ld = (H + 2 * KV) * HD;
    float *qs = q_s + warp * HD;
    for (int i = lane; i < HD; i += 32) qs[i] = qkv[(size_t)t * ld + (size_t)h * HD + i];
    __syncwarp();
    float m = -CUDART_INF_F, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    for (int k0 = key_lo; k0 < key_hi; k0 += 32) {
        const int key = k0 + lane;
        float s = -CUDART_INF_F;
        if (key < key_hi) {
            const uint4 *kr = reinterpret_cast<const uint4 *>(kc + ((size_t)key * KV + kvh) * HD);
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                const uint4 u = kr[c];
                const __half2 *hp = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 kf = __half22float2(hp[e]);
                    dot = fmaf(qs[8 * c + 2 * e], kf.x, dot);
                    dot = fmaf(qs[8 * c + 2 * e + 1], kf.y, dot);
                }
            }
            s = dot * scale;
        }
        float cm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float m_new = fmaxf(m, cm);
        const float corr = expf(m - m_new);          // 0 on the first chunk (m = -inf)
        const float pr = key < key_hi ? expf(s - m_new) : 0.f;
        float ps = pr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * corr + ps;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        const int nk = min(32, key_hi - k0);
        for (int j = 0; j < nk; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const __half *vr = vc + ((size_t)(k0 + j) * KV + kvh) * HD + DPL * lane;
            if (DPL == 4) {
                const uint2 u = *reinterpret_cast<const uint2 *>(vr);
                const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
                acc[0] = fmaf(pj, a.x, acc[0]); acc[1] = fmaf(pj, a.y, acc[1]);
                acc[2] = fmaf(pj, b.x, acc[2]); acc[3] = fmaf(pj, b.y, acc[3]);
            } else {
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pj, __half2float(vr[i]), acc[i]);
            }
        }
        m = m_new;
    }
    // partial of (t, h, z): [HD values | m | l]
    float *pp = part + (((size_t)t * H + h) * ATTN_SPLITS + z) * (HD + 2);
#pragma unroll
    for (int i = 0; i < DPL; ++i) pp[DPL * lane + i] = acc[i];
    if (lane == 0) { pp[HD] = m; pp[HD + 1] = l; }
}

// out[t, h, :] = sum_z w_z * acc_z / sum_z w_z * l_z with w_z = exp(m_z - max m); one warp per (t, h); shares are
// added in ascending z (empty shares have l = 0 and m = -inf)
template <int HD>
__global__ void __launch_bounds__(256) attention_merge_kernel(const float *__restrict__ part, float *__restrict__ out, int TH) {
    constexpr int DPL = HD / 32;
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int th = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (th >= TH) return;
    const float *pp = part + (size_t)th * ATTN_SPLITS * (HD + 2);
    float mx = -CUDART_INF_F;
    for (int z = 0; z < ATTN_SPLITS; ++z) mx = fmaxf(mx, pp[z * (HD + 2) + HD]);
    float l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    for (int z = 0; z < ATTN_SPLITS; ++z) {
        const float lz = pp[z * (HD + 2) + HD + 1];
        if (lz == 0.f) continue;
        const float wz = expf(pp[z * (HD + 2) + HD] - mx);
        l = fmaf(wz, lz, l);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = fmaf(wz, pp[z * (HD + 2) + DPL * lane + i], acc[i]);
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < DPL; ++i) out[(size_t)th * HD + DPL * lane + i] = acc[i] * inv;
}

// arg-max of a row, lowest index on ties (greedy sampling); one CTA
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ v, int n, int32_t *__restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    float best = -CUDART_INF_F;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = v[i];
        if (x > best || (x == best && i < idx)) { best = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = bv[threadIdx.x]; idx = bi[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
        }
        if (threadIdx.x == 0) *out = idx == 0x7fffffff ? 0 : idx;
    }
}

__global__ void advance_pos_kernel(int *pos, int by) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    if (threadIdx.x == 0 && blockIdx.x == 0) *pos += by;
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
int launch_rmsnorm_rows(float *y, const float *x, const float *w, int S, int D, float eps, cudaStream_t st) {
    if (!y || !x || !w || S <= 0 || D <= 0 || D % 4) return ZMOE_ERR_ARG;
    count_launches(1);
    return cu(launch_pdl(rmsnorm_kernel, dim3(S), dim3(256), 0, st, y, x, w, D, eps));
}

int launch_quantize_q8_0(const float *x, int ldx, int8_t *q, float *d, int rows, int I, cudaStream_t st) {
    const long blocks = (long)rows * (I / 32);
    long grid = (blocks + 7) / 8;
    const long cap = 8L * device_sm_count();
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    count_launches(1);
    return cu(launch_pdl(quantize_q8_0_kernel, dim3((unsigned)grid), dim3(256), 0, st, x, ldx, q, d, rows, I));
}

constexpr int MM_SC = 8;   // activation rows per pass over the weights
int launch_q8_0_mm(float *y, int ldy, const void *w, const int8_t *xq, const float *xd, int S, int I, int O, int accumulate,
                   cudaStream_t st) {
    const int nb = I / 32, rb = nb * 34, rbs = (rb + 32 + 15) & ~15;
    const size_t smem = (size_t)MM_SC * I + (size_t)MM_SC * nb * 4 + (size_t)MM_WARPS * rbs;
    if (smem > 200 * 1024) return ZMOE_ERR_SHAPE;
    auto fn = q8_0_matmul_kernel<MM_SC>;
    if (smem > 48 * 1024 && raise_dynamic_smem(reinterpret_cast<const void *>(fn), smem) != ZMOE_OK) return ZMOE_ERR_CUDA;
    long grid = ((long)O + MM_WARPS - 1) / MM_WARPS;
    const long cap = 4L * device_sm_count();
    if (grid > cap) grid = cap;
    count_launches(1);
    return cu(launch_pdl(fn, dim3((unsigned)grid), dim3(32 * MM_WARPS), smem, st, y, ldy, static_cast<const uint8_t *>(w),
                         (size_t)O * rb, xq, xd, S, I, O, accumulate));
}

// per-device scratch of the handle-free Q8_0 entry: quantised activations
struct Q8Scratch {
    int8_t *q = nullptr;
    float *d = nullptr;
    size_t cap = 0;   // elements
};
Q8Scratch g_q8[64];
std::mutex g_q8_mu;

}  // namespace

// ---------------------------------------------------------------------------
// the decoder
// ---------------------------------------------------------------------------
struct zmoe_decoder {
    zmoe_decoder_desc d;
    std::vector<const float *> attn_norm, ffn_norm;
    std::vector<const void *> wqkv, wo;
    std::vector<zmoe_layer *> moe;
    int qkv_cols = 0;
    float *h = nullptr, *xn = nullptr, *qkv = nullptr, *ao = nullptr, *logits = nullptr, *apart = nullptr;
    int8_t *aq = nullptr;
    float *ad = nullptr;
    __half *kc = nullptr, *vc = nullptr;     // [layers][max_ctx][KV * hd]
    int *pos = nullptr;
    int32_t *next = nullptr;
};

extern "C" {

void launch_rmsnorm(float *y, const float *x, const float *w, int S, int D, float eps) {
    set_last_status(launch_rmsnorm_rows(y, x, w, S, D, eps, nullptr));
}

void launch_q8_0_matmul_stream(float *y, const float *x, const void *weights, int S, int I, int O, void *stream) {
    if (!y || !x || !weights || S <= 0 || I <= 0 || O <= 0) { set_last_status(ZMOE_ERR_ARG); return; }
    if (I % 32) { set_last_status(ZMOE_ERR_SHAPE); return; }
    if (reinterpret_cast<size_t>(weights) & 15) { set_last_status(ZMOE_ERR_ALIGN); return; }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_last_status(ZMOE_ERR_CUDA); return; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the scratch stays locked from sizing to enqueue; it is reallocated only after the device has drained
    std::lock_guard<std::mutex> lock(g_q8_mu);
    Q8Scratch &s = g_q8[dev];
    const size_t need = (size_t)S * I;
    if (need > s.cap) {
        if (s.q) { cudaDeviceSynchronize(); cudaFree(s.q); cudaFree(s.d); s.q = nullptr; s.d = nullptr; s.cap = 0; }
        if (cudaMalloc(reinterpret_cast<void **>(&s.q), need) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void **>(&s.d), (need / 32) * sizeof(float)) != cudaSuccess) {
            set_last_status(ZMOE_ERR_CUDA);
            return;
        }
        s.cap = need;
    }
    int rc = launch_quantize_q8_0(x, I, s.q, s.d, S, I, st);
    if (!rc) rc = launch_q8_0_mm(y, O, weights, s.q, s.d, S, I, O, 0, st);
    set_last_status(rc);
}

void launch_q8_0_matmul(float *y, const float *x, const void *weights, int S, int I, int O) {
    launch_q8_0_matmul_stream(y, x, weights, S, I, O, nullptr);
}

void zmoe_decoder_destroy(zmoe_decoder *dec) {
    if (!dec) return;
    cudaFree(dec->h); cudaFree(dec->xn); cudaFree(dec->qkv); cudaFree(dec->ao); cudaFree(dec->logits); cudaFree(dec->apart);
    cudaFree(dec->aq); cudaFree(dec->ad); cudaFree(dec->kc); cudaFree(dec->vc); cudaFree(dec->pos); cudaFree(dec->next);
    delete dec;
}

int zmoe_decoder_create(const zmoe_decoder_desc *desc, zmoe_decoder **out) {
    if (!desc || !out) return ZMOE_ERR_ARG;
    const zmoe_decoder_desc &d = *desc;
    if (d.n_layers <= 0 || d.d_model <= 0 || d.n_heads <= 0 || d.n_kv_heads <= 0 || d.vocab <= 0 || d.max_ctx <= 0 ||
        d.max_tokens <= 0 || !d.attn_norm_w || !d.wqkv || !d.wo || !d.ffn_norm_w || !d.moe || !d.tok_embd ||
        !d.out_norm_w || !d.lm_head)
        return ZMOE_ERR_ARG;
    if ((d.head_dim != 64 && d.head_dim != 128) || d.n_heads % d.n_kv_heads || d.n_heads / d.n_kv_heads > 32 ||
        d.d_model % 32 || (d.n_heads * d.head_dim) % 32)
        return ZMOE_ERR_SHAPE;
    zmoe_decoder *dec = new (std::nothrow) zmoe_decoder();
    if (!dec) return ZMOE_ERR_ARG;
    dec->d = d;
    for (int l = 0; l < d.n_layers; ++l) {
        if (!d.attn_norm_w[l] || !d.wqkv[l] || !d.wo[l] || !d.ffn_norm_w[l] || !d.moe[l]) {
            delete dec;
            return ZMOE_ERR_ARG;
        }
        dec->attn_norm.push_back(d.attn_norm_w[l]);
        dec->ffn_norm.push_back(d.ffn_norm_w[l]);
        dec->wqkv.push_back(d.wqkv[l]);
        dec->wo.push_back(d.wo[l]);
        dec->moe.push_back(d.moe[l]);
    }
    dec->qkv_cols = (d.n_heads + 2 * d.n_kv_heads) * d.head_dim;
    const size_t T = d.max_tokens, D = d.d_model, QO = (size_t)d.n_heads * d.head_dim;
    const size_t widest = D > QO ? D : QO;
    const size_t kv = (size_t)d.n_layers * d.max_ctx * d.n_kv_heads * d.head_dim;
    auto A = [](auto **p, size_t n) { return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(**p)) != cudaSuccess; };
    int bad = 0;
    bad |= A(&dec->h, T * D); bad |= A(&dec->xn, T * D); bad |= A(&dec->qkv, T * dec->qkv_cols); bad |= A(&dec->ao, T * QO);
    bad |= A(&dec->logits, (size_t)d.vocab);
    bad |= A(&dec->apart, T * d.n_heads * ATTN_SPLITS * (d.head_dim + 2));
    bad |= A(&dec->aq, T * widest); bad |= A(&dec->ad, T * widest / 32);
    bad |= A(&dec->kc, kv); bad |= A(&dec->vc, kv);
    bad |= A(&dec->pos, 1); bad |= A(&dec->next, 1);
    if (!bad) bad |= cudaMemset(dec->pos, 0, sizeof(int)) != cudaSuccess || cudaMemset(dec->next, 0, sizeof(int32_t)) != cudaSuccess;
    if (bad) {
        zmoe_decoder_destroy(dec);
        return ZMOE_ERR_CUDA;
    }
    *out = dec;
    return ZMOE_OK;
}

int zmoe_decoder_reset(zmoe_decoder *dec, void *stream) {
    if (!dec) return ZMOE_ERR_ARG;
    return cu(cudaMemsetAsync(dec->pos, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
}

int zmoe_decoder_step(zmoe_decoder *dec, const int32_t *tokens_dev, int T, void *stream) {
    if (!dec || T <= 0) return ZMOE_ERR_ARG;
    const zmoe_decoder_desc &d = dec->d;
    if (T > d.max_tokens) return ZMOE_ERR_CAPACITY;
    if (!tokens_dev) {
        if (T != 1) return ZMOE_ERR_ARG;
        tokens_dev = dec->next;             // the token the previous step produced
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int D = d.d_model, H = d.n_heads, KV = d.n_kv_heads, hd = d.head_dim, QO = H * hd;
    const size_t kv_layer = (size_t)d.max_ctx * KV * hd;
    const float scale = 1.0f / sqrtf((float)hd);
    const float theta_scale = powf(d.rope_theta, -2.0f / (float)hd);
    int rc = cu(launch_pdl(embed_q8_0_kernel, dim3(T), dim3(256), 0, st, tokens_dev, static_cast<const uint8_t *>(d.tok_embd),
                           dec->h, D, d.vocab));
    count_launches(1);
    for (int l = 0; l < d.n_layers && !rc; ++l) {
        // ---- attention block: h += Wo . attention(rope(Wqkv . rmsnorm(h))) ----
        rc = cu(launch_pdl(rmsnorm_q8_0_kernel, dim3(T), dim3(256), 0, st, dec->aq, dec->ad, (const float *)dec->h,
                           (const float *)dec->attn_norm[l], D, d.rms_eps));
        count_launches(1);
        if (!rc) rc = launch_q8_0_mm(dec->qkv, dec->qkv_cols, dec->wqkv[l], dec->aq, dec->ad, T, D, dec->qkv_cols, 0, st);
        if (!rc) rc = cu(launch_pdl(rope_kv_kernel, dim3(T, H + KV), dim3(hd / 2), 0, st, dec->qkv, dec->kc + l * kv_layer,
                                    dec->vc + l * kv_layer, (const int *)dec->pos, H, KV, hd, theta_scale, d.max_ctx));
        if (!rc) {
            const int warps = H / KV;
            const size_t smem = (size_t)warps * hd * sizeof(float);
            const __half *kl = dec->kc + l * kv_layer, *vl = dec->vc + l * kv_layer;
            if (hd == 128) {
                rc = cu(launch_pdl(attention_kernel<128>, dim3(T, KV, ATTN_SPLITS), dim3(32 * warps), smem, st,
                                   (const float *)dec->qkv, kl, vl, dec->apart, (const int *)dec->pos, H, KV, scale, d.max_ctx));
                if (!rc) rc = cu(launch_pdl(attention_merge_kernel<128>, dim3((T * H + 7) / 8), dim3(256), 0, st,
                                            (const float *)dec->apart, dec->ao, T * H));
            } else {
                rc = cu(launch_pdl(attention_kernel<64>, dim3(T, KV, ATTN_SPLITS), dim3(32 * warps), smem, st,
                                   (const float *)dec->qkv, kl, vl, dec->apart, (const int *)dec->pos, H, KV, scale, d.max_ctx));
                if (!rc) rc = cu(launch_pdl(attention_merge_kernel<64>, dim3((T * H + 7) / 8), dim3(256), 0, st,
                                            (const float *)dec->apart, dec->ao, T * H));
            }
        }
        count_launches(3);
        if (!rc) rc = launch_quantize_q8_0(dec->ao, QO, dec->aq, dec->ad, T, QO, st);
        if (!rc) rc = launch_q8_0_mm(dec->h, D, dec->wo[l], dec->aq, dec->ad, T, QO, D, 1, st);
        // ---- MoE block: h += MoE(rmsnorm(h)) ----
        if (!rc) rc = launch_rmsnorm_rows(dec->xn, dec->h, dec->ffn_norm[l], T, D, d.rms_eps, st);
        if (!rc) rc = zmoe_route(dec->moe[l], dec->xn, T, stream);
        if (!rc) rc = zmoe_expert_ffn(dec->moe[l], dec->h, T, 1, stream);
    }
    // ---- output head on the last token, greedy sampling ----
    if (!rc) {
        rc = cu(launch_pdl(rmsnorm_q8_0_kernel, dim3(1), dim3(256), 0, st, dec->aq, dec->ad,
                           (const float *)(dec->h + (size_t)(T - 1) * D), (const float *)d.out_norm_w, D, d.rms_eps));
        count_launches(1);
    }
    if (!rc) rc = launch_q8_0_mm(dec->logits, d.vocab, d.lm_head, dec->aq, dec->ad, 1, D, d.vocab, 0, st);
    if (!rc) rc = cu(launch_pdl(argmax_kernel, dim3(1), dim3(1024), 0, st, (const float *)dec->logits, d.vocab, dec->next));
    if (!rc) rc = cu(launch_pdl(advance_pos_kernel, dim3(1), dim3(32), 0, st, dec->pos, T));
    count_launches(2);
    return rc;
}

int zmoe_decoder_read(zmoe_decoder *dec, int32_t *next_token_host, int32_t *pos_host, float *logits_host, int n_logits) {
    if (!dec) return ZMOE_ERR_ARG;
    int rc = 0;
    if (next_token_host) rc |= cu(cudaMemcpy(next_token_host, dec->next, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (pos_host) rc |= cu(cudaMemcpy(pos_host, dec->pos, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (logits_host && n_logits > 0)
        rc |= cu(cudaMemcpy(logits_host, dec->logits, (size_t)(n_logits < dec->d.vocab ? n_logits : dec->d.vocab) * sizeof(float),
                            cudaMemcpyDeviceToHost));
    return rc ? ZMOE_ERR_CUDA : ZMOE_OK;
}

}  // extern "C"
