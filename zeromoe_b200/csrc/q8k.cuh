// q8k.cuh -- Q8_K activation quantiser, one warp per 256-element super-block.
//
// Bit-exact restatement of the rule the reference's CPU path applies before
// every quantised dot (ggml quantize_row_q8_K, called from reference
// backends/cpu/kernels_cpu.cpp:2641-2647): the element of largest magnitude,
// with its sign, maps to -127; iscale = -127/max; q = round-half-even(iscale*x)
// clipped above at 127; d = 1/iscale; bsums = sums of 16 consecutive q.
// Output goes to the packed row layout of zmoe_common.cuh.
#pragma once

#include "zmoe_common.cuh"

namespace zmoe {

// src: 256 floats of block b of the row; row_out: packed row base
__device__ __forceinline__ void quantize_block_q8k(const float *__restrict__ src, uint8_t *__restrict__ row_out,
                                                   int I, int b, int lane, int layout) {
    const float4 v0 = *reinterpret_cast<const float4 *>(src + 8 * lane);
    const float4 v1 = *reinterpret_cast<const float4 *>(src + 8 * lane + 4);
    const float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    // first occurrence of the largest |x| wins (strict >), as the scalar loop does
    float amax = 0.f, mx = 0.f;
    int idx = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float ax = fabsf(x[j]);
        if (ax > amax) { amax = ax; mx = x[j]; idx = 8 * lane + j; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
        const float om = __shfl_xor_sync(0xffffffffu, mx, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
    }
    int q[8];
    float d = 0.f;
    if (amax == 0.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = 0;
    } else {
        const float iscale = __fdiv_rn(-127.f, mx);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = min(127, __float2int_rn(__fmul_rn(iscale, x[j])));
        d = __fdiv_rn(1.f, iscale);
    }
    uint2 packed;
    packed.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    // the lane's 8 consecutive elements stay consecutive in either layout
    *reinterpret_cast<uint2 *>(row_out + q8row_elem_off(layout, b, 8 * lane)) = packed;
    int s = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0)
        *reinterpret_cast<int16_t *>(row_out + q8_bs_off(b) + 2 * (lane >> 1)) = (int16_t)s;
    if (lane == 0) *reinterpret_cast<float *>(row_out + q8_d_off(b)) = d;
}

}  // namespace zmoe
