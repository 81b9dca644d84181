// quant_units.cuh -- integer dot products of quantised weight "units" against
// Q8_K activations, one unit = 64 of the 256 elements of a super-block.
//
// A unit is the grain a lane owns: 16 weight/activation word pairs -> 16 dp4a.
// Which 64 elements form a unit depends on how the format packs its quants:
//   planar (Q2_K, Q3_K): unit (n,h) = bytes 16h..16h+15 of the 32-byte group n,
//       i.e. elements 128n + 32j + 16h + i for j<4, i<16  (four 16-element
//       scale groups 8n+2j+h).  Layouts: reference kernels/quant/kquant_matmul.cu:55-72,179-199.
//   linear (Q4_K, IQ2_XXS): unit c = elements 64c .. 64c+63.
//       Layouts: reference kernels/quant/kquant_matmul.cu:74-92, kernels/quant/iq2_matmul.cu:73-91.
// Integer sums are exact, so a super-block's isum/msum is the sum over its four
// units whatever the lane order; only the f32 assembly order differs from the
// CPU path.
#pragma once

#include <cuda_fp16.h>

#include "zmoe_common.cuh"

namespace zmoe {

template <int TYPE> struct QTraits;
template <> struct QTraits<Q2_K> { static constexpr int kBytes = 84, kAlign = 4; static constexpr bool kPlanar = true, kHasMin = true; };
template <> struct QTraits<Q3_K> { static constexpr int kBytes = 110, kAlign = 2; static constexpr bool kPlanar = true, kHasMin = false; };
template <> struct QTraits<Q4_K> { static constexpr int kBytes = 144, kAlign = 16; static constexpr bool kPlanar = false, kHasMin = true; };
template <> struct QTraits<IQ2_XXS> { static constexpr int kBytes = 66, kAlign = 2; static constexpr bool kPlanar = false, kHasMin = false; };

// activation side of one unit, held in registers
struct UnitAct {
    int q[16];   // planar: q[4*j+m]; linear: 16 consecutive words
    int bs[2];   // planar: bsums of groups j=0,1 and j=2,3 as packed int16 pairs;
                 // Q4_K: bs[0], bs[1] = bsums of the low / high 32 elements
    float d;     // Q8_K scale of the unit's super-block
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Load the activation words unit u (block b = u>>2, sub = u&3) needs from a
// packed activation row that sits in shared memory at `row` (16-byte aligned).
template <int TYPE>
__device__ __forceinline__ void load_unit_act(uint32_t row, int I, int u, UnitAct &a) {
    const int b = u >> 2, sub = u & 3;
    a.d = __uint_as_float(lds32(row + q8_d_off(b)));
    const uint32_t bs = row + q8_bs_off(b);
    const uint32_t base = row + q8_unit_off(u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 v = lds128(base + 16 * j);
        a.q[4 * j + 0] = v.x; a.q[4 * j + 1] = v.y; a.q[4 * j + 2] = v.z; a.q[4 * j + 3] = v.w;
    }
    if (QTraits<TYPE>::kPlanar) {
        const int n = sub >> 1, h = sub & 1;
        const uint4 w = lds128(bs + 16 * n);  // bsums[8n .. 8n+7]; group 8n+2j+h is half h of word j
        const uint32_t sel = h ? 0x7632u : 0x5410u;
        a.bs[0] = (int)__byte_perm(w.x, w.y, sel);
        a.bs[1] = (int)__byte_perm(w.z, w.w, sel);
    } else {
        if (TYPE == Q4_K) {
            const uint2 w = lds64(bs + 8 * sub);  // bsums[4c .. 4c+3]
            a.bs[0] = (int)(short)(w.x & 0xffffu) + ((int)w.x >> 16);
            a.bs[1] = (int)(short)(w.y & 0xffffu) + ((int)w.y >> 16);
        }
    }
}

// IQ2_XXS tables in shared memory: 256 x u64 magnitudes, then 128 x u64 byte
// masks (0xFF where the element is negated).
struct Iq2Tables {
    uint32_t grid;   // shared address of uint64_t[256]
    uint32_t signs;  // shared address of uint64_t[128]
};

// One unit: returns the integer scale-weighted sum and the integer min-weighted
// sum, and the block's fp16 scales as floats.
//   contribution to the row = (d * a.d) * isum - (dmin * a.d) * msum     [x 1/8 for IQ2_XXS, applied by the caller]
template <int TYPE>
__device__ __forceinline__ void unit_dot(uint32_t blk, int sub, const UnitAct &a, const Iq2Tables &tb,
                                         int &isum, int &msum, float &d, float &dmin) {
    constexpr int AL = QTraits<TYPE>::kAlign;
    isum = 0;
    msum = 0;
    dmin = 0.f;
    if (TYPE == Q2_K) {
        // scales[16] @0, qs[64] @16, d @80, dmin @82
        const int n = sub >> 1, h = sub & 1;
        uint32_t qs[4];
        lds32xN_any<AL, 4>(blk + 16 + 32 * n + 16 * h, qs);
        const uint32_t s0 = lds32(blk + 8 * n), s1 = lds32(blk + 8 * n + 4);
        const uint32_t dd = lds32(blk + 80);
        d = half_bits_to_float(dd);
        dmin = half_bits_to_float(dd >> 16);
        // bytes j = scale | min << 4 of groups 8n + 2j + h
        const uint32_t w4 = __byte_perm(s0, s1, h ? 0x7531u : 0x6420u);
        const uint32_t sc4 = w4 & 0x0F0F0F0Fu, mn4 = (w4 >> 4) & 0x0F0F0F0Fu;
        int S[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // dp4a on the plane left in place: bytes hold q*4^j, the sum is an exact multiple
            int t = 0;
#pragma unroll
            for (int m = 0; m < 4; ++m) t = dp4a_us(qs[m] & (0x03030303u << (2 * j)), a.q[4 * j + m], t);
            S[j] = t >> (2 * j);   // |S| <= 16*3*127: fits 16 bits
        }
        isum = dp2a_hi_su(pack16(S[2], S[3]), sc4, dp2a_lo_su(pack16(S[0], S[1]), sc4, 0));
        msum = dp2a_hi_su((uint32_t)a.bs[1], mn4, dp2a_lo_su((uint32_t)a.bs[0], mn4, 0));
    } else if (TYPE == Q3_K) {
        // hmask[32] @0, qs[64] @32, scales[12] @96, d @108
        const int n = sub >> 1, h = sub & 1;
        uint32_t qs[4], hm[4], sc[3];
        lds32xN_any<AL, 4>(blk + 32 + 32 * n + 16 * h, qs);
        lds32xN_any<AL, 4>(blk + 16 * h, hm);
        lds32xN_any<AL, 3>(blk + 96, sc);
        d = half_bits_to_float(lds16(blk + 108));
#pragma unroll
        for (int m = 0; m < 4; ++m) hm[m] >>= 4 * n;   // plane bits j = 0..3 now sit at bit j of every byte
        int S[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int t = 0;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                // q2 | hbit << 2 in one select: low two bits from qs, bit 2 from hmask
                const uint32_t hb = (j < 2 ? hm[m] << (2 - j) : hm[m] >> (j - 2)) & 0x04040404u;
                const uint32_t q = ((qs[m] >> (2 * j)) & 0x03030303u) | hb;
                t = dp4a_us(q, a.q[4 * j + m], t);
            }
            S[j] = t;   // |S| <= 16*7*127: fits 16 bits
        }
        // q3 = (q2 | hbit << 2) - 4: subtract 4 * bsum of the group
        const int b01 = a.bs[0], b23 = a.bs[1];
        S[0] -= 4 * (int)(short)(b01 & 0xffff); S[1] -= 4 * (b01 >> 16);
        S[2] -= 4 * (int)(short)(b23 & 0xffff); S[3] -= 4 * (b23 >> 16);
        // 6-bit scales of groups k = 8n + 2j + h: low nibbles in bytes 0..7 (low half for k < 8,
        // high half for k >= 8), the two high bits in bytes 8..11 at bit 2*(k>>2) of byte k&3
        const uint32_t lo = (__byte_perm(sc[0], sc[1], h ? 0x7531u : 0x6420u) >> (4 * n)) & 0x0F0F0F0Fu;
        const uint32_t hs = __byte_perm(sc[2], 0, h ? 0x3131u : 0x2020u) >> (4 * n);
        const uint32_t hi = (hs & 0x00000303u) | ((hs >> 2) & 0x03030000u);
        const uint32_t sc6 = lo | (hi << 4);
        const int tot = S[0] + S[1] + S[2] + S[3];
        // sum (sc6 - 32) * S; |S| can reach 16*7*127 + 4*16*127 which still fits 16 bits
        isum = dp2a_hi_su(pack16(S[2], S[3]), sc6, dp2a_lo_su(pack16(S[0], S[1]), sc6, 0)) - 32 * tot;
    } else if (TYPE == Q4_K) {
        // d @0, dmin @2, scales[12] @4, qs[128] @16
        const int c = sub;
        const uint4 q0 = lds128(blk + 16 + 32 * c), q1 = lds128(blk + 32 + 32 * c);
        const uint32_t qs[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t dd = lds32(blk);
        d = half_bits_to_float(dd);
        dmin = half_bits_to_float(dd >> 16);
        const uint32_t s0 = lds32(blk + 4), s1 = lds32(blk + 8), s2 = lds32(blk + 12);
        // pairs j = 2c, 2c+1 (reference kernels/quant/kquant_matmul.cu:41-48)
        int sc_lo, sc_hi, m_lo, m_hi;
        if (c < 2) {
            sc_lo = (s0 >> (16 * c)) & 63;
            sc_hi = (s0 >> (16 * c + 8)) & 63;
            m_lo = (s1 >> (16 * c)) & 63;
            m_hi = (s1 >> (16 * c + 8)) & 63;
        } else {
            const int cc = c - 2;  // j-4 = 2cc, 2cc+1
            const uint32_t a0 = (s2 >> (16 * cc)) & 0xffu, a1 = (s2 >> (16 * cc + 8)) & 0xffu;
            sc_lo = (int)((a0 & 0xFu) | ((((s0 >> (16 * cc)) & 0xffu) >> 6) << 4));
            sc_hi = (int)((a1 & 0xFu) | ((((s0 >> (16 * cc + 8)) & 0xffu) >> 6) << 4));
            m_lo = (int)((a0 >> 4) | ((((s1 >> (16 * cc)) & 0xffu) >> 6) << 4));
            m_hi = (int)((a1 >> 4) | ((((s1 >> (16 * cc + 8)) & 0xffu) >> 6) << 4));
        }
        int slo = 0, shi = 0;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            slo = dp4a_us(qs[m] & 0x0F0F0F0Fu, a.q[m], slo);
            shi = dp4a_us(qs[m] & 0xF0F0F0F0u, a.q[8 + m], shi);   // the high nibbles in place: 16 x the sum, exactly
        }
        isum = sc_lo * slo + sc_hi * (shi >> 4);
        msum = m_lo * a.bs[0] + m_hi * a.bs[1];
    } else {  // IQ2_XXS: d @0, qs[32] u16 @2 ; unit = sub-blocks 2*sub, 2*sub+1
        uint32_t aux[4];
        lds32xN_any<AL, 4>(blk + 2 + 16 * sub, aux);
        d = half_bits_to_float(lds16(blk));
#pragma unroll
        for (int ib = 0; ib < 2; ++ib) {
            const uint32_t a0 = aux[2 * ib], a1 = aux[2 * ib + 1];
            int s = 0;
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                const uint2 g = lds64(tb.grid + 8 * ((a0 >> (8 * l)) & 255u));
                const uint2 neg = lds64(tb.signs + 8 * ((a1 >> (7 * l)) & 127u));
                const int x0 = a.q[8 * ib + 2 * l], x1 = a.q[8 * ib + 2 * l + 1];
                // sum(g*sign*x) = sum(g*x) - 2*sum over negated bytes
                s = dp4a_us(g.x, x0, s);
                s = dp4a_us(g.y, x1, s);
                s -= 2 * dp4a_us(g.x & neg.x, x0, dp4a_us(g.y & neg.y, x1, 0));
            }
            isum += (int)(2 * (a1 >> 28) + 1) * s;
        }
    }
}

// One whole Q2_K super-block of one row (of two rows, NM = 2: the same block of the gate and of the up matrix)
// against one activation block.  Same integers as four unit_dot calls; the work that does not depend on the unit
// is done once per block: one load of d / dmin, the sixteen scale nibbles taken in place (a dp2a pairs the sums of
// the two units h = 0, 1 of a 32-byte group with two adjacent scale bytes, so no byte is moved), the mins against
// the group sums straight from the packed row, one int -> float conversion per sum.
//   blk[m]: the block in shared memory (4-byte aligned); arow: the packed activation row; b: its block index
//   acc[m] += d * d8 * isum - dmin * d8 * msum
template <int NM>
__device__ __forceinline__ void q2k_block_dot(const uint32_t (&blk)[NM], uint32_t arow, int I, int b, float (&acc)[NM]) {
    uint32_t sc[NM][4];
    int isum[NM];
#pragma unroll
    for (int m = 0; m < NM; ++m) {
#pragma unroll
        for (int w = 0; w < 4; ++w) sc[m][w] = lds32(blk[m] + 4 * w);
        isum[m] = 0;
    }
    // the halves run as a loop (not unrolled: the consumer loop has to stay inside the instruction cache)
#pragma unroll 1
    for (int n = 0; n < 2; ++n) {
        // the two units of this half: aq[h][4 * j + i] multiplies word i of the 16 bytes h, plane j
        uint32_t aq[2][16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t base = arow + Q8_BLOCK_STRIDE * b + Q8_UNIT_STRIDE * (2 * n + h);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = lds128(base + 16 * j);
                aq[h][4 * j + 0] = v.x; aq[h][4 * j + 1] = v.y; aq[h][4 * j + 2] = v.z; aq[h][4 * j + 3] = v.w;
            }
        }
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            uint32_t qs[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) qs[i] = lds32(blk[m] + 16 + 32 * n + 4 * i);
            int S[4][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int t = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) t = dp4a_us(qs[4 * h + i] & (0x03030303u << (2 * j)), (int)aq[h][4 * j + i], t);
                    S[j][h] = t >> (2 * j);
                }
            }
            const uint32_t s0 = (n ? sc[m][2] : sc[m][0]) & 0x0F0F0F0Fu, s1 = (n ? sc[m][3] : sc[m][1]) & 0x0F0F0F0Fu;
            int t = isum[m];
            t = dp2a_lo_su(pack16(S[0][0], S[0][1]), s0, t);
            t = dp2a_hi_su(pack16(S[1][0], S[1][1]), s0, t);
            t = dp2a_lo_su(pack16(S[2][0], S[2][1]), s1, t);
            t = dp2a_hi_su(pack16(S[3][0], S[3][1]), s1, t);
            isum[m] = t;
        }
    }
    // mins: word w of the group sums holds groups 2w, 2w + 1; byte g of the min nibbles is group g
    const uint32_t bs = arow + q8_bs_off(b);
    const uint4 b0 = lds128(bs), b1 = lds128(bs + 16);
    const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const float d8 = __uint_as_float(lds32(arow + q8_d_off(b)));
#pragma unroll
    for (int m = 0; m < NM; ++m) {
        int ms = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t mn = (sc[m][w] >> 4) & 0x0F0F0F0Fu;
            ms = dp2a_lo_su(bw[2 * w], mn, ms);
            ms = dp2a_hi_su(bw[2 * w + 1], mn, ms);
        }
        const uint32_t dd = lds32(blk[m] + 80);
        const float d = half_bits_to_float(dd), dmin = half_bits_to_float(dd >> 16);
        acc[m] = fmaf(d * d8, (float)isum[m], acc[m]);
        acc[m] = fmaf(-(dmin * d8), (float)ms, acc[m]);
    }
}

// One half (128 elements: the units (n, h = 0, 1), scale groups 8n .. 8n + 7) of a Q3_K super-block of one row (of
// two rows, NM = 2) against the matching half of an activation block.  Same integers as two unit_dot calls.  Done
// once per half instead of once per unit: the eight six-bit scales (taken as signed bytes sc - 32, so that a dp2a
// pairs the sums of the units h = 0, 1 with two adjacent scale bytes), the -4 offset of the quants (the same dp2a on
// the group sums of the packed row, which sit in group order), d, and the int -> float conversion.  The 2-bit
// planes and the high-bit plane stay in place under the dp4a: byte values q << 2j and 1 << (4n + j) give exact
// multiples, which one shift per plane brings back.
//   blk[m]: the block in shared memory (2-byte aligned); arow: the packed activation row; b: its block index
//   acc[m] += d * d8 * isum
template <int NM>
__device__ __forceinline__ void q3k_half_dot(const uint32_t (&blk)[NM], int n, uint32_t arow, int I, int b, float (&acc)[NM]) {
    uint32_t aq[2][16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t base = arow + Q8_BLOCK_STRIDE * b + Q8_UNIT_STRIDE * (2 * n + h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 v = lds128(base + 16 * j);
            aq[h][4 * j + 0] = v.x; aq[h][4 * j + 1] = v.y; aq[h][4 * j + 2] = v.z; aq[h][4 * j + 3] = v.w;
        }
    }
    const uint4 bw = lds128(arow + q8_bs_off(b) + 16 * n);   // group sums 8n .. 8n + 7
    const float d8 = __uint_as_float(lds32(arow + q8_d_off(b)));
    const uint32_t hbit = 0x01010101u << (4 * n);
#pragma unroll
    for (int m = 0; m < NM; ++m) {
        // hmask[32] @0, qs[64] @32, scales[12] @96, d @108
        uint32_t qs[8], hm[8], sc[3];
        lds32xN_any<2, 8>(blk[m] + 32 + 32 * n, qs);
        lds32xN_any<2, 8>(blk[m], hm);
        lds32xN_any<2, 3>(blk[m] + 96, sc);
        const float d = half_bits_to_float(lds16(blk[m] + 108));
        int S[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int tq = 0, th = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    tq = dp4a_us(qs[4 * h + i] & (0x03030303u << (2 * j)), (int)aq[h][4 * j + i], tq);
                    th = dp4a_us(hm[4 * h + i] & (hbit << j), (int)aq[h][4 * j + i], th);
                }
                S[j][h] = (tq >> (2 * j)) + 4 * (th >> (4 * n + j));   // |S| <= 16*7*127: fits 16 bits
            }
        }
        // scale of group 8n + i: low nibble = nibble n of byte i of the first eight bytes, high two bits = bits
        // 4n + 2 * (i >> 2) of byte i & 3 of the last four
        const uint32_t hs = sc[2] >> (4 * n);
        uint32_t s0 = ((sc[0] >> (4 * n)) & 0x0F0F0F0Fu) | ((hs & 0x03030303u) << 4);
        uint32_t s1 = ((sc[1] >> (4 * n)) & 0x0F0F0F0Fu) | (((hs >> 2) & 0x03030303u) << 4);
        // bytes 0..63 -> signed bytes sc - 32 (the top bit keeps the bytes apart during the subtraction)
        s0 = ((s0 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
        s1 = ((s1 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
        int t = dp2a_lo_ss(pack16(S[0][0], S[0][1]), s0, 0);
        t = dp2a_hi_ss(pack16(S[1][0], S[1][1]), s0, t);
        t = dp2a_lo_ss(pack16(S[2][0], S[2][1]), s1, t);
        t = dp2a_hi_ss(pack16(S[3][0], S[3][1]), s1, t);
        // q3 = (q2 | hbit << 2) - 4: minus 4 * scale * group sum
        int u = dp2a_lo_ss(bw.x, s0, 0);
        u = dp2a_hi_ss(bw.y, s0, u);
        u = dp2a_lo_ss(bw.z, s1, u);
        u = dp2a_hi_ss(bw.w, s1, u);
        acc[m] = fmaf(d * d8, (float)(t - 4 * u), acc[m]);
    }
}

// IQ2_XXS codebook (ggml data; reference backends/cpu/ggml_grids.cpp:11-15)
static __device__ const uint64_t k_iq2xxs_grid[256] = {
#include "iq2xxs_grid.inc"
};

// Fill the IQ2_XXS tables in shared memory from the codebook.  Every thread of
// the CTA must call it; the caller synchronises afterwards.
__device__ __forceinline__ void iq2_fill_tables(uint64_t *grid_smem, uint64_t *sign_smem) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) grid_smem[i] = k_iq2xxs_grid[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) {
        // sign byte = index with bit 7 chosen for even parity; expand bits to 0x00 / 0xFF bytes
        const uint32_t s = (uint32_t)i | ((uint32_t)(__popc(i) & 1) << 7);
        uint64_t m = 0;
        for (int j = 0; j < 8; ++j)
            if ((s >> j) & 1u) m |= 0xffull << (8 * j);
        sign_smem[i] = m;
    }
}

}  // namespace zmoe
