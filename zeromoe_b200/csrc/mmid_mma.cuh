// mmid_mma.cuh -- multi-token consumer path of the decode-shaped expert matmul.
//
// When several pairs are routed to one expert, the scalar path of mmid.cuh decodes
// the same weight row once per pair.  Here a warp decodes a 16-row slice of the
// tile ONCE into int8 operand fragments and multiplies it against up to
// MMID_MAXTOK activation rows with warp-level int8 tensor-core instructions
// (mma.sync m16n8k32 / m16n8k16, s32 accumulate).  The tile is bandwidth-bound
// work: the tensor cores take integer work off the issue ports, which are what
// limits the scalar path; their throughput is not the point.
//
// Integer sums are exact, so per super-block they equal those of the scalar path
// and of reference kernels/quant/kquant_matmul.cu:179-199 (Q2_K), :201-238 (Q3_K), :74-92 (Q4_K);
// the f32 assembly adds super-blocks in a different order (a warp owns a slice of
// the row, slices are added in shared memory in warp order).
//
// Fragment layout used throughout (lane = 4g + c):
//   A (16 x 32 bytes, row major):  a0 = row g,   k 4c..4c+3     a1 = row g+8, k 4c..4c+3
//                                  a2 = row g,   k 16+4c..      a3 = row g+8, k 16+4c..
//   B (32 x 8, column = pair):     b0 = k 4c..4c+3 of pair g    b1 = k 16+4c.. of pair g
//   C (16 x 8 s32):                c0 = (g, 2c) c1 = (g, 2c+1) c2 = (g+8, 2c) c3 = (g+8, 2c+1)
//   k16 form: A = {a0, a1}, B = {b0}.
// Only columns 0..MMID_MAXTOK-1 carry pairs.  The other columns read the same activation rows
// again (g modulo MMID_MAXTOK) so that no load needs a predicate; their sums are never stored.
#pragma once

#include "quant_units.cuh"

namespace zmoe {

constexpr int MMA_NTOK = 4;   // pairs per item the fragments are laid out for (== MMID_MAXTOK)

// ---- instruction wrappers ---------------------------------------------------------------------------------
// ZERO: start from zero instead of accumulating into c
template <bool ZERO>
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    if (ZERO)
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// k16, from zero.  SIGNED_A: A bytes are signed.
template <bool SIGNED_A>
__device__ __forceinline__ void mma_k16_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    if (SIGNED_A)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0), "r"(0));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// byte SEL & 3 of x, sign-extended (selector bit 3 of a nibble replicates the chosen byte's top bit)
__device__ __forceinline__ int sext_byte(uint32_t x, int j) {
    int v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(x), "r"(0u), "r"(((8 | j) * 0x1110) | j));
    return v;
}

// shared-memory word at base + OFF (OFF folds into the instruction)
template <int OFF>
__device__ __forceinline__ uint32_t ldso(uint32_t base) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(OFF));
    return v;
}
// the same where base + OFF is 2 modulo 4 (MIS): two aligned words, spliced
template <bool MIS, int OFF>
__device__ __forceinline__ uint32_t ldso_mis(uint32_t base) {
    if (!MIS) return ldso<OFF>(base);
    return __byte_perm(ldso<OFF - 2>(base), ldso<OFF + 2>(base), 0x5432);
}

// Group sums of the activations (int16, |v| <= 16 * 127) of groups 4c..4c+3 as two planes of bytes,
// v = 128 * hi + lo with 0 <= lo < 128 and -16 <= hi < 16: the B operand of k16 instructions whose A
// bytes are per-group factors.  w0, w1 hold the four int16 values.
__device__ __forceinline__ void bsum_planes(uint32_t w0, uint32_t w1, uint32_t &hi, uint32_t &lo) {
    lo = __byte_perm(w0, w1, 0x6420) & 0x7F7F7F7Fu;
    hi = __byte_perm(w0 >> 7, w1 >> 7, 0x6420);   // bits 7..14 of each value
}

// Activation fragments of half N (128 elements) of super-block b.  Planar packed rows: element
// 128n + 32s + 16h + i of block b is byte 16s + i of unit 4b + 2n + h.  qrow: the column's row + 4c.
template <int N>
__device__ __forceinline__ void load_b_half(uint32_t qrow_blk, uint32_t (&bq)[4][2]) {
    bq[0][0] = ldso<(2 * N) * Q8_UNIT_STRIDE + 0>(qrow_blk);  bq[0][1] = ldso<(2 * N + 1) * Q8_UNIT_STRIDE + 0>(qrow_blk);
    bq[1][0] = ldso<(2 * N) * Q8_UNIT_STRIDE + 16>(qrow_blk); bq[1][1] = ldso<(2 * N + 1) * Q8_UNIT_STRIDE + 16>(qrow_blk);
    bq[2][0] = ldso<(2 * N) * Q8_UNIT_STRIDE + 32>(qrow_blk); bq[2][1] = ldso<(2 * N + 1) * Q8_UNIT_STRIDE + 32>(qrow_blk);
    bq[3][0] = ldso<(2 * N) * Q8_UNIT_STRIDE + 48>(qrow_blk); bq[3][1] = ldso<(2 * N + 1) * Q8_UNIT_STRIDE + 48>(qrow_blk);
}

// ---- Q2_K: scales[16] @0 (scale | min << 4), qs[64] @16, d @80, dmin @82 -----------------------------------
// Quants of element 128n + 32s + i sit in byte 32n + i at bit 2s; its 16-element group is 8n + 2s + i/16.
// The 4-bit scale is multiplied into the quants (3 * 15 fits a byte), so one k32 instruction spans two
// groups and a whole super-block accumulates in one s32.
// rowA / rowB: the block in rows g and g+8.  FIRST: cm starts from zero.
// Two accumulators (even and odd s) halve the chain of dependent instructions; cx holds FOUR times the sums of the
// odd planes (they are multiplied where they sit), the caller adds cm + (cx >> 2).
template <int N, bool FIRST>
__device__ __forceinline__ void q2k_half(uint32_t rowA, uint32_t rowB, int c, const uint32_t (&bq)[4][2], int (&cm)[4],
                                         int (&cx)[4]) {
    const uint32_t qA = rowA + 4 * c, qB = rowB + 4 * c;
    const uint32_t qa[2] = {ldso<16 + 32 * N>(qA), ldso<32 + 32 * N>(qA)};
    const uint32_t qb[2] = {ldso<16 + 32 * N>(qB), ldso<32 + 32 * N>(qB)};
    const uint32_t sA[2] = {ldso<8 * N>(rowA) & 0x0F0F0F0Fu, ldso<8 * N + 4>(rowA) & 0x0F0F0F0Fu};
    const uint32_t sB[2] = {ldso<8 * N>(rowB) & 0x0F0F0F0Fu, ldso<8 * N + 4>(rowB) & 0x0F0F0F0Fu};
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int w = s >> 1, by = (s & 1) * 2;   // groups 2s, 2s+1 of the half: bytes by, by+1 of word w
        const uint32_t e0 = 0x4440u | by, e1 = 0x4440u | (by + 1);
        // odd s: the plane stays two bits up (bytes 4 * q * scale <= 180), so cx holds four times its sums
        const int sh = 4 * (s >> 1);
        const uint32_t mask = (s & 1) ? 0x0C0C0C0Cu : 0x03030303u;
        const uint32_t a0 = ((qa[0] >> sh) & mask) * __byte_perm(sA[w], 0, e0);
        const uint32_t a1 = ((qb[0] >> sh) & mask) * __byte_perm(sB[w], 0, e0);
        const uint32_t a2 = ((qa[1] >> sh) & mask) * __byte_perm(sA[w], 0, e1);
        const uint32_t a3 = ((qb[1] >> sh) & mask) * __byte_perm(sB[w], 0, e1);
        if (s & 1) {
            if (FIRST && s == 1) mma_u8s8_k32<true>(cx, a0, a1, a2, a3, bq[s][0], bq[s][1]);
            else mma_u8s8_k32<false>(cx, a0, a1, a2, a3, bq[s][0], bq[s][1]);
        } else {
            if (FIRST && s == 0) mma_u8s8_k32<true>(cm, a0, a1, a2, a3, bq[s][0], bq[s][1]);
            else mma_u8s8_k32<false>(cm, a0, a1, a2, a3, bq[s][0], bq[s][1]);
        }
    }
}
// sum over the block's groups of min * (group sum of the activations), for the block in rows g and g+8
__device__ __forceinline__ void q2k_mins(uint32_t rowA, uint32_t rowB, int c, uint32_t bs_hi, uint32_t bs_lo,
                                         int (&cn)[4]) {
    const uint32_t mA = (lds32(rowA + 4 * c) >> 4) & 0x0F0F0F0Fu, mB = (lds32(rowB + 4 * c) >> 4) & 0x0F0F0F0Fu;
    int hi[4];
    mma_k16_zero<false>(hi, mA, mB, bs_hi);
    mma_k16_zero<false>(cn, mA, mB, bs_lo);
#pragma unroll
    for (int i = 0; i < 4; ++i) cn[i] += hi[i] * 128;
}

// ---- Q3_K: hmask[32] @0, qs[64] @32, scales[12] @96, d @108 ------------------------------------------------
// value = (sc6 - 32) * ((q2 | hbit << 2) - 4).  One k16 instruction per 16-element group on the unsigned
// 3-bit quants; the signed 6-bit scale multiplies the group's sums afterwards.  The "- 4" becomes
// -4 * sum over groups of scale * (group sum of the activations): k16 instructions with the signed scales
// as A bytes, masked to this half's groups.
// rowA / rowB: the block in rows g and g+8; N: which half; acc: scaled integer sums of the super-block.
// N (which half) is a run-time value: one copy of this code per alignment instead of two keeps the consumer loop
// inside the instruction cache.
template <bool MIS>
__device__ __forceinline__ void q3k_half(uint32_t rowA, uint32_t rowB, int c, int N, const uint32_t (&bq)[4][2],
                                         uint32_t bs_hi, uint32_t bs_lo, int (&acc)[4]) {
    const uint32_t qA = rowA + 4 * c, qB = rowB + 4 * c;
    const uint32_t qAn = qA + 32 * N, qBn = qB + 32 * N;
    const uint32_t qa[2] = {ldso_mis<MIS, 32>(qAn), ldso_mis<MIS, 48>(qAn)};
    const uint32_t qb[2] = {ldso_mis<MIS, 32>(qBn), ldso_mis<MIS, 48>(qBn)};
    // plane bit of shift s of this half is bit 4n + s of the mask byte: bring bit 4n to bit 0
    const uint32_t ha[2] = {ldso_mis<MIS, 0>(qA) >> (4 * N), ldso_mis<MIS, 16>(qA) >> (4 * N)};
    const uint32_t hb[2] = {ldso_mis<MIS, 0>(qB) >> (4 * N), ldso_mis<MIS, 16>(qB) >> (4 * N)};
    // 6-bit scales of groups 8n + j: low nibbles in bytes 0..7 (low half for groups < 8), the two high
    // bits in bytes 8..11 at bit 2*(group / 4) of byte group % 4.  Bytes become sc6 - 32 (signed).
    // The four lanes c of a row pair share the work: lane c unpacks word c & 1 of row A (c < 2) or row B, a shuffle
    // inside the group of four passes the words on.
    uint32_t sA[2], sB[2];
    {
        const uint32_t rowS = (c & 2) ? rowB : rowA;
        const int ws = c & 1;
        const uint32_t w = ldso_mis<MIS, 96>(rowS + 4 * ws), w2 = ldso_mis<MIS, 104>(rowS);
        const uint32_t a = ((w >> (4 * N)) & 0x0F0F0F0Fu) | (((w2 >> (4 * N + 2 * ws)) & 0x03030303u) << 4);
        // bytes are < 64: with bit 7 set the subtraction cannot borrow across bytes
        const uint32_t sx = ((a | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
        sA[0] = __shfl_sync(0xffffffffu, sx, 0, 4);
        sA[1] = __shfl_sync(0xffffffffu, sx, 1, 4);
        sB[0] = __shfl_sync(0xffffffffu, sx, 2, 4);
        sB[1] = __shfl_sync(0xffffffffu, sx, 3, 4);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int j = 2 * s + h;   // group within the half
            const uint32_t hbA = (s < 2 ? ha[h] << (2 - s) : ha[h] >> (s - 2)) & 0x04040404u;
            const uint32_t hbB = (s < 2 ? hb[h] << (2 - s) : hb[h] >> (s - 2)) & 0x04040404u;
            const uint32_t a0 = ((qa[h] >> (2 * s)) & 0x03030303u) | hbA;
            const uint32_t a1 = ((qb[h] >> (2 * s)) & 0x03030303u) | hbB;
            int t[4];
            mma_k16_zero<false>(t, a0, a1, bq[s][h]);
            const int scA = sext_byte(sA[j >> 2], j & 3), scB = sext_byte(sB[j >> 2], j & 3);
            acc[0] += scA * t[0]; acc[1] += scA * t[1];
            acc[2] += scB * t[2]; acc[3] += scB * t[3];
        }
    }
    // lanes c hold groups 4c..4c+3 of the block: those of this half are c = 2n, 2n+1
    const bool mine = (c >> 1) == N;
    const uint32_t fa = mine ? sA[c & 1] : 0u, fb = mine ? sB[c & 1] : 0u;
    int hi[4], lo[4];
    mma_k16_zero<true>(hi, fa, fb, bs_hi);
    mma_k16_zero<true>(lo, fa, fb, bs_lo);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] -= 4 * (hi[i] * 128 + lo[i]);
}

// ---- Q4_K: d @0, dmin @2, scales[12] @4, qs[128] @16 ------------------------------------------------------
// Byte 32j + i holds element 64j + i in its low nibble and 64j + 32 + i in its high nibble; 32-element
// sub-block sb = 2j (low) or 2j + 1 (high) has a 6-bit scale and a 6-bit min.  One k32 instruction per
// sub-block on the nibbles; the scale multiplies the sub-block's sums afterwards.  Activation rows are in
// the linear layout: element 64u + i is byte i of unit u.
// rowA / rowB: the block in rows g and g+8; qblk: the column's activation row + unit 4b + 4c;
// acc: scaled integer sums of the super-block (from zero); mA / mB: the min bytes of sub-blocks 0-3 and 4-7.
__device__ __forceinline__ void q4k_block(uint32_t rowA, uint32_t rowB, int c, uint32_t qblk, int (&acc)[4],
                                          uint32_t (&mnA)[2], uint32_t (&mnB)[2]) {
    uint32_t scA[2], scB[2];
    {
        // scales[12] as words s0 s1 s2 (reference kernels/quant/kquant_matmul.cu:41-48): sub-blocks 0-3 take
        // 6 bits of s0 (scale) and s1 (min); 4-7 take nibbles of s2 plus the top two bits of s0 / s1
        const uint32_t a0 = ldso<4>(rowA), a1 = ldso<8>(rowA), a2 = ldso<12>(rowA);
        const uint32_t b0 = ldso<4>(rowB), b1 = ldso<8>(rowB), b2 = ldso<12>(rowB);
        scA[0] = a0 & 0x3F3F3F3Fu; scA[1] = (a2 & 0x0F0F0F0Fu) | ((a0 >> 2) & 0x30303030u);
        mnA[0] = a1 & 0x3F3F3F3Fu; mnA[1] = ((a2 >> 4) & 0x0F0F0F0Fu) | ((a1 >> 2) & 0x30303030u);
        scB[0] = b0 & 0x3F3F3F3Fu; scB[1] = (b2 & 0x0F0F0F0Fu) | ((b0 >> 2) & 0x30303030u);
        mnB[0] = b1 & 0x3F3F3F3Fu; mnB[1] = ((b2 >> 4) & 0x0F0F0F0Fu) | ((b1 >> 2) & 0x30303030u);
    }
    const uint32_t qA = rowA + 4 * c, qB = rowB + 4 * c;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t wa0, wa1, wb0, wb1, bl0, bl1, bh0, bh1;
        // immediate offsets need literals: one switch arm per j
        if (j == 0) { wa0 = ldso<16>(qA); wa1 = ldso<32>(qA); wb0 = ldso<16>(qB); wb1 = ldso<32>(qB);
                      bl0 = ldso<0>(qblk); bl1 = ldso<16>(qblk); bh0 = ldso<32>(qblk); bh1 = ldso<48>(qblk); }
        else if (j == 1) { wa0 = ldso<48>(qA); wa1 = ldso<64>(qA); wb0 = ldso<48>(qB); wb1 = ldso<64>(qB);
                           bl0 = ldso<Q8_UNIT_STRIDE>(qblk); bl1 = ldso<Q8_UNIT_STRIDE + 16>(qblk);
                           bh0 = ldso<Q8_UNIT_STRIDE + 32>(qblk); bh1 = ldso<Q8_UNIT_STRIDE + 48>(qblk); }
        else if (j == 2) { wa0 = ldso<80>(qA); wa1 = ldso<96>(qA); wb0 = ldso<80>(qB); wb1 = ldso<96>(qB);
                           bl0 = ldso<2 * Q8_UNIT_STRIDE>(qblk); bl1 = ldso<2 * Q8_UNIT_STRIDE + 16>(qblk);
                           bh0 = ldso<2 * Q8_UNIT_STRIDE + 32>(qblk); bh1 = ldso<2 * Q8_UNIT_STRIDE + 48>(qblk); }
        else { wa0 = ldso<112>(qA); wa1 = ldso<128>(qA); wb0 = ldso<112>(qB); wb1 = ldso<128>(qB);
               bl0 = ldso<3 * Q8_UNIT_STRIDE>(qblk); bl1 = ldso<3 * Q8_UNIT_STRIDE + 16>(qblk);
               bh0 = ldso<3 * Q8_UNIT_STRIDE + 32>(qblk); bh1 = ldso<3 * Q8_UNIT_STRIDE + 48>(qblk); }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int sb = 2 * j + h;
            int t[4];
            mma_u8s8_k32<true>(t, (wa0 >> (4 * h)) & 0x0F0F0F0Fu, (wb0 >> (4 * h)) & 0x0F0F0F0Fu,
                               (wa1 >> (4 * h)) & 0x0F0F0F0Fu, (wb1 >> (4 * h)) & 0x0F0F0F0Fu, h ? bh0 : bl0, h ? bh1 : bl1);
            const uint32_t e = 0x4440u | (sb & 3);
            const int sA = (int)__byte_perm(scA[sb >> 2], 0, e), sB = (int)__byte_perm(scB[sb >> 2], 0, e);
            acc[0] += sA * t[0]; acc[1] += sA * t[1];
            acc[2] += sB * t[2]; acc[3] += sB * t[3];
        }
    }
}
// Sums of the activations over each 32-element sub-block (two adjacent int16 group sums, |v| <= 4064) of
// sub-blocks 4c'..4c'+3 (c' = c & 1) as byte planes v = 128 * hi + lo.  w: the eight group sums.
__device__ __forceinline__ void bsum_pair_planes(uint4 w, uint32_t &hi, uint32_t &lo) {
    const int s0 = (int)(short)(w.x & 0xffffu) + ((int)w.x >> 16), s1 = (int)(short)(w.y & 0xffffu) + ((int)w.y >> 16);
    const int s2 = (int)(short)(w.z & 0xffffu) + ((int)w.z >> 16), s3 = (int)(short)(w.w & 0xffffu) + ((int)w.w >> 16);
    lo = (uint32_t)(s0 & 127) | ((uint32_t)(s1 & 127) << 8) | ((uint32_t)(s2 & 127) << 16) | ((uint32_t)(s3 & 127) << 24);
    hi = (uint32_t)((s0 >> 7) & 255) | ((uint32_t)((s1 >> 7) & 255) << 8) | ((uint32_t)((s2 >> 7) & 255) << 16) |
         ((uint32_t)((s3 >> 7) & 255) << 24);
}

template <int TYPE> struct MmaPath { static constexpr bool kHas = false; static constexpr int kGrain = 1; };
// kGrain: half super-blocks a warp's slice must be a multiple of
template <> struct MmaPath<Q2_K> { static constexpr bool kHas = true; static constexpr int kGrain = 2; };
template <> struct MmaPath<Q3_K> { static constexpr bool kHas = true; static constexpr int kGrain = 1; };
template <> struct MmaPath<Q4_K> { static constexpr bool kHas = true; static constexpr int kGrain = 2; };

// Rows g and g+8 of a 16-row slice against the item's pairs over half-blocks [hb0, hb1): the f32 sums of
// (row g, pair 2c), (row g, pair 2c+1), (row g+8, pair 2c), (row g+8, pair 2c+1) are added into f0 (tile0)
// and, for DUAL, f1 (tile1).  Lanes with c >= MMA_NTOK / 2 return sums of repeated columns: ignore them.
// DBG (the parity hook of the integer stage): the per-super-block s32 sums of tile0 are also written to
// dbg[((row * MMA_NTOK + pair) * (I / 256) + block) * 2 + {0: scale-weighted sum, 1: min-weighted sum}]; the range
// [hb0, hb1) must then cover whole super-blocks.
// NT: pair columns the fragments are laid out for, 4 or 8; column g reads activation row min(g & (NT - 1), maxrow)
// (maxrow + 1 = the rows the stage holds).  Columns past the item's pairs read whatever those rows hold and their
// sums are never stored.
template <int TYPE, bool DUAL, bool DBG = false, int NT = MMA_NTOK>
__device__ __forceinline__ void mma_rows(uint32_t tile0, uint32_t tile1, int rb, uint32_t q8rows, int q8_stride, int I,
                                         int hb0, int hb1, int lane, float (&f0)[4], float (&f1)[4], int *dbg = nullptr,
                                         int maxrow = NT - 1) {
    auto dbg_put = [&](int b, const int (&is)[4], const int (&ms)[4]) {
        const int g_ = lane >> 2, c_ = lane & 3;
        if (2 * c_ < NT) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = g_ + 8 * (i >> 1), pair = 2 * c_ + (i & 1);
                int *o = dbg + ((size_t)(row * NT + pair) * (I / 256) + b) * 2;
                o[0] = is[i];
                o[1] = ms[i];
            }
        }
    };
    constexpr int BB = QTraits<TYPE>::kBytes;
    const int g = lane >> 2, c = lane & 3;
    const uint32_t offA = (uint32_t)g * rb, offB = (uint32_t)(g + 8) * rb;
    const uint32_t qrow = q8rows + (uint32_t)min(g & (NT - 1), maxrow) * q8_stride;   // column g's activations
    const uint32_t drow = q8rows + (uint32_t)min((2 * c) & (NT - 1), maxrow) * q8_stride + (uint32_t)Q8_BLOCK_D;
    const uint32_t drow1 = q8rows + (uint32_t)min(((2 * c) & (NT - 1)) + 1, maxrow) * q8_stride + (uint32_t)Q8_BLOCK_D;
    const uint32_t bs_off = (uint32_t)Q8_BLOCK_BS + 8 * c;
    if (TYPE == Q2_K) {
        for (int b = hb0 >> 1; b < (hb1 >> 1); ++b) {
            uint32_t bs_hi, bs_lo;
            {
                const uint2 w = lds64(qrow + bs_off + Q8_BLOCK_STRIDE * b);
                bsum_planes(w.x, w.y, bs_hi, bs_lo);
            }
            const float dx0 = __uint_as_float(lds32(drow + Q8_BLOCK_STRIDE * b)), dx1 = __uint_as_float(lds32(drow1 + Q8_BLOCK_STRIDE * b));
            const uint32_t qblk = qrow + (uint32_t)b * Q8_BLOCK_STRIDE + 4 * c;
            const uint32_t boff = (uint32_t)b * BB;
            int cm0[4], cm1[4], cx0[4], cx1[4];
            uint32_t bq[4][2];
            load_b_half<0>(qblk, bq);
            q2k_half<0, true>(tile0 + offA + boff, tile0 + offB + boff, c, bq, cm0, cx0);
            if (DUAL) q2k_half<0, true>(tile1 + offA + boff, tile1 + offB + boff, c, bq, cm1, cx1);
            load_b_half<1>(qblk, bq);
            q2k_half<1, false>(tile0 + offA + boff, tile0 + offB + boff, c, bq, cm0, cx0);
            if (DUAL) q2k_half<1, false>(tile1 + offA + boff, tile1 + offB + boff, c, bq, cm1, cx1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                cm0[i] += cx0[i] >> 2;
                if (DUAL) cm1[i] += cx1[i] >> 2;
            }
#pragma unroll
            for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
                const uint32_t rowA = (m ? tile1 : tile0) + offA + boff, rowB = (m ? tile1 : tile0) + offB + boff;
                int (&cm)[4] = m ? cm1 : cm0;
                float (&f)[4] = m ? f1 : f0;
                int cn[4];
                q2k_mins(rowA, rowB, c, bs_hi, bs_lo, cn);
                if (DBG && m == 0) dbg_put(b, cm, cn);
                const uint32_t wa = lds32(rowA + 80), wb = lds32(rowB + 80);
                const float dA = half_bits_to_float(wa), mA = half_bits_to_float(wa >> 16);
                const float dB = half_bits_to_float(wb), mB = half_bits_to_float(wb >> 16);
                f[0] = fmaf(dA * dx0, (float)cm[0], f[0]); f[0] = fmaf(-(mA * dx0), (float)cn[0], f[0]);
                f[1] = fmaf(dA * dx1, (float)cm[1], f[1]); f[1] = fmaf(-(mA * dx1), (float)cn[1], f[1]);
                f[2] = fmaf(dB * dx0, (float)cm[2], f[2]); f[2] = fmaf(-(mB * dx0), (float)cn[2], f[2]);
                f[3] = fmaf(dB * dx1, (float)cm[3], f[3]); f[3] = fmaf(-(mB * dx1), (float)cn[3], f[3]);
            }
        }
    } else if (TYPE == Q4_K) {
        for (int b = hb0 >> 1; b < (hb1 >> 1); ++b) {
            // group sums of sub-blocks 4c'..4c'+3, c' = c & 1; lanes with c >= 2 multiply them by zero mins
            uint32_t bs_hi, bs_lo;
            bsum_pair_planes(lds128(qrow + (uint32_t)q8_bs_off(b) + 16 * (c & 1)), bs_hi, bs_lo);
            const float dx0 = __uint_as_float(lds32(drow + Q8_BLOCK_STRIDE * b)), dx1 = __uint_as_float(lds32(drow1 + Q8_BLOCK_STRIDE * b));
            const uint32_t qblk = qrow + (uint32_t)b * Q8_BLOCK_STRIDE + 4 * c;
            const uint32_t boff = (uint32_t)b * BB;
#pragma unroll
            for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
                const uint32_t rowA = (m ? tile1 : tile0) + offA + boff, rowB = (m ? tile1 : tile0) + offB + boff;
                float (&f)[4] = m ? f1 : f0;
                int cm[4], hi[4], cn[4];
                uint32_t mnA[2], mnB[2];
                q4k_block(rowA, rowB, c, qblk, cm, mnA, mnB);
                // k-slots 4c..4c+3 of the k16 instruction = sub-blocks 4c..4c+3: only c = 0, 1 exist
                const uint32_t fa = c < 2 ? mnA[c & 1] : 0u, fb = c < 2 ? mnB[c & 1] : 0u;
                mma_k16_zero<false>(hi, fa, fb, bs_hi);
                mma_k16_zero<false>(cn, fa, fb, bs_lo);
                if (DBG && m == 0) {
                    const int mt[4] = {cn[0] + 128 * hi[0], cn[1] + 128 * hi[1], cn[2] + 128 * hi[2], cn[3] + 128 * hi[3]};
                    dbg_put(b, cm, mt);
                }
                const uint32_t wa = lds32(rowA), wb = lds32(rowB);
                const float dA = half_bits_to_float(wa), mA = half_bits_to_float(wa >> 16);
                const float dB = half_bits_to_float(wb), mB = half_bits_to_float(wb >> 16);
                f[0] = fmaf(dA * dx0, (float)cm[0], f[0]); f[0] = fmaf(-(mA * dx0), (float)(cn[0] + 128 * hi[0]), f[0]);
                f[1] = fmaf(dA * dx1, (float)cm[1], f[1]); f[1] = fmaf(-(mA * dx1), (float)(cn[1] + 128 * hi[1]), f[1]);
                f[2] = fmaf(dB * dx0, (float)cm[2], f[2]); f[2] = fmaf(-(mB * dx0), (float)(cn[2] + 128 * hi[2]), f[2]);
                f[3] = fmaf(dB * dx1, (float)cm[3], f[3]); f[3] = fmaf(-(mB * dx1), (float)(cn[3] + 128 * hi[3]), f[3]);
            }
        }
    } else {
        int a0[4] = {0, 0, 0, 0}, a1[4] = {0, 0, 0, 0};
        for (int hb = hb0; hb < hb1; ++hb) {
            const int b = hb >> 1;
            uint32_t bs_hi, bs_lo;
            {
                const uint2 w = lds64(qrow + bs_off + Q8_BLOCK_STRIDE * b);
                bsum_planes(w.x, w.y, bs_hi, bs_lo);
            }
            const uint32_t qblk = qrow + (uint32_t)b * Q8_BLOCK_STRIDE + 4 * c;
            const uint32_t boff = (uint32_t)b * BB;
            uint32_t bq[4][2];
            // blocks of 110 bytes: every other block starts 2 modulo 4, the same for all lanes
            const bool mis0 = (tile0 + boff) & 2u, mis1 = (tile1 + boff) & 2u;
            {
                const int nh = hb & 1;
                load_b_half<0>(qblk + (uint32_t)(2 * nh) * Q8_UNIT_STRIDE, bq);
                if (mis0) q3k_half<true>(tile0 + offA + boff, tile0 + offB + boff, c, nh, bq, bs_hi, bs_lo, a0);
                else q3k_half<false>(tile0 + offA + boff, tile0 + offB + boff, c, nh, bq, bs_hi, bs_lo, a0);
                if (DUAL) {
                    if (mis1) q3k_half<true>(tile1 + offA + boff, tile1 + offB + boff, c, nh, bq, bs_hi, bs_lo, a1);
                    else q3k_half<false>(tile1 + offA + boff, tile1 + offB + boff, c, nh, bq, bs_hi, bs_lo, a1);
                }
            }
            if ((hb & 1) == 1 || hb + 1 == hb1) {
                // the super-block (or this warp's share of it) is complete: scale into f32
                const float dx0 = __uint_as_float(lds32(drow + Q8_BLOCK_STRIDE * b)), dx1 = __uint_as_float(lds32(drow1 + Q8_BLOCK_STRIDE * b));
#pragma unroll
                for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
                    const uint32_t t = m ? tile1 : tile0;
                    int (&a)[4] = m ? a1 : a0;
                    float (&f)[4] = m ? f1 : f0;
                    if (DBG && m == 0) {
                        const int zero[4] = {0, 0, 0, 0};
                        dbg_put(b, a, zero);
                    }
                    const float dA = half_bits_to_float(lds16(t + offA + boff + 108));
                    const float dB = half_bits_to_float(lds16(t + offB + boff + 108));
                    f[0] = fmaf(dA * dx0, (float)a[0], f[0]);
                    f[1] = fmaf(dA * dx1, (float)a[1], f[1]);
                    f[2] = fmaf(dB * dx0, (float)a[2], f[2]);
                    f[3] = fmaf(dB * dx1, (float)a[3], f[3]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[i] = 0;
                }
            }
        }
    }
}

}  // namespace zmoe
