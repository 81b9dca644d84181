// dequant_f16.cuh -- 32 consecutive weights of a quantised row -> 32 fp16 values (four
// 16-byte chunks).  Used by the prefill grouped GEMM to build its A tiles in shared memory.
//
// Split in two: load_raw_s<TYPE> fetches the 32 weights' bytes from a copy of the super-block in
// shared memory (the grouped GEMM stages raw blocks there with the TMA engine), load_raw<TYPE>
// does the same from global memory, convert_raw<TYPE> turns them into fp16.  Values follow the reference dequantisers (reference
// kernels/quant/kquant_matmul.cu:55-92,179-199, kernels/quant/iq2_matmul.cu:73-91):
// d*sc*q - dmin*m, d*(sc-32)*q3, d*(0.5+ls)*0.25*grid*sign; Q4_K and IQ2_XXS are assembled
// directly in fp16: the integer part is exact, the block scale is rounded to fp16 once.
#pragma once

#include "quant_units.cuh"
#include "umma.cuh"

namespace zmoe {

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ uint32_t ldg_u32_a2(const uint8_t *p) {  // 2-byte aligned 32-bit load
    return ldg_u16(p) | (ldg_u16(p + 2) << 16);
}

// tables the converters read from shared memory
struct DequantTables {
    uint32_t grid;   // shared address of the IQ2_XXS selector table: 256 entries x IQ2_TABLE_COPIES copies x 8 bytes
};

// Entry e of the table: four 16-bit byte-permute selectors, one per pair of elements (2p, 2p+1).  With
// i0, i1 the codes (0, 1, 2 for the magnitudes 8, 25, 43: their high nibbles) of the two elements, the
// selector's nibbles are (2 i0, 2 i0 + 1, 2 i1, 2 i1 + 1): the two bytes of each fp16 table entry.
// The table is kept in IQ2_TABLE_COPIES copies, entry e of copy c at index e * COPIES + c: lane l reads copy l % 16,
// so the sixteen lanes of a half-warp's 8-byte loads always fall into sixteen different bank pairs whatever
// entries the data asks for (one copy gave about three wavefronts per load from the data-dependent indices).
constexpr int IQ2_TABLE_COPIES = 16;
__device__ __forceinline__ void dequant_fill_tables(uint2 *grid_s) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint64_t g = k_iq2xxs_grid[i];
        uint32_t w[4];
        for (int pp = 0; pp < 4; ++pp) {
            const uint32_t i0 = (uint32_t)(g >> (16 * pp + 4)) & 3u, i1 = (uint32_t)(g >> (16 * pp + 12)) & 3u;
            w[pp] = 0x1010u + 0x22u * (i0 + 256u * i1);
        }
        const uint2 v = make_uint2(w[0] | (w[1] << 16), w[2] | (w[3] << 16));
        for (int c = 0; c < IQ2_TABLE_COPIES; ++c) grid_s[i * IQ2_TABLE_COPIES + c] = v;
    }
}

template <int TYPE> struct RawW;
template <> struct RawW<IQ2_XXS> { uint32_t aux0, aux1, d; };
template <> struct RawW<Q4_K> { uint4 q0, q1; uint32_t dd, s0, s1, s2; };
template <> struct RawW<Q2_K> { uint32_t w[8]; uint32_t sc, dd; };
template <> struct RawW<Q3_K> { uint32_t q[8], hm[8]; uint32_t a0, a1, tmp, d; };

// row: first byte of the weight row; k0: multiple of 32
template <int TYPE>
__device__ __forceinline__ void load_raw(const uint8_t *__restrict__ row, int k0, RawW<TYPE> &r);

template <>
__device__ __forceinline__ void load_raw<IQ2_XXS>(const uint8_t *__restrict__ row, int k0, RawW<IQ2_XXS> &r) {
    const uint8_t *blk = row + (size_t)(k0 >> 8) * 66;     // d @0, qs u16[32] @2, 2-byte aligned
    const int ib = (k0 & 255) >> 5;
    r.d = ldg_u16(blk);
    r.aux0 = ldg_u32_a2(blk + 2 + 8 * ib);
    r.aux1 = ldg_u32_a2(blk + 6 + 8 * ib);
}
template <>
__device__ __forceinline__ void load_raw<Q4_K>(const uint8_t *__restrict__ row, int k0, RawW<Q4_K> &r) {
    const uint8_t *blk = row + (size_t)(k0 >> 8) * 144;    // d @0, dmin @2, scales[12] @4, qs[128] @16
    const int c = (k0 & 255) >> 6;
    r.dd = *reinterpret_cast<const uint32_t *>(blk);
    r.s0 = *reinterpret_cast<const uint32_t *>(blk + 4);
    r.s1 = *reinterpret_cast<const uint32_t *>(blk + 8);
    r.s2 = *reinterpret_cast<const uint32_t *>(blk + 12);
    r.q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
    r.q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * c);
}
template <>
__device__ __forceinline__ void load_raw<Q2_K>(const uint8_t *__restrict__ row, int k0, RawW<Q2_K> &r) {
    const uint8_t *blk = row + (size_t)(k0 >> 8) * 84;     // scales[16] @0, qs[64] @16, d @80, dmin @82
    const int n = (k0 & 255) >> 7, j = (k0 & 127) >> 5;
    r.dd = *reinterpret_cast<const uint32_t *>(blk + 80);
    r.sc = ldg_u16(blk + 8 * n + 2 * j);
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * n + 4 * i);
}
template <>
__device__ __forceinline__ void load_raw<Q3_K>(const uint8_t *__restrict__ row, int k0, RawW<Q3_K> &r) {
    const uint8_t *blk = row + (size_t)(k0 >> 8) * 110;    // hmask[32] @0, qs[64] @32, scales[12] @96, d @108
    const int n = (k0 & 255) >> 7;
    r.d = ldg_u16(blk + 108);
    r.a0 = ldg_u32_a2(blk + 96); r.a1 = ldg_u32_a2(blk + 100); r.tmp = ldg_u32_a2(blk + 104);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        r.q[i] = ldg_u32_a2(blk + 32 + 32 * n + 4 * i);
        r.hm[i] = ldg_u32_a2(blk + 4 * i);
    }
}

// The same fields from a copy of the super-block in shared memory.  blk: shared address of the block's
// first byte (alignment as in the tensor: 2, 4 or 16 bytes by type); kin: offset of the 32 weights inside
// the super-block (multiple of 32).
template <int TYPE>
__device__ __forceinline__ void load_raw_s(uint32_t blk, int kin, RawW<TYPE> &r);

template <>
__device__ __forceinline__ void load_raw_s<IQ2_XXS>(uint32_t blk, int kin, RawW<IQ2_XXS> &r) {
    uint32_t a[2];
    lds32xN_any<2, 2>(blk + 2 + 8 * (kin >> 5), a);
    r.aux0 = a[0]; r.aux1 = a[1];
    r.d = lds16(blk);
}
template <>
__device__ __forceinline__ void load_raw_s<Q4_K>(uint32_t blk, int kin, RawW<Q4_K> &r) {
    const uint4 h = lds128(blk);
    r.dd = h.x; r.s0 = h.y; r.s1 = h.z; r.s2 = h.w;
    const int c = kin >> 6;
    r.q0 = lds128(blk + 16 + 32 * c);
    r.q1 = lds128(blk + 32 + 32 * c);
}
template <>
__device__ __forceinline__ void load_raw_s<Q2_K>(uint32_t blk, int kin, RawW<Q2_K> &r) {
    const int n = kin >> 7, j = (kin & 127) >> 5;
    r.dd = lds32(blk + 80);
    r.sc = lds16(blk + 8 * n + 2 * j);
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = lds32(blk + 16 + 32 * n + 4 * i);
}
template <>
__device__ __forceinline__ void load_raw_s<Q3_K>(uint32_t blk, int kin, RawW<Q3_K> &r) {
    const int n = kin >> 7;
    r.d = lds16(blk + 108);
    uint32_t sc[3];
    lds32xN_any<2, 3>(blk + 96, sc);
    r.a0 = sc[0]; r.a1 = sc[1]; r.tmp = sc[2];
    lds32xN_any<2, 8>(blk + 32 + 32 * n, r.q);
    lds32xN_any<2, 8>(blk, r.hm);
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

template <int TYPE>
__device__ __forceinline__ void convert_raw(const RawW<TYPE> &r, int k0, const DequantTables &tb, uint4 (&out)[4]);

// IQ2_XXS: the codebook holds only the magnitudes 8, 25 and 43, which index a three-entry fp16 table
// (the magnitudes times the sub-block scale) kept in a register pair; one byte permute per pair of
// elements assembles the values.  The shared-memory copy of the codebook holds, per entry, the four
// ready-made permute selectors (16 bits each) instead of the magnitudes: the converters are bound by
// instruction issue, and this takes the selector arithmetic out of the loop.
template <>
__device__ __forceinline__ void convert_raw<IQ2_XXS>(const RawW<IQ2_XXS> &r, int k0, const DequantTables &tb,
                                                     uint4 (&out)[4]) {
    const float db = __fmul_rn(__fmul_rn(half_bits_to_float(r.d), 0.5f + (float)(r.aux1 >> 28)), 0.25f);
    const uint32_t t0 = h2_bits(__floats2half2_rn(db * 8.f, db * 25.f));   // entries 0, 1
    const uint32_t t1 = h2_bits(__floats2half2_rn(db * 43.f, 0.f));        // entry 2
#pragma unroll
    for (int l = 0; l < 4; ++l) {
        const uint2 sel = lds64(tb.grid + 8 * (IQ2_TABLE_COPIES * ((r.aux0 >> (8 * l)) & 255u) + (threadIdx.x & (IQ2_TABLE_COPIES - 1))));
        // Sign bits of the eight elements: the seven stored ones and their parity (even number of minus
        // signs per group of eight).  Bit 2p goes to bit 15 and bit 2p+1 to bit 31 of word p with one
        // multiplication: s * (0x40008000 >> 2p) puts bit k of s at k + 15 - 2p and at k + 30 - 2p, the two
        // ranges never overlap (no carries), and the mask keeps bits 15 and 31.
        const uint32_t s7 = (r.aux1 >> (7 * l)) & 127u;
        const uint32_t s8 = s7 | ((__popc(s7) & 1u) << 7);
        // the permute reads only the low 16 bits of its selector
        out[l].x = __byte_perm(t0, t1, sel.x) ^ ((s8 * 0x40008000u) & 0x80008000u);
        out[l].y = __byte_perm(t0, t1, sel.x >> 16) ^ ((s8 * 0x10002000u) & 0x80008000u);
        out[l].z = __byte_perm(t0, t1, sel.y) ^ ((s8 * 0x04000800u) & 0x80008000u);
        out[l].w = __byte_perm(t0, t1, sel.y >> 16) ^ ((s8 * 0x01000200u) & 0x80008000u);
    }
}

// Q4_K: nibble | 0x6400 is the fp16 number 1024 + q; subtracting 1024 is exact, then one fused
// multiply-add per pair gives q * dl - ml.
template <>
__device__ __forceinline__ void convert_raw<Q4_K>(const RawW<Q4_K> &r, int k0, const DequantTables &tb,
                                                  uint4 (&out)[4]) {
    const int s = (k0 & 255) >> 5, hi = s & 1;
    const float d = half_bits_to_float(r.dd), dmin = half_bits_to_float(r.dd >> 16);
    // scale / min pair s (reference kernels/quant/kquant_matmul.cu:41-48)
    const int sh = 8 * (s & 3);
    int scv, mv;
    if (s < 4) {
        scv = (r.s0 >> sh) & 63;
        mv = (r.s1 >> sh) & 63;
    } else {
        const uint32_t b = (r.s2 >> sh) & 0xffu;
        scv = (int)((b & 0xFu) | ((((r.s0 >> sh) & 0xffu) >> 6) << 4));
        mv = (int)((b >> 4) | ((((r.s1 >> sh) & 0xffu) >> 6) << 4));
    }
    const float dl = d * (float)scv, ml = dmin * (float)mv;
    const __half2 dl2 = __float2half2_rn(dl);
    const __half2 off2 = __float2half2_rn(-ml);
    const __half2 k1024 = bits_h2(0x64006400u);
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const uint32_t x = hi ? (w[m] >> 4) : w[m];
        // bytes 0 and 2 / bytes 1 and 3 as (1024 + q) pairs
        const uint32_t e02 = (x & 0x000F000Fu) | 0x64006400u;
        const uint32_t e13 = ((x >> 8) & 0x000F000Fu) | 0x64006400u;
        const uint32_t v02 = h2_bits(__hfma2(__hsub2(bits_h2(e02), k1024), dl2, off2));
        const uint32_t v13 = h2_bits(__hfma2(__hsub2(bits_h2(e13), k1024), dl2, off2));
        const uint32_t p01 = __byte_perm(v02, v13, 0x5410u), p23 = __byte_perm(v02, v13, 0x7632u);
        uint32_t *o = reinterpret_cast<uint32_t *>(&out[m >> 1]);
        o[2 * (m & 1)] = p01;
        o[2 * (m & 1) + 1] = p23;
    }
}

template <>
__device__ __forceinline__ void convert_raw<Q2_K>(const RawW<Q2_K> &r, int k0, const DequantTables &tb,
                                                  uint4 (&out)[4]) {
    const int j = (k0 & 127) >> 5;
    const float d = half_bits_to_float(r.dd), dmin = half_bits_to_float(r.dd >> 16);
    const uint32_t s0 = r.sc & 0xffu, s1 = (r.sc >> 8) & 0xffu;
    // same trick as Q4_K with two-bit fields
    const __half2 dl0 = __float2half2_rn(d * (float)(s0 & 0xFu)), dl1 = __float2half2_rn(d * (float)(s1 & 0xFu));
    const __half2 of0 = __float2half2_rn(-(dmin * (float)(s0 >> 4)));
    const __half2 of1 = __float2half2_rn(-(dmin * (float)(s1 >> 4)));
    const __half2 k1024 = bits_h2(0x64006400u);
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const uint32_t x = r.w[m] >> (2 * j);
        const uint32_t e02 = (x & 0x00030003u) | 0x64006400u;
        const uint32_t e13 = ((x >> 8) & 0x00030003u) | 0x64006400u;
        const __half2 dl = m < 4 ? dl0 : dl1, of = m < 4 ? of0 : of1;
        const uint32_t v02 = h2_bits(__hfma2(__hsub2(bits_h2(e02), k1024), dl, of));
        const uint32_t v13 = h2_bits(__hfma2(__hsub2(bits_h2(e13), k1024), dl, of));
        uint32_t *o = reinterpret_cast<uint32_t *>(&out[m >> 1]);
        o[2 * (m & 1)] = __byte_perm(v02, v13, 0x5410u);
        o[2 * (m & 1) + 1] = __byte_perm(v02, v13, 0x7632u);
    }
}

template <>
__device__ __forceinline__ void convert_raw<Q3_K>(const RawW<Q3_K> &r, int k0, const DequantTables &tb,
                                                  uint4 (&out)[4]) {
    const int n = (k0 & 255) >> 7, j = (k0 & 127) >> 5;
    const float d = half_bits_to_float(r.d);
    __half2 dl[2];
    const __half2 k1028 = bits_h2(0x64046404u);    // 1028: (1024 + (q2 | hb << 2)) - 1028 = q3, exact
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int k = 8 * n + 2 * j + h;
        uint32_t lo = (((k & 4) ? r.a1 : r.a0) >> (8 * (k & 3))) & 0xffu;
        lo = k < 8 ? (lo & 0xFu) : (lo >> 4);
        const uint32_t hi2 = (r.tmp >> (8 * (k & 3) + 2 * (k >> 2))) & 3u;
        const float s = d * (float)((int)(lo | (hi2 << 4)) - 32);
        dl[h] = __float2half2_rn(s);
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const uint32_t q = (r.q[m] >> (2 * j)) & 0x03030303u;
        const uint32_t hb = ((r.hm[m] >> (4 * n + j)) & 0x01010101u) << 2;
        const uint32_t x = q | hb;                 // bytes 0..7
        const uint32_t e02 = (x & 0x00070007u) | 0x64006400u;
        const uint32_t e13 = ((x >> 8) & 0x00070007u) | 0x64006400u;
        const uint32_t v02 = h2_bits(__hmul2(__hsub2(bits_h2(e02), k1028), dl[m >> 2]));
        const uint32_t v13 = h2_bits(__hmul2(__hsub2(bits_h2(e13), k1028), dl[m >> 2]));
        uint32_t *o = reinterpret_cast<uint32_t *>(&out[m >> 1]);
        o[2 * (m & 1)] = __byte_perm(v02, v13, 0x5410u);
        o[2 * (m & 1) + 1] = __byte_perm(v02, v13, 0x7632u);
    }
}

}  // namespace zmoe
