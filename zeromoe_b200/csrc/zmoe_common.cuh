// zmoe_common.cuh -- shared device helpers for the sm_100a MoE expert path:
// quantised block geometry, bulk-async (TMA engine) copies with mbarriers,
// programmatic dependent launch, alignment-agnostic shared-memory loads.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace zmoe {

// GGUF / ggml type ids (reference models/base/gguf_loader.hpp:28-51)
enum QType : int { Q2_K = 10, Q3_K = 11, Q4_K = 12, IQ2_XXS = 16 };

constexpr int QK_K = 256;

__host__ __device__ constexpr int block_bytes(int type) {
    return type == Q2_K ? 84 : type == Q3_K ? 110 : type == Q4_K ? 144 : type == IQ2_XXS ? 66 : 0;
}

// ---------------------------------------------------------------------------
// Packed activation rows.  One Q8_K-quantised row of I elements is stored block by
// block, every super-block a record of 368 bytes:
//   [ 4 units x 80 bytes | float d (padded to 16 B) | int16 bsums[16] ]
// so that one bulk copy brings a row -- or the slice of a row that a chunk of weight
// blocks meets -- to shared memory.
// Same numbers as the 292-byte ggml block (reference backends/cpu/kernels_cpu.cpp:22-26),
// regrouped.  A unit is the 64 int8 values one lane multiplies (see
// quant_units.cuh) followed by 16 bytes of padding: with a stride of 80 bytes
// the eight lanes of a quarter-warp reading 16-byte chunks of consecutive units
// fall into eight different bank groups, so the loads are conflict-free.
// Which 64 values form unit u depends on the weight format the row will meet:
//   linear: elements 64u .. 64u+63 in order;
//   planar: u = 4b + 2n + h holds elements 256b + 128n + 32j + 16h + i at byte 16j + i.
// ---------------------------------------------------------------------------
constexpr int Q8_UNIT_STRIDE = 80;
constexpr int Q8_BLOCK_STRIDE = 4 * Q8_UNIT_STRIDE + 16 + 32;   // 368
constexpr int Q8_BLOCK_D = 4 * Q8_UNIT_STRIDE;                  // d of the block
constexpr int Q8_BLOCK_BS = Q8_BLOCK_D + 16;                    // its sixteen group sums
enum Q8Layout : int { Q8_LINEAR = 0, Q8_PLANAR = 1 };
// byte offsets inside a packed row: unit u = 4b + sub, d and group sums of block b
__host__ __device__ inline int q8_unit_off(int u) { return (u >> 2) * Q8_BLOCK_STRIDE + (u & 3) * Q8_UNIT_STRIDE; }
__host__ __device__ inline int q8_d_off(int b) { return b * Q8_BLOCK_STRIDE + Q8_BLOCK_D; }
__host__ __device__ inline int q8_bs_off(int b) { return b * Q8_BLOCK_STRIDE + Q8_BLOCK_BS; }
__host__ __device__ inline int q8row_stride(int I) { return (I / QK_K) * Q8_BLOCK_STRIDE; }
__host__ __device__ constexpr int q8_layout_of(int type) { return (type == Q2_K || type == Q3_K) ? Q8_PLANAR : Q8_LINEAR; }
// byte offset inside the packed row of element e (0..255) of super-block b
__host__ __device__ inline int q8row_elem_off(int layout, int b, int e) {
    if (layout == Q8_PLANAR) {
        const int n = e >> 7, j = (e >> 5) & 3, h = (e >> 4) & 1, i = e & 15;
        return q8_unit_off(4 * b + 2 * n + h) + 16 * j + i;
    }
    return q8_unit_off(4 * b + (e >> 6)) + (e & 63);
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may hold the thread for a hardware-defined time while the phase is
// incomplete; a warp that serves several queues must not be held on one of them)
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait that lets the hardware suspend the thread for up to `ns` nanoseconds while the phase is
// incomplete: a waiting warp then takes no issue slots from the warps that do the work
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait built on it: at most `limit` suspensions of up to `ns` nanoseconds each
__device__ __forceinline__ bool mbar_wait_suspend(uint64_t *bar, uint32_t parity, uint32_t ns = 2000,
                                                  uint32_t limit = (1u << 16)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait_suspend(bar, parity, ns)) return true;
    return false;
}
// Bounded wait: gives up after `limit` polls and reports failure instead of
// spinning forever; callers raise an error flag and unwind.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 19)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// The same for warps that expect to wait long while other warps of the SM do the work: sleep
// between polls so the polling does not take issue slots from them.
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t *bar, uint32_t parity, uint32_t sleep_ns,
                                                uint32_t limit = (1u << 17)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(sleep_ns);
    }
    return false;
}

// 1-D bulk asynchronous copy global -> shared of this CTA, completion counted
// in bytes on `bar`.  Source, destination and size must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// the same with the destination given as a shared-memory address
__device__ __forceinline__ void bulk_g2s_addr(uint32_t dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// programmatic dependent launch
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------
// shared-memory loads that tolerate any byte alignment.  Quantised blocks of
// 110 and 66 bytes land on 2-byte boundaries; the tile keeps its global
// address modulo 16 in shared memory, so alignment is a property of the type.
// Reads up to 3 bytes past the last requested byte: stage buffers are padded.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
template <int ALIGN>
__device__ __forceinline__ uint32_t lds32_any(uint32_t addr) {
    if (ALIGN >= 4) return lds32(addr);
    const uint32_t base = addr & ~3u;
    const uint32_t lo = lds32(base), hi = lds32(base + 4);
    return __funnelshift_r(lo, hi, (addr & 3u) * 8);
}
// N consecutive words from an arbitrarily aligned address: N+1 aligned loads
template <int ALIGN, int N>
__device__ __forceinline__ void lds32xN_any(uint32_t addr, uint32_t (&out)[N]) {
    if (ALIGN >= 4) {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = lds32(addr + 4 * i);
    } else {
        const uint32_t base = addr & ~3u, sh = (addr & 3u) * 8;
        uint32_t prev = lds32(base);
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const uint32_t nxt = lds32(base + 4 * (i + 1));
            out[i] = __funnelshift_r(prev, nxt, sh);
            prev = nxt;
        }
    }
}

// dp4a with unsigned bytes in a, signed bytes in b
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// dp2a with signed bytes in b
__device__ __forceinline__ int dp2a_lo_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// dp2a: two signed 16-bit halves of a times two unsigned bytes of b (lo: bytes 0,1; hi: bytes 2,3)
__device__ __forceinline__ int dp2a_lo_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// low 16 bits of lo and of hi packed into one word
__device__ __forceinline__ uint32_t pack16(int lo, int hi) { return __byte_perm((uint32_t)lo, (uint32_t)hi, 0x5410); }

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}

}  // namespace zmoe
