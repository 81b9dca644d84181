// zmoe_internal.h -- host-side declarations shared by the .cu files of the
// library (not part of the public C ABI; see include/zmoe_b200.h for that).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/zmoe_b200.h"

namespace zmoe {

// ---- small host services shared by the .cu files (implemented in api.cu) ----
// multiprocessor count of the current device (cached per device); 0 on failure
int device_sm_count();
// adds to the counter behind zmoe_kernel_launches()
void count_launches(uint64_t n);
// what zmoe_last_status() returns on this thread
void set_last_status(int rc);
// raises a kernel's dynamic shared-memory limit to at least `bytes` on the current device (the attribute
// is per function and per device; remembered under a mutex)
int raise_dynamic_smem(const void *fn, size_t bytes);
// error word of the no-allocation entry point on the current device, read and cleared; 0 when that entry
// point has not run on this device (implemented in noalloc.cu)
int noalloc_take_error(int *out);

// accessors of the opaque handles for the other .cu files (implemented in api.cu)
// device pointers of the route table a layer's context currently holds, and the layer's expert count
int layer_route_table(zmoe_layer *layer, const int32_t **ids_dev, const float **weights_dev, int *n_experts);
zmoe_ctx *layer_context(zmoe_layer *layer);
int context_path(const zmoe_ctx *ctx);

// device-resident routing plan buffers
struct PlanBuffers {
    int *hdr = nullptr, *active = nullptr, *offs = nullptr, *slot = nullptr;
    int *item_offs_gu = nullptr, *item_offs_dn = nullptr, *freq = nullptr;
    int *aoffs = nullptr, *antok = nullptr;
    int *pos = nullptr;    // [P] position of each pair in expert order (inverse of slot), -1 = inactive; optional
    int cap_e = 0;
    int mt_gu = 4, mt_dn = 4;   // pairs per item of the two projections (the geometry's maxtok)
};

constexpr int ROUTER_MAX_GROUPS = 64;   // token groups (of 4) the decode router can ticket: 256 tokens

struct RouterArgs {
    const float *x;        // [T, D]
    const float *wr;       // [E, D]
    const float *bias;     // [E] or null
    int T, D, E, K;
    int gating, normalize;
    float weight_scale;
    int n_groups, n_groups_used;
    float *logits;         // [T, E] scratch; holds probabilities afterwards
    int32_t *ids;          // [T, K]
    float *weights;        // [T, K]
    uint8_t *q8x;          // packed Q8_K rows of x, [T, q8row_stride(D)]
    int q8_layout;         // unit layout of q8x (that of the gate / up weight format)
    PlanBuffers plan;
    int nrt_gu, nrt_dn;
    unsigned *ticket;      // 1 + ROUTER_MAX_GROUPS zero-initialised counters, left at zero
    bool want_q8x = true;  // large batches: also quantise x into q8x (the tensor-core path does not read it)
    float *logits_part = nullptr;  // large batches: [ROUTER_MAX_SPLIT][T, E] partial logits of a k-split router GEMM, or null
    int n_sm = 0;
    unsigned long long *stats = nullptr;   // phase timers of the decode router (builds with ZMOE_GEMM_STATS), or null
};
constexpr int ROUTER_MAX_SPLIT = 4;

// geometry of one mmid launch, fixed per (type, I, O)
struct MmidGeom {
    int lpr, upl, ncw;     // lanes per row, units per lane, consumer warps
    int R;                 // rows per tile
    int nstage, stage_bytes, wtile_bytes;
    int rbs, q8s;          // shared-memory strides of weight rows and of activation rows
    size_t smem_bytes;
    // K-chunked kernel (mmid2.cuh), chosen where the shape allows it and the caller can supply its maps
    int v2 = 0;            // 1: launch_mmid takes the K-chunked kernel; R is then 32
    int cb = 0, nch = 0;   // super-blocks per chunk, chunks per row
    int acb = 0;           // super-blocks of the activation slice a stage holds (cb, or 4 where cb is 2)
    int pitch = 0;         // bytes between rows of a chunk in shared memory
    int lb_log2 = 0;       // log2 of the lanes that share a row on the one-pair path
    int q8s_l = 0;         // bytes between the pairs' activation slices in shared memory
    int maxtok = 4;        // pairs per item (8 where the K-chunked kernel has the tensor-core path and the stages fit)
    int tiled = 0;         // chunks come through tiled maps (make_chunk_map); 0: rows are copied whole as one run
};
// allow_v2: the caller passes maps made by make_chunk_map where g->tiled is set
int mmid_geometry(int type, int I, int O, bool dual, MmidGeom *g, bool allow_v2 = false);
// Map of a [E][O rows][rb bytes] weight tensor whose box is 32 rows of `pitch` bytes starting at any multiple of 16
// bytes inside a row: bytes past the end of a row and rows past the last arrive as zeros.
int make_chunk_map(CUtensorMap *m, const void *base, int E, int O, int rb, size_t expert_stride, int pitch);

struct MmidLaunch {
    int type;
    bool dual;
    const void *w0, *w1;
    size_t stride0, stride1, total0, total1;
    int I, O;
    const uint8_t *q8;
    int xdiv;
    float *y;
    int ldy;
    PlanBuffers plan;
    bool down;             // use the down-projection item space
    float clamp;
    int clamp_fused;
    int *err;
    int *bad = nullptr;    // [2] NaN / Inf counters of the fused SwiGLU epilogue, or null
    int *queue = nullptr;  // [4] zeroed ints: the chunked kernel deals its items through a ticket counter (two ints per
                           // projection, left zero by every launch); null = items dealt round-robin over the grid
    int n_sm;
    bool multi = false;    // some expert may hold two or more pairs: allow the tensor-core consumer path
    // optional tiled maps of w0 / w1 (make_rows_map) that deliver tiles with padded rows in one copy
    const CUtensorMap *tm0 = nullptr, *tm1 = nullptr;
};
// Map of a [E][O rows][rb bytes] weight tensor whose box is R rows of rb + 16 bytes: the 16 bytes past the
// end of a row are out of bounds and arrive as zeros, which pads the rows in shared memory.  Rows up to 2032 bytes.
int make_rows_map(CUtensorMap *m, const void *base, int E, int O, int rb, size_t expert_stride, int R);
// dst[i] = (float)src[i] for n bf16 values (n a multiple of 8, both 16-byte aligned)
int launch_widen_bf16(const void *src, float *dst, long n, int n_sm, cudaStream_t st);
// g[t] = sigmoid(w . x[t]) for T rows of D floats (D a multiple of 4)
int launch_token_gate(const float *x, const float *w, float *g, int T, int D, cudaStream_t st);
int launch_mmid(const MmidLaunch &L, const MmidGeom &g, cudaStream_t st);
// s32 sums of the tensor-core consumer path: out[16 rows][4 pair slots][I / 256][2]
int launch_mma_isums(int type, const void *w, const uint8_t *q8, int *out, int I, int pairs, cudaStream_t st);

// prefill path: tcgen05 grouped GEMM over fp16 activations (Q8_K round trip applied, rows scaled)
struct GemmLaunch {
    int type;
    bool dual;
    const void *w0, *w1;
    size_t stride0, stride1;
    int n_experts;         // experts the weight tensors hold
    int I, O;
    const void *x_f16;     // sorted activation rows [x_rows, I] fp16
    const float *xscale;   // their per-row scales
    int x_rows;            // rows the buffer holds
    float *y;
    int ldy;
    PlanBuffers plan;
    float clamp;
    int clamp_fused;
    int *err;
    int *bad = nullptr;    // [2] NaN / Inf counters of the fused SwiGLU epilogue, or null
    int n_sm;
};
bool gemm_sm100_supported(int type, int I, int O);
unsigned long long *gemm_stats_buffer(int which);
int gemm_stats_read(unsigned long long *out32);
int launch_gemm_sm100(const GemmLaunch &L, cudaStream_t st);
int launch_q8_roundtrip_f16(const float *x, int ldx, void *out_f16, float *scale, const PlanBuffers &plan,
                            int max_rows, int xdiv, int I, cudaStream_t st);
// the same for the layer input, where the K pairs of a token share one source row: the row is passed through
// Q8_K once and written to the K positions plan.pos names (needs plan.pos)
int launch_q8_roundtrip_tokens_f16(const float *x, int ldx, void *out_f16, float *scale, const PlanBuffers &plan,
                                   int T, int K, int I, cudaStream_t st);

int launch_router_decode(const RouterArgs &a, cudaStream_t st);
int launch_router_prefill(const RouterArgs &a, cudaStream_t st);  // four launches; for large T
// the planner, first copying routes from outside into the context's tables (ids, w); window: expert numbers
// outside [first, first + E) become -1
int launch_plan_ingest(const int32_t *src_ids, const float *src_w, int32_t *ids, float *w, int P, int E, int first,
                       bool window, const PlanBuffers &plan, int nrt_gu, int nrt_dn, cudaStream_t st, int topk = 0, int ids_ld = 0, int w_ld = 0);
int launch_plan_from_ids(const int32_t *ids, int P, int E, const PlanBuffers &plan, int nrt_gu, int nrt_dn,
                         cudaStream_t st);
int launch_plan_dense(int S, const PlanBuffers &plan, int nrt, cudaStream_t st);
int launch_quantize_rows(const float *x, int ldx, uint8_t *q8, int rows, int I, int layout, cudaStream_t st);
int launch_q8rows_to_blocks(const uint8_t *q8, uint8_t *blocks, int rows, int I, int layout, cudaStream_t st);
int launch_combine(float *out, const float *y, const float *w, const int32_t *ids, int T, int K, int D, int E,
                   int accumulate, cudaStream_t st);
int launch_block_isums(int type, const void *w, const uint8_t *q8, int32_t *isum, int32_t *msum, int rows, int I,
                       cudaStream_t st);

// launch helper: programmatic dependent launch attribute on every kernel of the chain
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace zmoe
