// noalloc.cu -- a dense quantised matmul entry point that never allocates.
//
// Some hosts of this library cannot allocate device memory at the moment they
// need a matmul: an inference engine that handed the whole GPU to its own pool
// allocator at start-up, a plug-in running inside another framework's stream
// capture (where cudaMalloc is illegal), or a real-time loop that may not take
// the allocator lock.  The other entry points keep their quantised-activation
// and planning scratch in cudaMalloc'ed buffers that grow on demand; this one
// keeps the same scratch in a fixed array that is part of the library image.
//
// The price: the array has a fixed size (ZMOE_NOALLOC_SCRATCH_BYTES, reserved on
// every GPU that loads the library, until the process exits), larger problems
// are refused, and all calls share the one array, so two calls whose kernels
// may overlap on the GPU (different streams, no ordering between them) race.
#include <mutex>

#include "zmoe_common.cuh"
#include "zmoe_internal.h"

using namespace zmoe;

namespace {

constexpr size_t kScratchBytes = ZMOE_NOALLOC_SCRATCH_BYTES;

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be passed
// to a kernel; the address each device gave is cached in g_base below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char *g_base[kMaxDevices] = {};
std::mutex g_mu;

// fixed offsets of the small planning arrays inside the scratch
constexpr size_t kOffErr = 0, kOffHdr = 64, kOffActive = 128, kOffOffs = 192, kOffItemsGu = 256, kOffItemsDn = 320,
                 kOffAoffs = 384, kOffAntok = 448, kOffSlot = 512;

// once per device, with that device current: ask the runtime where the array lives
int scratch_base(unsigned char **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ZMOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_base[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return ZMOE_ERR_CUDA;
        g_base[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_base[dev];
    return ZMOE_OK;
}

}  // namespace

extern "C" int zmoe_matmul_noalloc(int type, float *y, const float *x, const void *w, int S, int I, int O,
                                   void *stream) {
    if (!y || !x || !w || S <= 0 || I <= 0 || O <= 0) return ZMOE_ERR_ARG;
    MmidGeom g;
    int rc = mmid_geometry(type, I, O, false, &g);
    if (rc) return rc;
    // what this problem needs: pair slots, then the packed Q8_K rows of x
    const size_t slot_bytes = ((size_t)S * sizeof(int) + 255) & ~(size_t)255;
    const size_t q8_off = kOffSlot + slot_bytes;
    const size_t need = q8_off + (size_t)S * q8row_stride(I);
    if (need > kScratchBytes) return ZMOE_ERR_CAPACITY;
    unsigned char *base = nullptr;
    rc = scratch_base(&base);
    if (rc) return rc;
    int n_sm = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0)
        return ZMOE_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the array keeps whatever the last call left: the plan header must start at zero.  The error word in
    // front of it is left alone: it stays set until zmoe_device_status() has reported and cleared it.
    if (cudaMemsetAsync(base + kOffHdr, 0, kOffSlot - kOffHdr, st) != cudaSuccess) return ZMOE_ERR_CUDA;
    PlanBuffers plan;
    plan.hdr = reinterpret_cast<int *>(base + kOffHdr);
    plan.active = reinterpret_cast<int *>(base + kOffActive);
    plan.offs = reinterpret_cast<int *>(base + kOffOffs);
    plan.item_offs_gu = reinterpret_cast<int *>(base + kOffItemsGu);
    plan.item_offs_dn = reinterpret_cast<int *>(base + kOffItemsDn);
    plan.aoffs = reinterpret_cast<int *>(base + kOffAoffs);
    plan.antok = reinterpret_cast<int *>(base + kOffAntok);
    plan.slot = reinterpret_cast<int *>(base + kOffSlot);
    plan.freq = nullptr;
    plan.cap_e = 1;
    uint8_t *q8 = base + q8_off;
    const int nrt = (O + g.R - 1) / g.R;
    rc = launch_quantize_rows(x, I, q8, S, I, q8_layout_of(type), st);
    if (!rc) rc = launch_plan_dense(S, plan, nrt, st);
    if (rc) return rc;
    MmidLaunch m;
    m.type = type; m.dual = false;
    m.w0 = w; m.w1 = nullptr;
    m.stride0 = 0; m.stride1 = 0;
    m.total0 = (size_t)O * (I / QK_K) * block_bytes(type); m.total1 = 0;
    m.I = I; m.O = O;
    m.q8 = q8; m.xdiv = 1;
    m.y = y; m.ldy = O;
    m.plan = plan;
    m.down = false;
    m.clamp = 0.f; m.clamp_fused = 0;
    m.err = reinterpret_cast<int *>(base + kOffErr);
    m.n_sm = n_sm;
    m.multi = S > 1;
    count_launches(3);
    return launch_mmid(m, g, st);
}

// the error word of this device's array, read and cleared (the caller has synchronised the device)
int zmoe::noalloc_take_error(int *out) {
    *out = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ZMOE_ERR_CUDA;
    unsigned char *base;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        base = g_base[dev];
    }
    if (!base) return ZMOE_OK;   // the entry point has not run here: nothing to report
    if (cudaMemcpy(out, base + kOffErr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ZMOE_ERR_CUDA;
    if (*out && cudaMemset(base + kOffErr, 0, sizeof(int)) != cudaSuccess) return ZMOE_ERR_CUDA;
    return ZMOE_OK;
}
