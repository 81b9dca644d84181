// zmoe_host.hpp -- C++ host-side mirror of the reference's operator interface for the MoE
// expert path, implemented on the C ABI of libzmoe_b200.so.  Header only; link the library.
//
// Names, argument meaning and failure behaviour follow the reference:
//   CudaKernelDispatcher::matmul          reference backends/cuda/cuda_kernel_dispatcher.hpp:5-14
//   expert_ffn_gpu_issue / finish_stage1 / finish_stage2
//                                         reference core/gpu_expert_executor.hpp:42-58
//   BatchedDispatchPipeline::run          reference core/batched_dispatch_pipeline.hpp:5-14
//   GatingFunc / GGUFType ids             reference models/base/gguf_loader.hpp:28-51,177-181
// Differences, all forced by "weights resident in HBM, no CPU fallback": there is no
// ExpertLocation / residency resolution, `false` and `Abort` mean an error rather than
// "fall back to the CPU"; the per-expert issue / finish triple keeps the reference's argument lists.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/zmoe_b200.h"

namespace zmoe_host {

enum class GGUFType : int { Q8_0 = 8, Q2_K = 10, Q3_K = 11, Q4_K = 12, IQ2_XXS = 16 };
enum class GatingFunc : int { Softmax = 0, Sigmoid = 1, SqrtSoftplus = 2 };

// y[S,O] = x[S,I] . W^T on device pointers; false when the type has no kernel or the launch failed
// (the reference returns false for "unsupported", and its callers then use the CPU; here false is final)
class CudaKernelDispatcher {
public:
    static bool matmul(GGUFType type, float *y, const float *x, const void *w, int S, int I, int O) {
        switch (type) {
        case GGUFType::Q2_K: launch_q2_K_matmul(y, x, w, S, I, O); break;
        case GGUFType::Q3_K: launch_q3_K_matmul(y, x, w, S, I, O); break;
        case GGUFType::Q4_K: launch_q4_K_matmul(y, x, w, S, I, O); break;
        case GGUFType::IQ2_XXS: launch_iq2_xxs_matmul(y, x, w, S, I, O); break;
        default: return false;
        }
        return zmoe_last_status() == ZMOE_OK;
    }
};

// type and location of one projection of an expert slab (reference GGUFTensor: type + offset)
struct GGUFTensor {
    GGUFType type;
    size_t offset;   // bytes from the start of the expert's slab
};

// where an expert's slab lives (the fields of reference core/gpu_topology.hpp:191-205 this path reads):
// device_ptr points at the expert's gate tensor; up and down sit at their GGUFTensor offsets relative to gate
struct ExpertLocation {
    int gpu_id = -1;
    uint8_t *device_ptr = nullptr;
    size_t offset = 0, size = 0;
    int layer_idx = -1, expert_id = -1;
};

// the device's compute stream (the one member of the reference's GpuTopology the triple uses); release_hold is
// the reference's residency bookkeeping and has nothing to do here, where weights stay resident
class GpuTopology {
public:
    explicit GpuTopology(cudaStream_t compute_stream = nullptr) : stream_(compute_stream) {}
    cudaStream_t compute_stream(int /*gpu_id*/) const { return stream_; }
    void release_hold(int /*layer*/, int /*expert*/, const uint8_t * /*device_ptr*/, bool /*from_active_layer*/) {}

private:
    cudaStream_t stream_;
};

// device scratch of the per-expert triple (reference memory/scratch_buffers.hpp:14-35): ensure() sizes it
struct GpuExpertScratch {
    float *d_x = nullptr, *d_gate = nullptr, *d_up = nullptr, *d_prod = nullptr, *d_down = nullptr;
    int *d_bad = nullptr;   // NaN / Inf counters of the SwiGLU kernel
    size_t cap_x = 0, cap_f = 0, cap_d = 0;
    bool ensure(int S, int D, int moe_inter, int /*gpu_id*/) {
        const size_t nx = (size_t)S * D, nf = (size_t)S * moe_inter;
        auto grow = [](float **p, size_t *cap, size_t n) {
            if (n <= *cap) return true;
            cudaFree(*p);
            *cap = 0;
            if (cudaMalloc(reinterpret_cast<void **>(p), n * sizeof(float)) != cudaSuccess) { *p = nullptr; return false; }
            *cap = n;
            return true;
        };
        size_t cg = cap_f, cu = cap_f, cp = cap_f;
        bool ok = grow(&d_x, &cap_x, nx) && grow(&d_gate, &cg, nf) && grow(&d_up, &cu, nf) && grow(&d_prod, &cp, nf) &&
                  grow(&d_down, &cap_d, nx);
        cap_f = ok ? (cg < cu ? (cg < cp ? cg : cp) : (cu < cp ? cu : cp)) : 0;
        return ok;
    }
    int *ensure_bad_counter() {
        if (!d_bad && (cudaMalloc(reinterpret_cast<void **>(&d_bad), 2 * sizeof(int)) != cudaSuccess ||
                       cudaMemset(d_bad, 0, 2 * sizeof(int)) != cudaSuccess))
            d_bad = nullptr;
        return d_bad;
    }
    void release() {
        cudaFree(d_x); cudaFree(d_gate); cudaFree(d_up); cudaFree(d_prod); cudaFree(d_down); cudaFree(d_bad);
        *this = GpuExpertScratch();
    }
};

// The per-expert triple with the reference's argument lists (core/gpu_expert_executor.hpp:42-58,
// core/gpu_expert_executor.cpp:214-389, 391-515, 517-533).  Differences, all from "weights resident, no CPU
// fallback": `false` means an error, never "compute this expert on the CPU"; the activation always runs on the
// device (gate_buffer / up_buffer are not written); needs_release / location_from_active_layer are accepted and
// ignored.  The matmuls run on the legacy default stream like the reference's dispatcher calls do.

// uploads `input` (host, [S, D]; skipped when shared_device_input is given) and issues the gate and up matmuls
inline bool expert_ffn_gpu_issue(GpuExpertScratch &scratch, const ExpertLocation *location, const float *input,
                                 const GGUFTensor &gate_meta, const GGUFTensor &up_meta, int S, int D, int moe_inter,
                                 GpuTopology *topology, const float *shared_device_input = nullptr) {
    if (!location || !location->device_ptr || (!input && !shared_device_input)) return false;
    if (!scratch.ensure(S, D, moe_inter, location->gpu_id)) return false;
    const float *device_input = shared_device_input;
    if (!device_input) {
        cudaStream_t up = topology ? topology->compute_stream(location->gpu_id) : nullptr;
        if (cudaMemcpyAsync(scratch.d_x, input, (size_t)S * D * sizeof(float), cudaMemcpyHostToDevice, up) != cudaSuccess)
            return false;
        if (up && cudaStreamSynchronize(up) != cudaSuccess) return false;   // the matmuls below run on the default stream
        device_input = scratch.d_x;
    }
    const uint8_t *gate_device = location->device_ptr;
    const uint8_t *up_device = location->device_ptr + (up_meta.offset - gate_meta.offset);
    return CudaKernelDispatcher::matmul(gate_meta.type, scratch.d_gate, device_input, gate_device, S, D, moe_inter) &&
           CudaKernelDispatcher::matmul(up_meta.type, scratch.d_up, device_input, up_device, S, D, moe_inter);
}

// SwiGLU on the device (non-finite inputs counted), then the down matmul into scratch.d_down
inline void expert_ffn_gpu_finish_stage1(GpuExpertScratch &scratch, const ExpertLocation *location, float * /*gate_buffer*/,
                                         float * /*up_buffer*/, const GGUFTensor &gate_meta, const GGUFTensor &down_meta,
                                         int /*layer_idx*/, int /*expert_id*/, int S, int D, int moe_inter,
                                         float swiglu_clamp, GpuTopology * /*topology*/, bool clamp_fused = false) {
    launch_expert_swiglu(scratch.d_prod, scratch.d_gate, scratch.d_up, S * moe_inter, swiglu_clamp, clamp_fused ? 1 : 0,
                         scratch.ensure_bad_counter(), nullptr);
    const uint8_t *down_device = location->device_ptr + (down_meta.offset - gate_meta.offset);
    CudaKernelDispatcher::matmul(down_meta.type, scratch.d_down, scratch.d_prod, down_device, S, moe_inter, D);
}

// the expert's rows back to the host ([S, D]); synchronises
inline void expert_ffn_gpu_finish_stage2(const ExpertLocation *location, float *output, int layer_idx, int expert_id, int S,
                                         int D, GpuTopology *topology, bool needs_release, bool location_from_active_layer,
                                         GpuExpertScratch &scratch) {
    if (needs_release && topology)
        topology->release_hold(layer_idx, expert_id, location->device_ptr, location_from_active_layer);
    cudaMemcpy(output, scratch.d_down, (size_t)S * D * sizeof(float), cudaMemcpyDeviceToHost);
}

// weighted scatter of an expert's device rows into the layer accumulator (reference cuda_manager.hpp:1699-1773), for
// callers that keep the accumulator on the device instead of calling finish_stage2
inline void expert_scatter_accum(const GpuExpertScratch &scratch, const int *tok_dev, const float *w_dev, float *accum_dev,
                                 int n, int D, int S, void *stream = nullptr) {
    launch_expert_scatter_accum(scratch.d_down, tok_dev, w_dev, accum_dev, n, D, S, stream);
}

enum class BatchedDispatchResult { Continue, Handled, Abort };

// the fields of the reference's MoePipelineContext this path reads (core/moe_pipeline_internal.hpp:28-54)
struct MoePipelineContext {
    zmoe_layer *layer = nullptr;           // created once from the layer's weights (zmoe_layer_create)
    const float *hidden_states = nullptr;  // [S, D] host, post ffn_norm
    float *output = nullptr;               // [S, D] host
    int S = 0;
};

class BatchedDispatchPipeline {
public:
    // Handled: output holds the layer result.  Abort: an error (status in `last_status`).
    // Continue is never returned: there is no later per-token stage to hand over to.
    static BatchedDispatchResult run(MoePipelineContext &context) {
        last_status() = zmoe_moe_forward_host(context.layer, context.hidden_states, context.output, context.S);
        return last_status() == ZMOE_OK ? BatchedDispatchResult::Handled : BatchedDispatchResult::Abort;
    }
    static int &last_status() {
        static thread_local int s = ZMOE_OK;
        return s;
    }
};

}  // namespace zmoe_host
