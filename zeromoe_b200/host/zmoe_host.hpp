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
// "fall back to the CPU", and the per-expert issue/finish triple works on a one-expert view.
#pragma once

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

// device scratch of the per-expert triple (reference memory/scratch_buffers.hpp:14-35)
struct GpuExpertScratch {
    float *d_x = nullptr, *d_gate = nullptr, *d_up = nullptr, *d_prod = nullptr, *d_down = nullptr;
    int *d_bad = nullptr;   // NaN / Inf counters of the SwiGLU kernel
};

// gate and up matmuls of one expert for S rows already on the device in scratch.d_x
inline bool expert_ffn_gpu_issue(GpuExpertScratch &scratch, const uint8_t *slab_dev, const GGUFTensor &gate_meta,
                                 const GGUFTensor &up_meta, int S, int D, int moe_inter) {
    return CudaKernelDispatcher::matmul(gate_meta.type, scratch.d_gate, scratch.d_x, slab_dev + gate_meta.offset, S, D,
                                        moe_inter) &&
           CudaKernelDispatcher::matmul(up_meta.type, scratch.d_up, scratch.d_x, slab_dev + up_meta.offset, S, D,
                                        moe_inter);
}
// SwiGLU on the device, then the down matmul
inline bool expert_ffn_gpu_finish_stage1(GpuExpertScratch &scratch, const uint8_t *slab_dev,
                                         const GGUFTensor &down_meta, int S, int D, int moe_inter, float swiglu_clamp,
                                         bool clamp_fused, void *stream = nullptr) {
    launch_expert_swiglu(scratch.d_prod, scratch.d_gate, scratch.d_up, S * moe_inter, swiglu_clamp, clamp_fused ? 1 : 0,
                         scratch.d_bad, stream);
    return CudaKernelDispatcher::matmul(down_meta.type, scratch.d_down, scratch.d_prod, slab_dev + down_meta.offset, S,
                                        moe_inter, D);
}
// weighted scatter of the expert's rows into the layer accumulator (reference cuda_manager.hpp:1699-1773)
inline void expert_ffn_gpu_finish_stage2(const GpuExpertScratch &scratch, const int *tok_dev, const float *w_dev,
                                         float *accum_dev, int n, int D, int S, void *stream = nullptr) {
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
