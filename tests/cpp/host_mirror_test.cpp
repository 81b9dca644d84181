// Drives the C++ host mirror the way the reference's native tests drive its dispatcher
// (tests/native/tests_basic_cuda.cpp:141-279: quantised matmul against a CPU reference with
// |a-b| <= 1e-4 + 0.01 |ref|, here on exactly representable activations so that the reference's
// f32 dequantise-and-dot and this library's Q8_K arithmetic agree).  Prints PASS / FAIL lines.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "../../oracle/zmoe_oracle.h"
#include "../../zeromoe_b200/host/zmoe_host.hpp"

using namespace zmoe_host;

static std::vector<uint8_t> random_blocks(int type, size_t nblocks, std::mt19937 &rng) {
    const size_t bb = zo_block_bytes(type);
    std::vector<uint8_t> w(nblocks * bb);
    for (auto &b : w) b = (uint8_t)rng();
    // plausible fp16 super-scales (0.002 .. 0.03) at the format's offsets
    auto put = [&](size_t blk, size_t off) { const uint16_t h = 0x1C00 + (rng() % 0x0A00); w[blk * bb + off] = h & 0xff; w[blk * bb + off + 1] = h >> 8; };
    for (size_t i = 0; i < nblocks; ++i) {
        if (type == ZO_TYPE_Q2_K) { put(i, 80); put(i, 82); }
        else if (type == ZO_TYPE_Q3_K) put(i, 108);
        else if (type == ZO_TYPE_Q4_K) { put(i, 0); put(i, 2); }
        else put(i, 0);
    }
    return w;
}

static bool check_matmul(GGUFType type, int I, int O, int S) {
    std::mt19937 rng(42);
    const int t = (int)type;
    auto w = random_blocks(t, (size_t)O * (I / 256), rng);
    std::vector<float> x((size_t)S * I), ref((size_t)S * O), got((size_t)S * O), deq(I);
    for (int s = 0; s < S; ++s)
        for (int i = 0; i < I; ++i) x[(size_t)s * I + i] = (i % 256 == 0) ? -127.f : (float)((int)(rng() % 255) - 127);
    const size_t rb = (size_t)(I / 256) * zo_block_bytes(t);
    for (int o = 0; o < O; ++o) {
        zo_dequantize_row(t, w.data() + o * rb, deq.data(), I);
        for (int s = 0; s < S; ++s) {
            double a = 0;
            for (int i = 0; i < I; ++i) a += (double)deq[i] * x[(size_t)s * I + i];
            ref[(size_t)s * O + o] = (float)a;
        }
    }
    float *dx, *dy; void *dw;
    cudaMalloc(&dx, x.size() * 4); cudaMalloc(&dy, got.size() * 4); cudaMalloc(&dw, w.size());
    cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dw, w.data(), w.size(), cudaMemcpyHostToDevice);
    const bool ok = CudaKernelDispatcher::matmul(type, dy, dx, dw, S, I, O);
    cudaDeviceSynchronize();
    cudaMemcpy(got.data(), dy, got.size() * 4, cudaMemcpyDeviceToHost);
    cudaFree(dx); cudaFree(dy); cudaFree(dw);
    if (!ok) return false;
    for (size_t i = 0; i < got.size(); ++i)
        if (std::fabs(got[i] - ref[i]) > 1e-4f + 0.01f * std::fabs(ref[i])) {
            std::printf("  mismatch at %zu: %g vs %g\n", i, got[i], ref[i]);
            return false;
        }
    return true;
}

// one expert through the issue / finish triple, slab = [gate | up | down], host input and host output, against the
// oracle's layer with that one expert
static bool check_triple() {
    std::mt19937 rng(7);
    const int D = 512, F = 256, S = 3;
    const int tg = ZO_TYPE_Q2_K, td = ZO_TYPE_Q3_K;
    auto wg = random_blocks(tg, (size_t)F * (D / 256), rng), wu = random_blocks(tg, (size_t)F * (D / 256), rng);
    auto wd = random_blocks(td, (size_t)D * (F / 256), rng);
    std::vector<uint8_t> slab;
    slab.insert(slab.end(), wg.begin(), wg.end());
    slab.insert(slab.end(), wu.begin(), wu.end());
    slab.insert(slab.end(), wd.begin(), wd.end());
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> x((size_t)S * D), ref((size_t)S * D), got((size_t)S * D);
    for (auto &v : x) v = nd(rng);
    std::vector<int32_t> ids(S, 0);
    std::vector<float> w(S, 1.0f);
    zo_layer L = {D, F, 1, 1, tg, tg, td, wg.data(), wu.data(), wd.data(), wg.size(), wu.size(), wd.size(), 0.0f, 0};
    zo_moe_ffn(&L, x.data(), ids.data(), w.data(), S, ref.data(), nullptr);
    uint8_t *dslab = nullptr;
    cudaMalloc(&dslab, slab.size() + 64);
    cudaMemcpy(dslab, slab.data(), slab.size(), cudaMemcpyHostToDevice);
    ExpertLocation loc;
    loc.gpu_id = 0; loc.device_ptr = dslab; loc.size = slab.size(); loc.layer_idx = 0; loc.expert_id = 0;
    const GGUFTensor gate_meta{GGUFType::Q2_K, 1000}, up_meta{GGUFType::Q2_K, 1000 + wg.size()},
        down_meta{GGUFType::Q3_K, 1000 + wg.size() + wu.size()};   // offsets inside the file-side slab; only differences count
    GpuTopology topo;
    GpuExpertScratch scratch;
    bool ok = expert_ffn_gpu_issue(scratch, &loc, x.data(), gate_meta, up_meta, S, D, F, &topo);
    if (ok) {
        expert_ffn_gpu_finish_stage1(scratch, &loc, nullptr, nullptr, gate_meta, down_meta, 0, 0, S, D, F, 0.0f, &topo);
        expert_ffn_gpu_finish_stage2(&loc, got.data(), 0, 0, S, D, &topo, true, false, scratch);
    }
    ok = ok && zmoe_last_status() == ZMOE_OK;
    double m = 0, n = 0;
    for (size_t i = 0; i < got.size(); ++i) { m = std::fmax(m, std::fabs((double)got[i] - ref[i])); n += (double)ref[i] * ref[i]; }
    if (m / (std::sqrt(n) + 1e-30) > 1e-3) { std::printf("  triple error/norm %.3e\n", m / std::sqrt(n)); ok = false; }
    // a missing location is an error, not a CPU fallback
    ok = ok && !expert_ffn_gpu_issue(scratch, nullptr, x.data(), gate_meta, up_meta, S, D, F, &topo);
    scratch.release();
    cudaFree(dslab);
    return ok;
}

int main() {
    int fails = 0;
    struct { GGUFType t; int I, O, S; const char *name; } cases[] = {
        {GGUFType::Q2_K, 512, 8, 3, "Q2_K 512x8 S=3"},     {GGUFType::Q3_K, 512, 8, 3, "Q3_K 512x8 S=3"},
        {GGUFType::Q4_K, 512, 8, 3, "Q4_K 512x8 S=3"},     {GGUFType::IQ2_XXS, 512, 8, 3, "IQ2_XXS 512x8 S=3"},
        {GGUFType::IQ2_XXS, 4096, 4, 2, "IQ2_XXS 4096x4 S=2"}, {GGUFType::Q4_K, 8192, 64, 1, "Q4_K 8192x64 S=1"},
    };
    for (auto &c : cases) {
        const bool ok = check_matmul(c.t, c.I, c.O, c.S);
        std::printf("%s matmul %s\n", ok ? "PASS" : "FAIL", c.name);
        fails += !ok;
    }
    // an unsupported type is refused, not mis-computed
    const bool refused = !CudaKernelDispatcher::matmul(GGUFType::Q8_0, nullptr, nullptr, nullptr, 1, 256, 1);
    std::printf("%s unsupported type refused\n", refused ? "PASS" : "FAIL");
    fails += !refused;
    {
        const bool ok = check_triple();
        std::printf("%s per-expert issue / finish triple with the reference's argument lists\n", ok ? "PASS" : "FAIL");
        fails += !ok;
    }
    // a layer call with a null layer aborts instead of falling back
    MoePipelineContext ctx;
    const bool aborted = BatchedDispatchPipeline::run(ctx) == BatchedDispatchResult::Abort;
    std::printf("%s null layer aborts\n", aborted ? "PASS" : "FAIL");
    fails += !aborted;
    return fails;
}
