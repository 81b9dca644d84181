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
    // a layer call with a null layer aborts instead of falling back
    MoePipelineContext ctx;
    const bool aborted = BatchedDispatchPipeline::run(ctx) == BatchedDispatchResult::Abort;
    std::printf("%s null layer aborts\n", aborted ? "PASS" : "FAIL");
    fails += !aborted;
    return fails;
}
