// Tests of the ggml bridge header against a stand-in for ggml's declarations.
//   --match : chain recognition only (no device): the chains the reference's graph builder emits
//             (models/graph/moe_routed_ggml.hpp:156-215) are found; near misses are refused.
//   (none)  : the same plus the device part: a recognised chain runs through FusedExperts and agrees with the
//             CPU oracle; the per-node hook trampoline computes one MUL_MAT_ID.
// Prints PASS / FAIL lines.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../../oracle/zmoe_oracle.h"
#include "../../zeromoe_b200/host/zmoe_ggml_bridge.hpp"
#include "ggml_standin.h"

ZMOE_GGML_DEFINE_INSTALL(ggml_tensor)

using Chain = zmoe_ggml::ExpertChain<ggml_tensor>;

struct Built {
    StandinGraph g;
    ggml_tensor *wg, *wu, *wd, *x, *ids, *weights, *out;
    int first;
};

// the graph the reference's builder makes: [some unrelated nodes], up, gate, activation, down, weighted, reduction
static void build(Built &b, int D, int F, int E, int K, int T, float clamp, bool fused, int type = ST_Q2_K) {
    StandinGraph &g = b.g;
    b.wg = g.leaf(type, D, F, E);
    b.wu = g.leaf(type, D, F, E);
    b.wd = g.leaf(type == ST_Q2_K ? ST_Q3_K : type, F, D, E);
    b.x = g.leaf(ST_F32, D, 1, T);
    // ids: the first K columns of an [E, T] argsort result
    ggml_tensor *sorted = g.leaf(ST_I32, E, T);
    b.ids = g.leaf(ST_I32, K, T);
    b.ids->nb[1] = sorted->nb[1];
    b.ids->view_src = sorted;
    b.weights = g.leaf(ST_F32, 1, K, T);
    g.add(b.x, b.x);   // something before the chain
    b.first = (int)g.nodes.size();
    ggml_tensor *up = g.mul_mat_id(b.wu, b.x, b.ids);
    ggml_tensor *gate = g.mul_mat_id(b.wg, b.x, b.ids);
    ggml_tensor *act;
    if (clamp > 0 && fused) {
        ggml_tensor *up_c = g.clamp(up, -clamp, clamp);
        ggml_tensor *gate_c = g.clamp(gate, -INFINITY, clamp);
        act = g.mul(g.silu(gate_c), up_c);
    } else {
        act = g.swiglu_split(gate, up);
        if (clamp > 0) act = g.clamp(act, -clamp, clamp);
    }
    ggml_tensor *down = g.mul_mat_id(b.wd, act, b.ids);
    ggml_tensor *weighted = g.mul(down, b.weights);
    ggml_tensor *out = g.view_2d(weighted, D, T, weighted->nb[2], 0);
    if (K <= 1) out = g.cont(out);
    for (int k = 1; k < K; ++k) out = g.add(out, g.view_2d(weighted, D, T, weighted->nb[2], (size_t)k * weighted->nb[1]));
    b.out = out;
    g.mul(out, out);   // something after the chain
}

static int fails = 0;
static void report(bool ok, const char *what) {
    std::printf("%s %s\n", ok ? "PASS" : "FAIL", what);
    fails += !ok;
}

static bool matches(Built &b, Chain *c) {
    return zmoe_ggml::match_expert_chain<StandinOps>(b.g.nodes.data(), (int)b.g.nodes.size(), b.first, c);
}

static void test_matching() {
    for (int K : {1, 2, 4, 8}) {
        for (int variant = 0; variant < 3; ++variant) {
            Built b;
            const float clamp = variant == 0 ? 0.0f : 7.0f;
            build(b, 512, 256, 8, K, 3, clamp, variant == 2);
            Chain c;
            bool ok = matches(b, &c);
            ok = ok && c.w_gate == b.wg && c.w_up == b.wu && c.w_down == b.wd && c.x == b.x && c.ids == b.ids &&
                 c.weights == b.weights && c.out == b.out && c.topk == K && c.n_tokens == 3 && c.first == b.first &&
                 b.g.nodes[c.last] == b.out && c.clamp == clamp && c.clamp_fused == (variant == 2);
            ok = ok && !zmoe_ggml::used_outside(b.g.nodes.data(), (int)b.g.nodes.size(), c, 4);
            // no other start index matches
            Chain d;
            for (int i = 0; i < (int)b.g.nodes.size(); ++i)
                if (i != b.first && zmoe_ggml::match_expert_chain<StandinOps>(b.g.nodes.data(), (int)b.g.nodes.size(), i, &d)) ok = false;
            char name[96];
            std::snprintf(name, sizeof(name), "chain found, topk %d, %s", K, variant == 0 ? "no clamp" : variant == 1 ? "clamped product" : "clamped gate/up");
            report(ok, name);
        }
    }
    Chain c;
    {   // gate and up on different ids
        Built b; build(b, 512, 256, 8, 4, 3, 0, false);
        b.g.nodes[b.first + 1]->src[2] = b.g.leaf(ST_I32, 4, 3);
        report(!matches(b, &c), "refused: gate and up routed by different ids");
    }
    {   // a GLU that is not SwiGLU
        Built b; build(b, 512, 256, 8, 4, 3, 0, false);
        b.g.nodes[b.first + 2]->variant = SV_GEGLU;
        report(!matches(b, &c), "refused: another GLU function");
    }
    {   // asymmetric clamp of the product
        Built b; build(b, 512, 256, 8, 4, 3, 7.0f, false);
        b.g.nodes[b.first + 3]->bounds[0] = -3.0f;
        report(!matches(b, &c), "refused: asymmetric clamp");
    }
    {   // one slice summed twice, one never
        Built b; build(b, 512, 256, 8, 4, 3, 0, false);
        for (ggml_tensor *t : b.g.nodes)
            if (t->op == SO_VIEW && t->view_offs == 3 * t->view_src->nb[1]) t->view_offs = 2 * t->view_src->nb[1];
        report(!matches(b, &c), "refused: reduction that does not cover every route once");
    }
    {   // the reduction stops early (graph ends)
        Built b; build(b, 512, 256, 8, 4, 3, 0, false);
        b.g.nodes.resize(b.g.nodes.size() - 3);
        report(!matches(b, &c), "refused: truncated reduction");
    }
    {   // weights of the wrong shape
        Built b; build(b, 512, 256, 8, 4, 3, 0, false);
        b.weights->ne[1] = 2;
        report(!matches(b, &c), "refused: weights not [1, topk, tokens]");
    }
    {   // an intermediate read by a node outside the chain
        Built b; build(b, 512, 256, 8, 2, 3, 0, false);
        bool ok = matches(b, &c);
        b.g.mul(b.g.nodes[b.first + 2], b.g.nodes[b.first + 2]);
        report(ok && zmoe_ggml::used_outside(b.g.nodes.data(), (int)b.g.nodes.size(), c, 4), "intermediate used outside is reported");
    }
    report(!zmoe_ggml_install_hook(), "install reports false without a ggml-cuda that exports the setter");
}

// ---------------------------------------------------------------------------------------------------------------
static std::vector<uint8_t> random_blocks(int type, size_t nblocks, std::mt19937 &rng) {
    const size_t bb = zo_block_bytes(type);
    std::vector<uint8_t> w(nblocks * bb);
    for (auto &b : w) b = (uint8_t)rng();
    auto put = [&](size_t blk, size_t off) { const uint16_t h = 0x1C00 + (rng() % 0x0A00); w[blk * bb + off] = h & 0xff; w[blk * bb + off + 1] = h >> 8; };
    for (size_t i = 0; i < nblocks; ++i) {
        if (type == ZO_TYPE_Q2_K) { put(i, 80); put(i, 82); }
        else if (type == ZO_TYPE_Q3_K) put(i, 108);
        else if (type == ZO_TYPE_Q4_K) { put(i, 0); put(i, 2); }
        else put(i, 0);
    }
    return w;
}

template <class T> static T *to_device(const std::vector<T> &v) {
    T *d = nullptr;
    cudaMalloc(&d, v.size() * sizeof(T));
    cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

static double rel_to_norm(const std::vector<float> &got, const std::vector<float> &ref) {
    double m = 0, n = 0;
    for (size_t i = 0; i < got.size(); ++i) { m = std::fmax(m, std::fabs((double)got[i] - ref[i])); n += (double)ref[i] * ref[i]; }
    return m / (std::sqrt(n) + 1e-30);
}

static void test_device(int K, int T, float clamp, bool fused) {
    const int D = 512, F = 512, E = 8;
    std::mt19937 rng(7 + K + T);
    Built b;
    build(b, D, F, E, K, T, clamp, fused);
    auto wg = random_blocks(ZO_TYPE_Q2_K, (size_t)E * F * (D / 256), rng), wu = random_blocks(ZO_TYPE_Q2_K, (size_t)E * F * (D / 256), rng);
    auto wd = random_blocks(ZO_TYPE_Q3_K, (size_t)E * D * (F / 256), rng);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> x((size_t)T * D), w((size_t)T * K), ref((size_t)T * D), got((size_t)T * D);
    for (auto &v : x) v = nd(rng);
    // ids as the first K columns of a per-token permutation of the experts (rows E apart)
    std::vector<int32_t> sorted((size_t)T * E), ids((size_t)T * K);
    for (int t = 0; t < T; ++t) {
        for (int e = 0; e < E; ++e) sorted[(size_t)t * E + e] = e;
        for (int e = E - 1; e > 0; --e) std::swap(sorted[(size_t)t * E + e], sorted[(size_t)t * E + rng() % (e + 1)]);
        float s = 0;
        for (int k = 0; k < K; ++k) { ids[(size_t)t * K + k] = sorted[(size_t)t * E + k]; w[(size_t)t * K + k] = 0.1f + (rng() % 100) / 100.f; s += w[(size_t)t * K + k]; }
        for (int k = 0; k < K; ++k) w[(size_t)t * K + k] /= s;
    }
    zo_layer L = {D, F, E, K, ZO_TYPE_Q2_K, ZO_TYPE_Q2_K, ZO_TYPE_Q3_K, wg.data(), wu.data(), wd.data(),
                  wg.size() / E, wu.size() / E, wd.size() / E, clamp, fused ? 1 : 0};
    zo_moe_ffn(&L, x.data(), ids.data(), w.data(), T, ref.data(), nullptr);
    b.wg->data = to_device(wg); b.wu->data = to_device(wu); b.wd->data = to_device(wd);
    b.x->data = to_device(x);
    b.ids->data = to_device(sorted);
    b.weights->data = to_device(w);
    float *d_out = nullptr;
    cudaMalloc(&d_out, got.size() * 4);
    b.out->data = d_out;
    Chain c;
    bool ok = matches(b, &c);
    zmoe_ggml::FusedExperts<ggml_tensor> fe(64, D, F, E, 8);
    ok = ok && fe.status() == ZMOE_OK && fe.supports(c);
    int rc = ok ? fe.run(c, nullptr) : -100;
    if (ok && !rc) rc = fe.run(c, nullptr);     // the second call takes the cached layer
    cudaDeviceSynchronize();
    cudaMemcpy(got.data(), d_out, got.size() * 4, cudaMemcpyDeviceToHost);
    const double err = rel_to_norm(got, ref);
    char name[128];
    std::snprintf(name, sizeof(name), "fused chain topk %d tokens %d clamp %g%s: status %d, error/norm %.2e", K, T, clamp, fused ? " (gate/up)" : "", rc, err);
    report(ok && rc == 0 && err < 1e-3 && fe.launches() == 2, name);

    // the per-node trampoline on the gate node: y [F, K, T]
    ggml_tensor *gate = b.g.nodes[b.first + 1];
    std::vector<float> yref((size_t)T * K * F), ygot(yref.size());
    zo_mul_mat_id(ZO_TYPE_Q2_K, yref.data(), x.data(), wg.data(), wg.size() / E, ids.data(), T, K, E, D, F, 0);
    float *d_y = nullptr;
    cudaMalloc(&d_y, ygot.size() * 4);
    gate->data = d_y;
    const bool sup = zmoe_ggml::f32_quant_hook<ggml_tensor>(b.wg, b.x, b.ids, gate, nullptr, false);
    const bool ran = sup && zmoe_ggml::f32_quant_hook<ggml_tensor>(b.wg, b.x, b.ids, gate, nullptr, true);
    cudaDeviceSynchronize();
    cudaMemcpy(ygot.data(), d_y, ygot.size() * 4, cudaMemcpyDeviceToHost);
    std::snprintf(name, sizeof(name), "hook trampoline MUL_MAT_ID topk %d tokens %d: error/norm %.2e", K, T, rel_to_norm(ygot, yref));
    report(ran && rel_to_norm(ygot, yref) < 1e-3, name);
    for (void *p : {b.wg->data, b.wu->data, b.wd->data, b.x->data, b.ids->data, b.weights->data, (void *)d_out, (void *)d_y}) cudaFree(p);
}

int main(int argc, char **argv) {
    test_matching();
    if (!(argc > 1 && !std::strcmp(argv[1], "--match"))) {
        test_device(2, 5, 0.0f, false);
        test_device(4, 1, 7.0f, false);
        test_device(8, 33, 0.5f, true);
        test_device(1, 3, 0.0f, false);
    }
    std::printf("%s\n", fails ? "SOME FAILED" : "ALL PASSED");
    return fails ? 1 : 0;
}
