// zmoe_ggml_bridge.hpp -- the glue between a ggml compute graph and libzmoe_b200.so.  Header only; compiled by the
// host against ITS ggml.h (the library itself never sees a ggml type).
//
// Three parts, each replacing a piece of the reference:
//   1. f32_quant_hook<Tensor>: a trampoline with the signature ggml-cuda calls for MUL_MAT / MUL_MAT_ID nodes on
//      quantised weights (reference patches/ggml/0010-native-f32-quant-graph-hook.patch:12-16), forwarding to
//      zmoe_f32_quant_hook.  ZMOE_GGML_DEFINE_INSTALL(ggml_tensor) defines the function that registers it, with the
//      weak-symbol test of reference kernels/quant/kquant_matmul.cu:757-761.
//   2. match_expert_chain<Ops>: recognises, in graph order, the routed-expert sub-graph the reference builds
//      (models/graph/moe_routed_ggml.hpp:156-215): two MUL_MAT_ID on the same input and ids, SwiGLU (split GLU, or
//      the clamp / silu / mul form), optional clamp, MUL_MAT_ID down, MUL by the route weights, and the
//      view / add reduction over the top-k axis.
//   3. FusedExperts: runs a recognised chain as ONE call of the layer entry (zmoe_set_routes_strided +
//      zmoe_expert_ffn), with layers cached per weight triple.
//
// The tensor type is a template parameter.  It must have the members every ggml graph consumer reads:
//   type, ne[4], nb[4], op, src[], data, view_src, view_offs.
// Everything whose encoding is private to ggml (operator numbers, the GLU / unary variant, clamp bounds) comes in
// through the Ops policy, which the host writes with ggml's own accessors, e.g.
//   struct GgmlOps {
//     enum { MUL_MAT_ID = GGML_OP_MUL_MAT_ID, MUL = GGML_OP_MUL, ADD = GGML_OP_ADD, VIEW = GGML_OP_VIEW,
//            CONT = GGML_OP_CONT, CLAMP = GGML_OP_CLAMP, GLU = GGML_OP_GLU, UNARY = GGML_OP_UNARY,
//            TYPE_F32 = GGML_TYPE_F32, TYPE_I32 = GGML_TYPE_I32 };
//     static bool is_swiglu_split(const ggml_tensor *t) { return ggml_get_glu_op(t) == GGML_GLU_OP_SWIGLU && t->src[1]; }
//     static bool is_silu(const ggml_tensor *t) { return ggml_get_unary_op(t) == GGML_UNARY_OP_SILU; }
//     static void clamp_bounds(const ggml_tensor *t, float *lo, float *hi) {
//       *lo = ggml_get_op_params_f32(t, 0); *hi = ggml_get_op_params_f32(t, 1); }
//   };
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <vector>

#include "../../include/zmoe_b200.h"

namespace zmoe_ggml {

template <class Tensor> inline zmoe_tensor view_of(const Tensor *t) {
    zmoe_tensor v;
    v.type = (int)t->type;
    for (int d = 0; d < 4; ++d) { v.ne[d] = (int64_t)t->ne[d]; v.nb[d] = (size_t)t->nb[d]; }
    v.data = t->data;
    return v;
}

// the hook ggml-cuda calls: execute == false is a support query without side effects
template <class Tensor>
inline bool f32_quant_hook(const Tensor *w, const Tensor *x, const Tensor *ids, Tensor *y, void *stream, bool execute) {
    if (!w || !x || !y) return false;
    const zmoe_tensor vw = view_of(w), vx = view_of(x);
    zmoe_tensor vi, vy = view_of(y);
    if (ids) vi = view_of(ids);
    return zmoe_f32_quant_hook(&vw, &vx, ids ? &vi : nullptr, &vy, stream, execute);
}

// ---------------------------------------------------------------------------------------------------------------
// chain recognition
// ---------------------------------------------------------------------------------------------------------------
template <class Tensor> struct ExpertChain {
    Tensor *w_gate = nullptr, *w_up = nullptr, *w_down = nullptr;
    Tensor *x = nullptr;        // [D, 1, T] f32
    Tensor *ids = nullptr;      // [K, T] i32, rows nb[1] apart
    Tensor *weights = nullptr;  // [1, K, T] f32
    Tensor *out = nullptr;      // [D, T] f32: the last node of the chain
    int first = -1, last = -1;  // node range [first, last] the chain covers
    int topk = 0;
    int64_t n_tokens = 0;
    float clamp = 0.0f;
    bool clamp_fused = false;
};

namespace detail {
template <class Tensor> inline bool same_shape(const Tensor *a, const Tensor *b) {
    for (int d = 0; d < 4; ++d)
        if (a->ne[d] != b->ne[d]) return false;
    return true;
}
}  // namespace detail

// Tries to match the chain whose first node is nodes[i].  On success fills *c and returns true; the caller then
// skips to c->last + 1.  Nothing is matched unless every intermediate has exactly the shape and consumers the
// builder gives it inside [first, last]; a graph that reads an intermediate elsewhere must not be fused, which
// the caller checks with `used_outside` (see below).
template <class Ops, class Tensor>
inline bool match_expert_chain(Tensor *const *nodes, int n_nodes, int i, ExpertChain<Tensor> *c) {
    auto at = [&](int j) -> Tensor * { return j < n_nodes ? nodes[j] : nullptr; };
    auto is = [&](const Tensor *t, int op) { return t && (int)t->op == op; };
    Tensor *a = at(i), *b = at(i + 1);
    if (!is(a, Ops::MUL_MAT_ID) || !is(b, Ops::MUL_MAT_ID)) return false;
    if (a->src[1] != b->src[1] || a->src[2] != b->src[2] || !detail::same_shape(a, b)) return false;
    if ((int)a->type != Ops::TYPE_F32 || (int)a->src[1]->type != Ops::TYPE_F32 || (int)a->src[2]->type != Ops::TYPE_I32)
        return false;
    ExpertChain<Tensor> r;
    r.first = i;
    r.x = a->src[1];
    r.ids = a->src[2];
    int j = i + 2;
    Tensor *gate = nullptr, *up = nullptr, *act = nullptr;
    Tensor *n = at(j);
    if (is(n, Ops::GLU) && Ops::is_swiglu_split(n)) {
        // act = silu(src0) * src1
        if (!((n->src[0] == a && n->src[1] == b) || (n->src[0] == b && n->src[1] == a))) return false;
        gate = n->src[0];
        up = n->src[1];
        act = n;
        ++j;
        n = at(j);
        if (is(n, Ops::CLAMP) && n->src[0] == act) {
            float lo, hi;
            Ops::clamp_bounds(n, &lo, &hi);
            if (!(hi > 0.0f) || lo != -hi) return false;
            r.clamp = hi;
            act = n;
            ++j;
        }
    } else if (is(n, Ops::CLAMP)) {
        // clamp(up, -c, c), clamp(gate, -inf, c), silu, mul -- the two clamps in either order
        Tensor *c0 = n, *c1 = at(j + 1), *s = at(j + 2), *m = at(j + 3);
        if (!is(c1, Ops::CLAMP) || !is(s, Ops::UNARY) || !Ops::is_silu(s) || !is(m, Ops::MUL)) return false;
        Tensor *gate_c = s->src[0];
        if (gate_c != c0 && gate_c != c1) return false;
        Tensor *up_c = gate_c == c0 ? c1 : c0;
        if (!((m->src[0] == s && m->src[1] == up_c) || (m->src[1] == s && m->src[0] == up_c))) return false;
        gate = gate_c->src[0];
        up = up_c->src[0];
        if (!((gate == a && up == b) || (gate == b && up == a))) return false;
        float glo, ghi, ulo, uhi;
        Ops::clamp_bounds(gate_c, &glo, &ghi);
        Ops::clamp_bounds(up_c, &ulo, &uhi);
        if (!(ghi > 0.0f) || ghi != uhi || ulo != -uhi || !(std::isinf(glo) && glo < 0)) return false;
        r.clamp = ghi;
        r.clamp_fused = true;
        act = m;
        j += 4;
    } else {
        return false;
    }
    r.w_gate = gate->src[0];
    r.w_up = up->src[0];
    Tensor *down = at(j);
    if (!is(down, Ops::MUL_MAT_ID) || down->src[1] != act || down->src[2] != r.ids) return false;
    r.w_down = down->src[0];
    ++j;
    Tensor *weighted = at(j);
    if (!is(weighted, Ops::MUL)) return false;
    if (weighted->src[0] == down) r.weights = weighted->src[1];
    else if (weighted->src[1] == down) r.weights = weighted->src[0];
    else return false;
    ++j;
    const int64_t D = down->ne[0], K = down->ne[1], T = down->ne[2];
    if (K < 1 || K > 64 || r.ids->ne[0] != K || r.ids->ne[1] != T) return false;
    if (r.weights->ne[0] != 1 || r.weights->ne[1] != K || r.weights->ne[2] != T || (int)r.weights->type != Ops::TYPE_F32)
        return false;
    if (!detail::same_shape(weighted, down)) return false;
    // the reduction over k: K views of `weighted`, slice k at offset k * nb[1], folded left to right by K - 1 adds
    // (K == 1: the one view made contiguous)
    auto slice_of = [&](const Tensor *t) -> int64_t {   // which k a node is the view of, -1 when it is none
        if (!is(t, Ops::VIEW) || (t->view_src != weighted && t->src[0] != weighted)) return -1;
        if (t->ne[0] != D || t->ne[1] != T || t->ne[2] != 1 || t->nb[1] != weighted->nb[2]) return -1;
        if (t->view_offs % weighted->nb[1]) return -1;
        const uint64_t k = t->view_offs / weighted->nb[1];
        return k < (uint64_t)K ? (int64_t)k : -1;
    };
    uint64_t seen = 0;
    Tensor *sum = nullptr;
    int adds = 0;
    for (;; ++j) {
        Tensor *t = at(j);
        if (is(t, Ops::VIEW)) {
            const int64_t k = slice_of(t);
            if (k < 0 || (seen >> k & 1)) return false;
            seen |= 1ull << k;
            if (k == 0) sum = t;
            continue;
        }
        if (!sum) return false;
        if (K == 1) {
            if (!is(t, Ops::CONT) || t->src[0] != sum) return false;
            sum = t;
            break;
        }
        // the running sum on the left, the next slice (in k order) on the right
        if (!is(t, Ops::ADD) || t->src[0] != sum || slice_of(t->src[1]) != adds + 1 || !(seen >> (adds + 1) & 1)) return false;
        sum = t;
        if (++adds == K - 1) break;
    }
    if (seen != (K == 64 ? ~0ull : (1ull << K) - 1) || !sum) return false;
    r.out = sum;
    r.last = j;
    r.topk = (int)K;
    r.n_tokens = T;
    *c = r;
    return true;
}

// true when a node outside [c.first, c.last] reads one of the chain's intermediates (everything in the range but
// the last node): such a graph needs the intermediates in memory and is left to the per-node path
template <class Tensor> inline bool used_outside(Tensor *const *nodes, int n_nodes, const ExpertChain<Tensor> &c, int max_src) {
    for (int j = 0; j < n_nodes; ++j) {
        if (j >= c.first && j <= c.last) continue;
        for (int s = 0; s < max_src; ++s) {
            const Tensor *src = nodes[j]->src[s];
            if (!src) continue;
            for (int k = c.first; k < c.last; ++k)
                if (src == nodes[k] || nodes[j]->view_src == nodes[k]) return true;
        }
    }
    return false;
}

// ---------------------------------------------------------------------------------------------------------------
// running a chain through the layer entry
// ---------------------------------------------------------------------------------------------------------------
template <class Tensor> class FusedExperts {
public:
    FusedExperts(int max_tokens, int max_d_model, int max_d_ff, int max_experts, int max_topk) {
        status_ = zmoe_ctx_create(max_tokens, max_d_model, max_d_ff, max_experts, max_topk, &ctx_);
    }
    ~FusedExperts() {
        for (Entry &e : layers_) zmoe_layer_destroy(e.layer);
        if (ctx_) zmoe_ctx_destroy(ctx_);
    }
    FusedExperts(const FusedExperts &) = delete;
    FusedExperts &operator=(const FusedExperts &) = delete;

    int status() const { return status_; }
    uint64_t launches() const { return launches_; }

    // side-effect-free: can `run` take this chain?
    bool supports(const ExpertChain<Tensor> &c) const {
        if (status_ != ZMOE_OK || !c.out) return false;
        const Tensor *g = c.w_gate, *u = c.w_up, *d = c.w_down;
        const int64_t D = g->ne[0], F = g->ne[1], E = g->ne[2];
        if (u->ne[0] != D || u->ne[1] != F || u->ne[2] != E || d->ne[0] != F || d->ne[1] != D || d->ne[2] != E) return false;
        if (D % 256 || F % 256) return false;
        if (c.x->ne[0] != D || c.x->ne[1] != 1 || c.x->ne[2] != c.n_tokens) return false;
        if (c.x->nb[0] != 4 || (int64_t)c.x->nb[2] != D * 4) return false;
        if (c.out->ne[0] != D || c.out->ne[1] != c.n_tokens || c.out->nb[0] != 4 || (int64_t)c.out->nb[1] != D * 4) return false;
        if (c.ids->nb[0] != 4 || c.weights->nb[1] != 4) return false;
        // packed rows of a type the library has a layer kernel for
        for (const Tensor *w : {g, u, d}) {
            const size_t bb = block_bytes((int)w->type);
            if (!bb || w->nb[1] != (size_t)(w->ne[0] / 256) * bb || w->nb[2] < w->nb[1] * (size_t)w->ne[1]) return false;
        }
        return true;
    }

    // enqueues the whole chain on `stream`; ZMOE_OK or the failing call's status
    int run(const ExpertChain<Tensor> &c, void *stream) {
        if (!supports(c)) return ZMOE_ERR_SHAPE;
        zmoe_layer *layer = nullptr;
        const int rc = layer_for(c, &layer);
        if (rc) return rc;
        const int T = (int)c.n_tokens;
        int st = zmoe_set_routes_strided(layer, static_cast<const float *>(c.x->data), static_cast<const int32_t *>(c.ids->data),
                                         c.ids->nb[1], static_cast<const float *>(c.weights->data), c.weights->nb[2], T, stream);
        if (!st) st = zmoe_expert_ffn(layer, static_cast<float *>(c.out->data), T, 0, stream);
        if (!st) ++launches_;
        return st;
    }

private:
    struct Entry {
        const void *g, *u, *d;
        int topk;
        float clamp;
        bool fused;
        zmoe_layer *layer;
    };
    static size_t block_bytes(int type) {
        switch (type) {
        case ZMOE_TYPE_Q2_K: return 84;
        case ZMOE_TYPE_Q3_K: return 110;
        case ZMOE_TYPE_Q4_K: return 144;
        case ZMOE_TYPE_IQ2_XXS: return 66;
        }
        return 0;
    }
    int layer_for(const ExpertChain<Tensor> &c, zmoe_layer **out) {
        for (Entry &e : layers_)
            if (e.g == c.w_gate->data && e.u == c.w_up->data && e.d == c.w_down->data && e.topk == c.topk &&
                e.clamp == c.clamp && e.fused == c.clamp_fused) {
                *out = e.layer;
                return ZMOE_OK;
            }
        zmoe_layer_desc d = {};
        d.d_model = (int)c.w_gate->ne[0];
        d.d_ff = (int)c.w_gate->ne[1];
        d.n_experts = (int)c.w_gate->ne[2];
        d.topk = c.topk;
        const Tensor *ws[3] = {c.w_gate, c.w_up, c.w_down};
        zmoe_weight *dst[3] = {&d.gate, &d.up, &d.down};
        for (int i = 0; i < 3; ++i) {
            dst[i]->data_dev = ws[i]->data;
            dst[i]->expert_stride = ws[i]->nb[2];
            dst[i]->bytes = 0;
            dst[i]->type = (int)ws[i]->type;
        }
        d.swiglu_clamp = c.clamp;
        d.swiglu_clamp_fused = c.clamp_fused ? 1 : 0;
        zmoe_layer *layer = nullptr;
        const int rc = zmoe_layer_create(ctx_, &d, &layer);
        if (rc) return rc;
        layers_.push_back(Entry{c.w_gate->data, c.w_up->data, c.w_down->data, c.topk, c.clamp, c.clamp_fused, layer});
        *out = layer;
        return ZMOE_OK;
    }

    zmoe_ctx *ctx_ = nullptr;
    int status_ = ZMOE_OK;
    uint64_t launches_ = 0;
    std::vector<Entry> layers_;
};

}  // namespace zmoe_ggml

// Defines `bool zmoe_ggml_install_hook()`: registers f32_quant_hook<TENSOR> with a ggml-cuda that carries the hook
// patch; false when the linked ggml-cuda does not export the setter (the weak symbol resolves to null).
#define ZMOE_GGML_DEFINE_INSTALL(TENSOR)                                                                               \
    extern "C" void ggml_cuda_set_f32_quant_matmul_hook(                                                               \
        bool (*)(const TENSOR *, const TENSOR *, const TENSOR *, TENSOR *, void *, bool)) __attribute__((weak));       \
    inline bool zmoe_ggml_install_hook() {                                                                             \
        if (!ggml_cuda_set_f32_quant_matmul_hook) return false;                                                        \
        ggml_cuda_set_f32_quant_matmul_hook(&zmoe_ggml::f32_quant_hook<TENSOR>);                                       \
        return true;                                                                                                   \
    }
