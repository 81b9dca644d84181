// A stand-in for the handful of ggml declarations the bridge header is compiled against in the tests.  It is NOT
// ggml's header: only the member NAMES the bridge reads are kept (type, ne, nb, op, src, data, view_src,
// view_offs); member order, the operator numbering and the parameter encoding are this file's own, which is the
// point -- the bridge must depend on none of them.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <deque>
#include <vector>

enum standin_type { ST_F32 = 0, ST_I32 = 26, ST_Q2_K = 10, ST_Q3_K = 11, ST_Q4_K = 12, ST_IQ2_XXS = 16 };
enum standin_op { SO_NONE = 0, SO_ADD = 3, SO_MUL = 5, SO_CLAMP = 7, SO_CONT = 11, SO_VIEW = 13, SO_MUL_MAT = 17,
                  SO_MUL_MAT_ID = 19, SO_GLU = 23, SO_UNARY = 29, SO_RESHAPE = 31 };
enum standin_variant { SV_NONE = 0, SV_SWIGLU = 1, SV_GEGLU = 2, SV_SILU = 3, SV_GELU = 4 };

struct ggml_tensor {
    void *data = nullptr;
    ggml_tensor *src[4] = {nullptr, nullptr, nullptr, nullptr};
    int op = SO_NONE;
    int variant = SV_NONE;       // which GLU / unary function
    float bounds[2] = {0, 0};    // clamp
    ggml_tensor *view_src = nullptr;
    size_t view_offs = 0;
    size_t nb[4] = {0, 0, 0, 0};
    int64_t ne[4] = {1, 1, 1, 1};
    int type = ST_F32;
};

struct StandinOps {
    enum { MUL_MAT_ID = SO_MUL_MAT_ID, MUL = SO_MUL, ADD = SO_ADD, VIEW = SO_VIEW, CONT = SO_CONT, CLAMP = SO_CLAMP,
           GLU = SO_GLU, UNARY = SO_UNARY, TYPE_F32 = ST_F32, TYPE_I32 = ST_I32 };
    static bool is_swiglu_split(const ggml_tensor *t) { return t->variant == SV_SWIGLU && t->src[1]; }
    static bool is_silu(const ggml_tensor *t) { return t->variant == SV_SILU; }
    static void clamp_bounds(const ggml_tensor *t, float *lo, float *hi) { *lo = t->bounds[0]; *hi = t->bounds[1]; }
};

// a tiny graph builder: tensors live in a deque, nodes are appended in creation order of the operators (a
// post-order walk of the final result gives the same order for the chains built in the tests)
struct StandinGraph {
    std::deque<ggml_tensor> pool;
    std::vector<ggml_tensor *> nodes;

    static size_t elem_bytes(int type, int64_t n) {
        switch (type) {
        case ST_Q2_K: return (size_t)(n / 256) * 84;
        case ST_Q3_K: return (size_t)(n / 256) * 110;
        case ST_Q4_K: return (size_t)(n / 256) * 144;
        case ST_IQ2_XXS: return (size_t)(n / 256) * 66;
        }
        return (size_t)n * 4;
    }
    ggml_tensor *leaf(int type, int64_t n0, int64_t n1 = 1, int64_t n2 = 1, void *data = nullptr) {
        pool.emplace_back();
        ggml_tensor *t = &pool.back();
        t->type = type;
        t->ne[0] = n0; t->ne[1] = n1; t->ne[2] = n2; t->ne[3] = 1;
        t->nb[0] = type == ST_F32 || type == ST_I32 ? 4 : elem_bytes(type, 256);
        t->nb[1] = elem_bytes(type, n0);
        t->nb[2] = t->nb[1] * n1;
        t->nb[3] = t->nb[2] * n2;
        t->data = data;
        return t;
    }
    ggml_tensor *node(int op, ggml_tensor *like, ggml_tensor *a, ggml_tensor *b = nullptr, ggml_tensor *c = nullptr) {
        ggml_tensor *t = leaf(ST_F32, like->ne[0], like->ne[1], like->ne[2]);
        t->op = op;
        t->src[0] = a; t->src[1] = b; t->src[2] = c;
        nodes.push_back(t);
        return t;
    }
    ggml_tensor *mul_mat_id(ggml_tensor *w, ggml_tensor *x, ggml_tensor *ids) {
        ggml_tensor shape;
        shape.ne[0] = w->ne[1]; shape.ne[1] = ids->ne[0]; shape.ne[2] = ids->ne[1];
        return node(SO_MUL_MAT_ID, &shape, w, x, ids);
    }
    ggml_tensor *swiglu_split(ggml_tensor *gate, ggml_tensor *up) {
        ggml_tensor *t = node(SO_GLU, gate, gate, up);
        t->variant = SV_SWIGLU;
        return t;
    }
    ggml_tensor *silu(ggml_tensor *a) {
        ggml_tensor *t = node(SO_UNARY, a, a);
        t->variant = SV_SILU;
        return t;
    }
    ggml_tensor *clamp(ggml_tensor *a, float lo, float hi) {
        ggml_tensor *t = node(SO_CLAMP, a, a);
        t->bounds[0] = lo; t->bounds[1] = hi;
        return t;
    }
    ggml_tensor *mul(ggml_tensor *a, ggml_tensor *b) { return node(SO_MUL, a, a, b); }
    ggml_tensor *add(ggml_tensor *a, ggml_tensor *b) { return node(SO_ADD, a, a, b); }
    ggml_tensor *cont(ggml_tensor *a) { return node(SO_CONT, a, a); }
    ggml_tensor *view_2d(ggml_tensor *a, int64_t n0, int64_t n1, size_t nb1, size_t offs) {
        ggml_tensor shape;
        shape.ne[0] = n0; shape.ne[1] = n1;
        ggml_tensor *t = node(SO_VIEW, &shape, a);
        t->view_src = a;
        t->view_offs = offs;
        t->nb[1] = nb1;
        t->nb[2] = t->nb[3] = nb1 * n1;
        t->data = a->data ? static_cast<char *>(a->data) + offs : nullptr;
        return t;
    }
};
