"""CPU checks of the C ABI: the library loads, exports every symbol the public
header declares, and validates arguments before touching a device."""
import ctypes as C
import os
import re

from zeromoe_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "zmoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:void|int|bool|uint64_t)\s+(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    L = lib.load()
    decl = declared_symbols()
    assert len(decl) >= 30
    for name in decl:
        assert hasattr(L, name), name
    assert sorted(lib.EXPORTS) == decl


def test_argument_validation_needs_no_device():
    L = lib.load()
    h = C.c_void_p()
    assert L.zmoe_ctx_create(0, 4096, 1536, 128, 8, C.byref(h)) == -1
    assert L.zmoe_ctx_create(16, 4000, 1536, 128, 8, C.byref(h)) == -3       # not a multiple of 256
    assert L.zmoe_layer_create(None, None, C.byref(h)) == -1
    assert L.zmoe_route(None, None, 1, None) == -1
    assert L.zmoe_expert_ffn(None, None, 1, 0, None) == -1
    assert L.zmoe_set_routes(None, None, None, None, 1, None) == -1
    assert L.zmoe_set_routes_window(None, None, None, None, 1, 0, None) == -1
    assert L.zmoe_ctx_set_path(None, 0) == -1
    assert L.zmoe_quantize_q8_K(None, None, 1, 256, lib.Q4_K, None) == -1
    assert L.zmoe_block_isums(99, None, None, None, None, 1, 256, None) == -1
    assert L.zmoe_reserve(4, 100) == -1
    assert L.zmoe_ctx_bad_counts(None, None, 0) == -1
    assert L.zmoe_gemm_min_pairs_per_expert() == 24
    assert not L.zeromoe_install_f32_quant_graph_hook()
    assert not L.zmoe_f32_quant_hook(None, None, None, None, None, False)


def test_hook_support_query_is_pure():
    """execute=false must validate shapes without any device work"""
    L = lib.load()

    def tensor(t, ne, nb):
        T = lib.Tensor()
        T.type = t
        T.ne[:] = ne
        T.nb[:] = nb
        T.data = 256          # never dereferenced by a support query
        return T
    I, O, E, K, Tk = 512, 64, 4, 2, 3
    rb = I // 256 * 84
    w = tensor(lib.Q2_K, [I, O, E, 1], [0, rb, rb * O, rb * O * E])
    x = tensor(lib.GGML_F32, [I, 1, Tk, 1], [4, 4 * I, 4 * I, 4 * I * Tk])
    ids = tensor(lib.GGML_I32, [K, Tk, 1, 1], [4, 4 * K, 4 * K * Tk, 4 * K * Tk])
    y = tensor(lib.GGML_F32, [O, K, Tk, 1], [4, 4 * O, 4 * O * K, 4 * O * K * Tk])
    q = lambda *a: L.zmoe_f32_quant_hook(*[C.byref(t) for t in a], None, False)
    assert q(w, x, ids, y)
    w_bad = tensor(lib.Q2_K, [I, O, E, 1], [0, rb + 4, (rb + 4) * O, 0])          # padded rows
    assert not q(w_bad, x, ids, y)
    y_bad = tensor(lib.GGML_F32, [O + 1, K, Tk, 1], [4, 4 * O, 4 * O * K, 0])
    assert not q(w, x, ids, y_bad)
    ids_bad = tensor(lib.GGML_F32, [K, Tk, 1, 1], [4, 4 * K, 0, 0])
    assert not q(w, x, ids_bad, y)
    w8 = tensor(8, [I, O, E, 1], [0, 34 * 16, 0, 0])                               # Q8_0: no kernel
    assert not q(w8, x, ids, y)
