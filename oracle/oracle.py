"""ctypes loader for the CPU oracle (oracle/libzmoe_oracle.so).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg; never by the zeromoe_b200 package itself.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libzmoe_oracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libzmoe_ref.so")

Q2_K, Q3_K, Q4_K, IQ2_XXS = 10, 11, 12, 16
BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, IQ2_XXS: 66}
Q8K_BYTES = 292


def build(force=False):
    """Compile the oracle (and the reference shim when the reference checkout exists)."""
    srcs = [os.path.join(HERE, f) for f in ("zmoe_oracle.c", "zmoe_oracle_fast.c", "zmoe_oracle_dense.c", "zmoe_oracle.h")]
    stale = os.path.exists(LIB_PATH) and any(os.path.getmtime(f) > os.path.getmtime(LIB_PATH) for f in srcs)
    if force or stale or not os.path.exists(LIB_PATH):
        subprocess.check_call(["make", "-C", HERE, "-s", "-B", "libzmoe_oracle.so"])
    # the reference checkout, where there is one: named by ZMOE_REFERENCE_ROOT, else looked for beside
    # this repository (../reference); without it the `ref` target is skipped
    ref_root = os.environ.get("ZMOE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    if os.path.isdir(ref_root) and (force or not os.path.exists(REF_PATH)):
        subprocess.call(["make", "-C", HERE, "-s", "ref", "REF=" + ref_root])


class RouterSpec(C.Structure):
    _fields_ = [("n_experts", C.c_int), ("topk", C.c_int), ("gating", C.c_int),
                ("normalize", C.c_int), ("weight_scale", C.c_float),
                ("n_groups", C.c_int), ("n_groups_used", C.c_int)]


class Layer(C.Structure):
    _fields_ = [("D", C.c_int), ("F", C.c_int), ("E", C.c_int), ("K", C.c_int),
                ("type_gate", C.c_int), ("type_up", C.c_int), ("type_down", C.c_int),
                ("w_gate", C.c_void_p), ("w_up", C.c_void_p), ("w_down", C.c_void_p),
                ("stride_gate", C.c_size_t), ("stride_up", C.c_size_t), ("stride_down", C.c_size_t),
                ("clamp", C.c_float), ("clamp_fused", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        L.zo_fp16_to_fp32.restype = C.c_float
        L.zo_fp16_to_fp32.argtypes = [C.c_uint16]
        L.zo_block_bytes.restype = C.c_size_t
        L.zo_vec_dot_q8_K.restype = C.c_float
        L.zo_vec_dot_q8_K.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.zo_vec_dot_q8_K_variant.restype = C.c_float
        L.zo_vec_dot_q8_K_variant.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.zo_vec_dot_q8_K_fast.restype = C.c_float
        L.zo_vec_dot_q8_K_fast.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.zo_router_min_margin.restype = C.c_float
        L.zo_moe_ffn.restype = C.c_int
        L.zo_moe_ffn_fast.restype = C.c_int
        L.zo_fast_kind.restype = C.c_int
        L.zo_fast_force.argtypes = [C.c_int]
        L.zo_fast_force.restype = None
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def quantize_q8_K(x):
    """x [..., k] f32 -> uint8 [..., k/256*292]"""
    x = _f32(x)
    k = x.shape[-1]
    assert k % 256 == 0
    rows = x.reshape(-1, k)
    out = np.zeros((rows.shape[0], k // 256 * Q8K_BYTES), dtype=np.uint8)
    for r in range(rows.shape[0]):
        lib().zo_quantize_row_q8_K(_p(rows[r]), _p(out[r]), C.c_int64(k))
    return out.reshape(x.shape[:-1] + (out.shape[1],))


def q8_fields(q8):
    """split Q8_K bytes [..., nb*292] into (d [...,nb] f32, qs [...,nb,256] i8, bsums [...,nb,16] i16)"""
    b = np.ascontiguousarray(q8).reshape(q8.shape[:-1] + (-1, Q8K_BYTES))
    d = b[..., 0:4].copy().view(np.float32)[..., 0]
    qs = b[..., 4:260].copy().view(np.int8)
    bs = b[..., 260:292].copy().view(np.int16)
    return d, qs, bs


def dequantize(qtype, w, k):
    """w: uint8 rows [..., k/256*block_bytes] -> f32 [..., k]"""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    rows = w.reshape(-1, w.shape[-1])
    out = np.zeros((rows.shape[0], k), dtype=np.float32)
    for r in range(rows.shape[0]):
        lib().zo_dequantize_row(C.c_int(qtype), _p(rows[r]), _p(out[r]), C.c_int64(k))
    return out.reshape(w.shape[:-1] + (k,))


def block_isums(qtype, wrow, q8row):
    """per super-block (isum, msum) int32 arrays for one weight row against one Q8_K row"""
    bb = BLOCK_BYTES[qtype]
    nb = wrow.size // bb
    wrow = np.ascontiguousarray(wrow, dtype=np.uint8)
    q8row = np.ascontiguousarray(q8row, dtype=np.uint8)
    isum = np.zeros(nb, dtype=np.int32)
    msum = np.zeros(nb, dtype=np.int32)
    a, b = C.c_int32(), C.c_int32()
    for i in range(nb):
        lib().zo_block_isums(C.c_int(qtype), C.c_void_p(wrow.ctypes.data + i * bb),
                             C.c_void_p(q8row.ctypes.data + i * Q8K_BYTES), C.byref(a), C.byref(b))
        isum[i], msum[i] = a.value, b.value
    return isum, msum


def vec_dot(qtype, wrow, q8row, n, variant="scalar"):
    """variant: "scalar" (ggml order), "fast" (AVX2 twin), or an int for zo_vec_dot_q8_K_variant"""
    wrow = np.ascontiguousarray(wrow, dtype=np.uint8)
    q8row = np.ascontiguousarray(q8row, dtype=np.uint8)
    if isinstance(variant, int):
        return float(lib().zo_vec_dot_q8_K_variant(qtype, n, _p(wrow), _p(q8row), variant))
    fn = {"scalar": lib().zo_vec_dot_q8_K, "fast": lib().zo_vec_dot_q8_K_fast}[variant]
    return float(fn(qtype, n, _p(wrow), _p(q8row)))


def matmul(qtype, x, w, S, I, O):
    x = _f32(x)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    y = np.zeros((S, O), dtype=np.float32)
    lib().zo_matmul(C.c_int(qtype), _p(y), _p(x), _p(w), C.c_int(S), C.c_int(I), C.c_int(O))
    return y


def mul_mat_id(qtype, x, w, expert_stride, ids, T, K, E, I, O, x_per_route):
    x = _f32(x)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    y = np.zeros((T, K, O), dtype=np.float32)
    lib().zo_mul_mat_id(C.c_int(qtype), _p(y), _p(x), _p(w), C.c_size_t(expert_stride), _p(ids),
                        C.c_int(T), C.c_int(K), C.c_int(E), C.c_int(I), C.c_int(O), C.c_int(x_per_route))
    return y


Q8_0 = 8
Q8_0_BYTES = 34


def quantize_q8_0(x):
    """x [..., k] f32 -> uint8 [..., k/32*34] (ggml Q8_0 blocks)"""
    x = _f32(x)
    k = x.shape[-1]
    rows = x.reshape(-1, k)
    out = np.zeros((rows.shape[0], k // 32 * Q8_0_BYTES), dtype=np.uint8)
    for r in range(rows.shape[0]):
        lib().zo_quantize_row_q8_0(_p(rows[r]), _p(out[r]), C.c_int64(k))
    return out.reshape(x.shape[:-1] + (out.shape[1],))


def dequantize_q8_0(w, k):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    rows = w.reshape(-1, w.shape[-1])
    out = np.zeros((rows.shape[0], k), dtype=np.float32)
    for r in range(rows.shape[0]):
        lib().zo_dequantize_row_q8_0(_p(rows[r]), _p(out[r]), C.c_int64(k))
    return out.reshape(w.shape[:-1] + (k,))


def matmul_q8_0(x, w, S, I, O):
    """y[S, O] = x[S, I] . W^T with W packed rows of Q8_0 blocks, activations quantised to Q8_0"""
    x = _f32(x)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    y = np.zeros((S, O), dtype=np.float32)
    lib().zo_matmul_q8_0(_p(y), _p(x), _p(w), C.c_int(S), C.c_int(I), C.c_int(O))
    return y


def swiglu(gate, up, clamp=0.0, fused=0):
    gate, up = _f32(gate), _f32(up)
    out = np.zeros_like(gate)
    lib().zo_swiglu(_p(out), _p(gate), _p(up), C.c_int(gate.size), C.c_float(clamp), C.c_int(fused))
    return out


def router_logits(x, wr):
    x, wr = _f32(x), _f32(wr)
    T, D = x.shape
    E = wr.shape[0]
    out = np.zeros((T, E), dtype=np.float32)
    lib().zo_router_logits(_p(out), _p(x), _p(wr), C.c_int(T), C.c_int(D), C.c_int(E))
    return out


def router_select(logits, topk, gating=0, normalize=1, weight_scale=0.0, bias=None,
                  n_groups=0, n_groups_used=0):
    """returns (probs [T,E], ids [T,K], weights [T,K], margin)"""
    probs = _f32(logits).copy()
    T, E = probs.shape
    spec = RouterSpec(E, topk, gating, normalize, weight_scale, n_groups, n_groups_used)
    ids = np.zeros((T, topk), dtype=np.int32)
    w = np.zeros((T, topk), dtype=np.float32)
    b = None if bias is None else _f32(bias)
    lib().zo_router_select(C.byref(spec), _p(probs), None if b is None else _p(b), _p(ids), _p(w), C.c_int(T))
    margin = float(lib().zo_router_min_margin(C.byref(spec), _p(probs), None if b is None else _p(b), C.c_int(T)))
    return probs, ids, w, margin


def group_by_expert(ids, E):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    T, K = ids.shape
    offs = np.zeros(E + 1, dtype=np.int32)
    slot = np.zeros(max(T * K, 1), dtype=np.int32)
    lib().zo_group_by_expert(_p(ids), C.c_int(T), C.c_int(K), C.c_int(E), _p(offs), _p(slot))
    return offs, slot[:offs[E]]


def combine(y, weights):
    y, weights = _f32(y), _f32(weights)
    T, K, D = y.shape
    out = np.zeros((T, D), dtype=np.float32)
    lib().zo_combine(_p(out), _p(y), _p(weights), C.c_int(T), C.c_int(K), C.c_int(D))
    return out


def make_layer(D, F, E, K, types, w_gate, w_up, w_down, strides=None, clamp=0.0, fused=0):
    """keeps references to the arrays on the returned struct"""
    bb = BLOCK_BYTES
    if strides is None:
        strides = (F * (D // 256) * bb[types[0]], F * (D // 256) * bb[types[1]], D * (F // 256) * bb[types[2]])
    L = Layer(D, F, E, K, types[0], types[1], types[2], _p(w_gate), _p(w_up), _p(w_down),
              strides[0], strides[1], strides[2], clamp, fused)
    L._keep = (w_gate, w_up, w_down)
    return L


FAST_KINDS = {0: "scalar", 1: "AVX2", 2: "AVX-512 VNNI"}


def fast_kind():
    """the instruction set the timed CPU baseline (vec_dot "fast", moe_ffn(fast=True)) runs its dots on"""
    return FAST_KINDS[lib().zo_fast_kind()]


def fast_force(kind):
    """tests: cap the baseline's instruction set (0 scalar, 1 AVX2, 2 AVX-512 VNNI; -1 the best the CPU has)"""
    lib().zo_fast_force(kind)


def moe_ffn(layer, x, ids, weights, want_act=False, fast=False, threads=0):
    x, weights = _f32(x), _f32(weights)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    T = x.shape[0]
    out = np.zeros((T, layer.D), dtype=np.float32)
    if fast:
        used = lib().zo_moe_ffn_fast(C.byref(layer), _p(x), _p(ids), _p(weights), C.c_int(T), _p(out), C.c_int(threads))
        return out, used
    act = np.zeros((T, layer.K, layer.F), dtype=np.float32) if want_act else None
    rc = lib().zo_moe_ffn(C.byref(layer), _p(x), _p(ids), _p(weights), C.c_int(T), _p(out),
                          None if act is None else _p(act))
    assert rc == 0
    return (out, act) if want_act else out
