"""Generates tests/golden/reference_vectors.npz: inputs and the outputs of the
REFERENCE's own code for them.

Run in a container where the reference checkout exists (it compiles
oracle/_ref/libzmoe_ref.so from reference sources, see oracle/ref_shim.cpp):

    python tests/golden/make_golden.py

The .npz travels with the repository, so the oracle can be checked against
reference outputs on machines that have no reference checkout.  Contents, all
produced by reference functions on seeded random inputs:
  q2k_* : bench/q2k_dot_bench.cpp dot_stock (ggml's Q2_K x Q8_K AVX2 dot, verbatim copy)
  q4k_* : bench/q3k_q4k_dot_bench.cpp dot_q4k_512 (bit-exact twin of ggml's Q4_K dot)
  iq2_* : bench/kernels/iq2xxs_dot_bench.cpp dot_ref (ggml's IQ2_XXS x Q8_K AVX2 dot)
          and backends/cpu/kernels_cpu.cpp dot_iq2_xxs_avx2_prototype
  deq_* : backends/cpu/kernels_cpu.cpp dequantize_row_{q2_K,q3_K,iq2_xxs}_avx512
  gate_*: core/moe_router.cpp apply_gating_activation
  swiglu_*: core/expert_activation.hpp swiglu_clamp_fused_inplace
The Q8_K blocks fed to the dots are arbitrary int8 blocks with consistent bsums
(the dots do not care how they were produced), so these vectors do not depend
on the activation quantiser.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O          # noqa: E402
from zeromoe_b200 import synth          # noqa: E402


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def random_q8(rng, nb):
    blk = np.zeros((nb, 292), dtype=np.uint8)
    d = rng.uniform(0.005, 0.05, size=nb).astype(np.float32)
    qs = rng.integers(-127, 128, size=(nb, 256)).astype(np.int8)
    bs = qs.reshape(nb, 16, 16).sum(-1).astype(np.int16)
    blk[:, 0:4] = d.view(np.uint8).reshape(nb, 4)
    blk[:, 4:260] = qs.view(np.uint8)
    blk[:, 260:292] = bs.view(np.uint8).reshape(nb, 32)
    return blk.reshape(-1)


def main():
    O.build(force=False)
    R = C.CDLL(O.REF_PATH)
    for n in ("ref_q2k_dot_stock", "ref_q4k_dot_512", "ref_iq2xxs_dot", "ref_iq2xxs_dot_bench"):
        getattr(R, n).restype = C.c_float
        getattr(R, n).argtypes = [C.c_int, C.c_void_p, C.c_void_p]
    rng = synth.rng_for(20261125, 99)
    out = {}
    nb, rows = 8, 48
    k = nb * 256
    q8 = random_q8(rng, nb)
    out["q8"] = q8
    for name, qt, fns in (("q2k", synth.Q2_K, [("stock", R.ref_q2k_dot_stock)]),
                          ("q4k", synth.Q4_K, [("512", R.ref_q4k_dot_512)]),
                          ("iq2", synth.IQ2_XXS, [("bench", R.ref_iq2xxs_dot_bench), ("proto", R.ref_iq2xxs_dot)])):
        w = synth.random_blocks(qt, rows * nb, rng).reshape(rows, -1)
        out[name + "_w"] = w
        for tag, fn in fns:
            out["%s_dot_%s" % (name, tag)] = np.array([fn(k, p(w[r]), p(q8)) for r in range(rows)], dtype=np.float32)
    for name, qt, fn in (("q2k", synth.Q2_K, R.ref_dequant_q2k), ("q3k", synth.Q3_K, R.ref_dequant_q3k),
                         ("iq2", synth.IQ2_XXS, R.ref_dequant_iq2xxs)):
        w = synth.random_blocks(qt, 4 * nb, rng).reshape(4, -1)
        y = np.zeros((4, k), dtype=np.float32)
        for r in range(4):
            fn(p(w[r]), p(y[r]), C.c_int64(k))
        out["deq_%s_w" % name] = w
        out["deq_%s_y" % name] = y
    logits = (rng.standard_normal((3, 128)) * 3).astype(np.float32)
    out["gate_in"] = logits
    for g in (0, 1, 2):
        a = logits.copy()
        for r in range(3):
            R.ref_apply_gating(g, p(a[r]), 128)
        out["gate_out_%d" % g] = a
    g = (rng.standard_normal(512) * 4).astype(np.float32)
    u = rng.standard_normal(512).astype(np.float32)
    out["swiglu_g"], out["swiglu_u"] = g, u
    for tag, lim in (("noclamp", 0.0), ("clamp", 2.5)):
        a = g.copy()
        R.ref_swiglu_fused(p(a), p(u), 512, C.c_float(lim))
        out["swiglu_fused_" + tag] = a
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
