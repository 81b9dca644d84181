"""GPU parity tests: every stage of the CUDA path, called through the C ABI,
against the CPU oracle on the same seeded inputs.

Integer stages (Q8_K bytes, per-super-block int32 sums, expert ids, grouping)
must match bit for bit; f32 outputs within 1e-3 max-abs relative to the norm
of the reference output (helpers.REL_TO_NORM).  Shapes and recipes follow the
reference's own tests: tests/native/tests_basic_cuda.cpp:301-320,367,414
(matmul shapes), tests/test_phase_alias_numerics.cpp:104-107 (exact inputs),
tests/test_qwen_moe_router_ggml.cpp:22-188 (router literals),
tests/test_option_b_compact_ggml.cpp:21-145 (negative ids),
tests/test_dsv41_cache_graph.cpp:60-185 (strided slabs, untouched weights),
tests/native/tests_expert_cache.cpp:772-841 (device accumulate).
"""
import ctypes as C

import numpy as np
import pytest

from helpers import REL_TO_NORM, TYPES, rel_to_norm, routed_inputs, to_dev
from zeromoe_b200 import synth

pytestmark = pytest.mark.gpu


def _sync():
    import torch
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------
# activation quantisation
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("for_type", [synth.Q2_K, synth.Q4_K])     # the two packed-row layouts
def test_q8k_bytes_bit_exact(zlib, oracle, dev, for_type):
    import torch
    rng = synth.rng_for(11, 0)
    rows, I = 7, 2048
    x = synth.activations(rows, I, rng)
    x[1, 256:512] = 0.0                       # an all-zero super-block
    x[2, 0:256] *= 1e-20                      # tiny magnitudes
    x[3, 0:256] *= 1e20                       # huge magnitudes
    x[4, 10] = 9.0
    x[4, 200] = -9.0                          # |max| tie with opposite signs: first wins
    x[5, 256:512] = np.round(x[5, 256:512] * 4) / 4 + 0.5   # many exact .5 products
    x[6, :] = synth.exact_activations(1, I, rng)[0]
    xd = to_dev(x, dev)
    out = torch.zeros(rows * (I // 256) * 292, dtype=torch.uint8, device=dev)
    zlib.check(zlib.load().zmoe_quantize_q8_K(zlib.ptr(xd), zlib.ptr(out), rows, I, for_type, None),
               "zmoe_quantize_q8_K")
    _sync()
    got = out.cpu().numpy().reshape(rows, -1)
    ref = oracle.quantize_q8_K(x)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("qtype", TYPES)
def test_block_int32_sums_bit_exact(zlib, oracle, dev, qtype):
    import torch
    rng = synth.rng_for(12, qtype)
    rows, I = 24, 1536
    nb = I // 256
    w = synth.random_blocks(qtype, rows * nb, rng).reshape(rows, -1)
    x = synth.activations(rows, I, rng) * rng.uniform(0.1, 4.0, size=(rows, 1)).astype(np.float32)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    isum = torch.zeros((rows, nb), dtype=torch.int32, device=dev)
    msum = torch.zeros((rows, nb), dtype=torch.int32, device=dev)
    zlib.check(zlib.load().zmoe_block_isums(qtype, zlib.ptr(wd), zlib.ptr(xd), zlib.ptr(isum), zlib.ptr(msum),
                                            rows, I, None), "zmoe_block_isums")
    _sync()
    q8 = oracle.quantize_q8_K(x)
    for r in range(rows):
        ri, rm = oracle.block_isums(qtype, w[r], q8[r])
        assert np.array_equal(isum[r].cpu().numpy(), ri), (qtype, r)
        assert np.array_equal(msum[r].cpu().numpy(), rm), (qtype, r)


@pytest.mark.parametrize("qtype", [synth.Q2_K, synth.Q3_K, synth.Q4_K])
@pytest.mark.parametrize("pairs", [2, 3, 4])
@pytest.mark.parametrize("I", [1536, 4096])
def test_tensor_core_path_int32_sums_bit_exact(zlib, oracle, dev, qtype, pairs, I):
    """the s32 sums mma.sync forms for 16 rows x `pairs` activation rows equal the oracle's, block by block"""
    import torch
    rng = synth.rng_for(14, qtype, pairs, I)
    nb = I // 256
    w = synth.random_blocks(qtype, 16 * nb, rng).reshape(16, -1)
    x = synth.activations(pairs, I, rng) * rng.uniform(0.1, 4.0, size=(pairs, 1)).astype(np.float32)
    wd, xd = to_dev(w, dev), to_dev(x, dev)
    sums = torch.zeros((16, 4, nb, 2), dtype=torch.int32, device=dev)
    zlib.check(zlib.load().zmoe_block_isums_pairs(qtype, zlib.ptr(wd), zlib.ptr(xd), zlib.ptr(sums), pairs, I, None),
               "zmoe_block_isums_pairs")
    _sync()
    got = sums.cpu().numpy()
    q8 = oracle.quantize_q8_K(x)
    for r in range(16):
        for p in range(pairs):
            ri, rm = oracle.block_isums(qtype, w[r], q8[p])
            assert np.array_equal(got[r, p, :, 0], ri), (qtype, r, p)
            assert np.array_equal(got[r, p, :, 1], rm), (qtype, r, p)
    assert zlib.load().zmoe_block_isums_pairs(synth.IQ2_XXS, zlib.ptr(wd), zlib.ptr(xd), zlib.ptr(sums), pairs, I, None) == -2


# ---------------------------------------------------------------------------
# launch_*_matmul (reference kernel-launch ABI)
# ---------------------------------------------------------------------------
MATMUL_SHAPES = [(512, 8, 3), (4096, 4, 2), (2048, 40, 1), (1536, 64, 5), (768, 12, 9), (7168, 16, 2), (256, 3, 1)]


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("shape", MATMUL_SHAPES)
def test_dense_matmul_vs_oracle(zlib, oracle, dev, qtype, shape):
    I, O, S = shape
    rng = synth.rng_for(13, qtype, I, O)
    w = synth.expert_weights(qtype, 1, O, I, rng)[0]
    x = synth.activations(S, I, rng)
    y = zlib.dense_matmul(qtype, to_dev(x, dev), to_dev(w, dev), O)
    _sync()
    ref = oracle.matmul(qtype, x, w, S, I, O)
    assert rel_to_norm(y.cpu().numpy(), ref) < REL_TO_NORM


@pytest.mark.parametrize("qtype", TYPES)
def test_dense_matmul_exact_inputs_vs_f64(zlib, oracle, dev, qtype):
    """with activations that Q8_K represents exactly the result must agree with a
    float64 dequantise-and-dot to 1e-4 relative L2 (the reference's EXACT_INPUTS check)"""
    I, O, S = 4096, 48, 2
    rng = synth.rng_for(14, qtype)
    w = synth.expert_weights(qtype, 1, O, I, rng)[0]
    x = synth.exact_activations(S, I, rng)
    y = zlib.dense_matmul(qtype, to_dev(x, dev), to_dev(w, dev), O).cpu().numpy()
    deq = oracle.dequantize(qtype, w, I).astype(np.float64)
    ref = x.astype(np.float64) @ deq.T
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 1e-4


def test_dense_matmul_rejects_bad_shapes(zlib, dev):
    import torch
    x = torch.zeros((1, 300), device=dev)
    w = torch.zeros(1024, dtype=torch.uint8, device=dev)
    y = torch.zeros((1, 4), device=dev)
    L = zlib.load()
    L.launch_q4_K_matmul(zlib.ptr(y), zlib.ptr(x), zlib.ptr(w), 1, 300, 4)
    assert L.zmoe_last_status() == -3
    L.launch_q4_K_matmul(None, zlib.ptr(x), zlib.ptr(w), 1, 256, 4)
    assert L.zmoe_last_status() == -1


# ---------------------------------------------------------------------------
# element-wise kernels of the reference ABI
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("clamp,fused", [(0.0, 0), (2.5, 0), (2.5, 1), (0.0, 1)])
def test_expert_swiglu(zlib, oracle, dev, clamp, fused):
    import torch
    rng = synth.rng_for(15, int(clamp * 10), fused)
    n = 5000
    g = (rng.standard_normal(n) * 4).astype(np.float32)
    u = (rng.standard_normal(n) * 2).astype(np.float32)
    g[7] = np.nan
    u[9] = np.inf
    gd, ud = to_dev(g, dev), to_dev(u, dev)
    out = torch.zeros(n, device=dev)
    bad = torch.zeros(2, dtype=torch.int32, device=dev)
    zlib.load().launch_expert_swiglu(zlib.ptr(out), zlib.ptr(gd), zlib.ptr(ud), n, clamp, fused, zlib.ptr(bad), None)
    _sync()
    ref = oracle.swiglu(g, u, clamp, fused)
    got = out.cpu().numpy()
    ok = np.isfinite(ref)
    assert np.allclose(got[ok], ref[ok], rtol=2e-6, atol=1e-7)
    assert bad.cpu().tolist() == [1, 1]


def test_scatter_accum(zlib, dev):
    import torch
    rng = np.random.default_rng(777)
    S, D, n = 9, 640, 6
    src = rng.standard_normal((n, D)).astype(np.float32)
    tok = np.array([3, 0, 8, 5, 3, 99], dtype=np.int32)   # repeated token, one out of range
    w = rng.standard_normal(n).astype(np.float32)
    dst = torch.zeros((S, D), device=dev)
    L = zlib.load()
    # rows of one call must target distinct tokens: issue the repeat as a second call
    for sel in ([0, 1, 2, 3, 5], [4]):
        s, t, ww = to_dev(src[sel], dev), to_dev(tok[sel], dev), to_dev(w[sel], dev)
        L.launch_expert_scatter_accum(zlib.ptr(s), zlib.ptr(t), zlib.ptr(ww), zlib.ptr(dst), len(sel), D, S, None)
    _sync()
    ref = np.zeros((S, D), dtype=np.float32)
    for i in range(n):
        if 0 <= tok[i] < S:
            ref[tok[i]] += w[i] * src[i]
    got = dst.cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-6, atol=1e-6)
    assert np.all(got[1] == 0.0)   # an untouched row stays exactly zero


# ---------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------
def test_router_reference_literals(zlib, dev):
    """fixed 3x4 router, two tokens, softmax, top-2, normalise, scale 1.5"""
    import torch
    router = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [.5, .5, .5]], dtype=np.float32)
    hidden = np.array([[0.1, 2.0, 1.0], [3.0, 0.5, -1.0]], dtype=np.float32)
    logits = hidden @ router.T
    ld = to_dev(logits, dev)
    ids = torch.zeros((2, 2), dtype=torch.int32, device=dev)
    w = torch.zeros((2, 2), dtype=torch.float32, device=dev)
    zlib.load().launch_glm5next_router_topk(zlib.ptr(ld), None, zlib.ptr(ids), zlib.ptr(w), 2, 4, 2, 0, 1, 1.5, None)
    _sync()
    ex = np.exp(logits - logits.max(1, keepdims=True))
    probs = ex / ex.sum(1, keepdims=True)
    order = np.argsort(-probs, axis=1)[:, :2]
    sel = np.take_along_axis(probs, order, 1)
    assert np.array_equal(ids.cpu().numpy(), order.astype(np.int32))
    assert np.allclose(w.cpu().numpy(), 1.5 * sel / sel.sum(1, keepdims=True), atol=1e-5)
    assert np.allclose(ld.cpu().numpy(), probs, atol=1e-5)   # logits are overwritten with probabilities


ROUTER_CASES = [
    dict(E=128, K=8, gating=0, normalize=1, scale=0.0, groups=(0, 0), bias=False),
    dict(E=128, K=8, gating=1, normalize=1, scale=2.5, groups=(0, 0), bias=True),
    dict(E=256, K=8, gating=1, normalize=1, scale=2.5, groups=(8, 4), bias=True),
    dict(E=64, K=6, gating=2, normalize=0, scale=1.0, groups=(0, 0), bias=False),
    dict(E=11, K=4, gating=0, normalize=1, scale=0.0, groups=(0, 0), bias=False),
]


@pytest.mark.parametrize("case", ROUTER_CASES)
@pytest.mark.parametrize("T", [1, 16, 37])
def test_layer_router_vs_oracle(zlib, oracle, dev, case, T):
    import torch
    E, K, D, F = case["E"], case["K"], 512, 256
    rng = synth.rng_for(16, E, K, T)
    bias = (rng.standard_normal(E) * 0.05).astype(np.float32) if case["bias"] else None
    wr, x, probs, ids_ref, w_ref = routed_inputs(oracle, 16 + E + T, T, D, E, K, gating=case["gating"],
                                                 normalize=case["normalize"], weight_scale=case["scale"], bias=bias,
                                                 n_groups=case["groups"][0], n_groups_used=case["groups"][1])
    w = synth.expert_weights(synth.Q4_K, E, F, D, rng)
    wdn = synth.expert_weights(synth.Q4_K, E, D, F, rng)
    ctx = zlib.Context(64, D, F, E, K)
    wd, wdd = to_dev(w, dev), to_dev(wdn, dev)
    layer = zlib.Layer(ctx, D, F, E, K, (synth.Q4_K,) * 3, wd, wd, wdd, router_w=to_dev(wr, dev),
                       router_bias=None if bias is None else to_dev(bias, dev), gating=case["gating"],
                       weights_norm=case["normalize"], weights_scale=case["scale"], n_groups=case["groups"][0],
                       n_groups_used=case["groups"][1])
    layer.route(to_dev(x, dev))
    _sync()
    ctx.check()
    ids, wts = ctx.routes(T, K)
    assert np.array_equal(ids, ids_ref)
    assert np.allclose(wts, w_ref, atol=1e-5)
    assert np.allclose(ctx.probs(T, E), probs, atol=1e-5)
    offs, _ = oracle.group_by_expert(ids_ref, E)
    assert np.array_equal(ctx.expert_freq(E), np.diff(offs))


# ---------------------------------------------------------------------------
# the whole layer
# ---------------------------------------------------------------------------
LAYER_CASES = [
    # D, F, E, K, types (gate, up, down), T
    (2048, 768, 128, 8, (synth.Q4_K, synth.Q4_K, synth.Q4_K), 1),       # benchmark configuration 1, decode
    (2048, 768, 128, 8, (synth.Q4_K, synth.Q4_K, synth.Q4_K), 64),      # configuration 1, 64 tokens
    (4096, 1536, 128, 8, (synth.Q2_K, synth.Q2_K, synth.Q3_K), 1),      # configuration 2
    (4096, 1536, 128, 8, (synth.Q2_K, synth.Q2_K, synth.Q3_K), 4),
    (4096, 1536, 128, 8, (synth.Q2_K, synth.Q2_K, synth.Q3_K), 16),
    (4096, 1536, 32, 8, (synth.IQ2_XXS, synth.IQ2_XXS, synth.IQ2_XXS), 5),   # configuration 3's types
    (1024, 512, 16, 4, (synth.Q2_K, synth.Q4_K, synth.Q3_K), 7),        # gate and up of different types
    (512, 256, 8, 8, (synth.Q3_K, synth.Q3_K, synth.Q2_K), 3),          # every expert used by every token
]


@pytest.mark.parametrize("case", LAYER_CASES)
def test_moe_layer_vs_oracle(zlib, oracle, dev, case):
    import torch
    D, F, E, K, types, T = case
    rng = synth.rng_for(17, D, F, E, T)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    wr, x, probs, ids_ref, w_ref = routed_inputs(oracle, 17 + D + T, T, D, E, K)
    ctx = zlib.Context(64, D, F, E, K)
    tg, tu, td = to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev)
    canary = [t.clone() for t in (tg, tu, td)]
    layer = zlib.Layer(ctx, D, F, E, K, types, tg, tu, td, router_w=to_dev(wr, dev))
    out = torch.full((T, D), float("nan"), device=dev)
    layer.forward(to_dev(x, dev), out)
    _sync()
    ctx.check()
    ids, wts = ctx.routes(T, K)
    assert np.array_equal(ids, ids_ref)
    Lr = oracle.make_layer(D, F, E, K, types, wg, wu, wd)
    ref, act_ref = oracle.moe_ffn(Lr, x, ids_ref, w_ref, want_act=True)
    act = ctx.act(T * K, F).reshape(T, K, F)
    assert rel_to_norm(act, act_ref) < REL_TO_NORM
    assert rel_to_norm(out.cpu().numpy(), ref) < REL_TO_NORM
    # weights are borrowed and must stay bit-identical
    for t, c in zip((tg, tu, td), canary):
        assert torch.equal(t, c)
    # the same call again gives the same bytes (fixed reduction order)
    out2 = torch.empty_like(out)
    layer.forward(to_dev(x, dev), out2)
    _sync()
    assert torch.equal(out, out2)


PREFILL_CASES = [
    # D, F, E, K, types, T : shapes where an expert sees tens to hundreds of pairs
    (2048, 768, 16, 4, (synth.Q4_K, synth.Q4_K, synth.Q4_K), 200),       # configuration 1's types, prefill-shaped
    (1024, 512, 8, 2, (synth.IQ2_XXS, synth.IQ2_XXS, synth.IQ2_XXS), 333),  # configuration 3's type, ragged pair blocks
    (1024, 512, 8, 2, (synth.Q2_K, synth.Q2_K, synth.Q3_K), 300),        # configuration 2's types
    (512, 256, 4, 2, (synth.Q4_K, synth.Q4_K, synth.Q4_K), 40),          # fewer pairs than one MMA tile
]


@pytest.mark.parametrize("case", PREFILL_CASES)
def test_prefill_tensor_core_path_vs_oracle(zlib, oracle, dev, case):
    """the tcgen05 grouped GEMM (forced with set_path(2)) against the oracle, and against the
    decode kernels on the same call; the tiled-GEMM router serves T > 64"""
    import torch
    D, F, E, K, types, T = case
    rng = synth.rng_for(23, D, F, E, T)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    wr, x, probs, ids_ref, w_ref = routed_inputs(oracle, 23 + D + T, T, D, E, K)
    ctx = zlib.Context(max(T, 16), D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev),
                       router_w=to_dev(wr, dev))
    xd = to_dev(x, dev)
    outs = {}
    for path in (1, 2):
        ctx.set_path(path)
        out = torch.full((T, D), float("nan"), device=dev)
        layer.forward(xd, out)
        _sync()
        ctx.check()
        outs[path] = out.cpu().numpy()
    ids, wts = ctx.routes(T, K)
    assert np.array_equal(ids, ids_ref)
    assert np.allclose(wts, w_ref, atol=1e-5)
    ref = oracle.moe_ffn(oracle.make_layer(D, F, E, K, types, wg, wu, wd), x, ids_ref, w_ref)
    assert rel_to_norm(outs[1], ref) < REL_TO_NORM
    assert rel_to_norm(outs[2], ref) < REL_TO_NORM          # fp16 operands: ~1e-4 here
    assert np.isfinite(outs[2]).all()
    out2 = torch.empty((T, D), device=dev)
    layer.forward(xd, out2)
    _sync()
    assert np.array_equal(out2.cpu().numpy().view(np.uint32), outs[2].view(np.uint32))   # reproducible


@pytest.mark.parametrize("types", [(synth.Q2_K, synth.Q2_K, synth.Q3_K), (synth.Q3_K, synth.Q3_K, synth.Q2_K)])
def test_experts_holding_one_to_nine_pairs(zlib, oracle, dev, types):
    """Experts with 2+ pairs take the tensor-core consumer path, 4 pairs per item: pin the pair count of
    every expert (1..9, so one-, two- and three-item experts with full and ragged last items), with a
    ragged last row tile in the down projection, and compare with the oracle and with the one-pair-at-a-time path."""
    import torch
    D, F, E, K = 1024, 1536, 9, 3          # the down projection's 1024 rows leave a ragged last 48-row tile
    counts = list(range(1, E + 1))         # expert e holds e + 1 pairs
    T = sum(counts) // K                   # 45 pairs = 15 tokens x 3 routes
    assert T * K == sum(counts)
    rng = synth.rng_for(23, types[0])
    # deal the experts' pairs to tokens so that no token gets one expert twice
    pool = [e for e, n in enumerate(counts) for _ in range(n)]
    ids = None
    for _ in range(1000):
        perm = rng.permutation(len(pool))
        cand = np.array(pool)[perm].reshape(T, K)
        if all(len(set(r)) == K for r in cand):
            ids = cand.astype(np.int32)
            break
    assert ids is not None
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    x = synth.activations(T, D, rng)
    wts = rng.uniform(0.05, 0.6, size=(T, K)).astype(np.float32)
    ctx = zlib.Context(16, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev))
    xd, idd, wtd = to_dev(x, dev), to_dev(ids, dev), to_dev(wts, dev)
    outs = {}
    for path in (0, 3):
        ctx.set_path(path)
        layer.set_routes(xd, idd, wtd)
        out = torch.full((T, D), float("nan"), device=dev)
        layer.expert_ffn(out)
        _sync()
        ctx.check()
        outs[path] = (out.cpu().numpy(), ctx.act(T * K, F).reshape(T, K, F).copy())
    ctx.set_path(0)
    Lr = oracle.make_layer(D, F, E, K, types, wg, wu, wd)
    ref, act_ref = oracle.moe_ffn(Lr, x, ids, wts, want_act=True)
    for path, (got, act) in outs.items():
        assert rel_to_norm(act, act_ref) < REL_TO_NORM, path
        assert rel_to_norm(got, ref) < REL_TO_NORM, path
    # the two paths add the same exact integer sums in a different f32 order
    assert rel_to_norm(outs[0][0], outs[3][0]) < 1e-5


@pytest.mark.parametrize("T", [6, 3])
def test_moe_layer_supplied_routes_with_inactive_ids(zlib, oracle, dev, T):
    """negative ids are inactive routes: they contribute a zero row.  T = 3 runs the small-batch launches
    that quantise act and add up the routes inside the matmul kernels."""
    import torch
    D, F, E, K = 1024, 512, 12, 10
    types = (synth.Q2_K, synth.Q2_K, synth.Q3_K)
    rng = synth.rng_for(18, 0)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    x = synth.activations(T, D, rng)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    ids[0, 3] = -1
    ids[2, :] = -1          # a token with no active route at all
    ids[T - 1, 9] = -1
    wts = rng.uniform(0.05, 0.3, size=(T, K)).astype(np.float32)
    ctx = zlib.Context(8, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev))
    xd = to_dev(x, dev)
    layer.set_routes(xd, to_dev(ids, dev), to_dev(wts, dev))
    out = torch.full((T, D), float("nan"), device=dev)
    layer.expert_ffn(out)
    _sync()
    ctx.check()
    Lr = oracle.make_layer(D, F, E, K, types, wg, wu, wd)
    ref = oracle.moe_ffn(Lr, x, ids, wts)
    got = out.cpu().numpy()
    assert rel_to_norm(got, ref) < REL_TO_NORM
    assert np.all(got[2] == 0.0)
    # accumulate = 1 adds to what is there
    base = torch.ones((T, D), device=dev)
    layer.expert_ffn(base, accumulate=1)
    _sync()
    assert rel_to_norm(base.cpu().numpy(), ref + 1.0) < REL_TO_NORM
    if T <= 4:
        # one pair at a time (path 3) a token's result does not depend on the batch it is in: the same
        # tokens twice in one batch give the same bytes as alone
        ctx.set_path(3)
        layer.set_routes(xd, to_dev(ids, dev), to_dev(wts, dev))
        alone = torch.full((T, D), float("nan"), device=dev)
        layer.expert_ffn(alone)
        x2, ids2, w2 = np.concatenate([x, x]), np.concatenate([ids, ids]), np.concatenate([wts, wts])
        layer.set_routes(to_dev(x2, dev), to_dev(ids2, dev), to_dev(w2, dev))
        out2 = torch.full((2 * T, D), float("nan"), device=dev)
        layer.expert_ffn(out2)
        _sync()
        ctx.check()
        both = out2.cpu().numpy()
        assert np.array_equal(both[:T].view(np.uint32), alone.cpu().numpy().view(np.uint32))
        assert np.array_equal(both[T:].view(np.uint32), both[:T].view(np.uint32))
        assert rel_to_norm(both[:T], ref) < REL_TO_NORM
        ctx.set_path(0)


def test_routes_of_a_window_of_experts(zlib, dev):
    """zmoe_set_routes_window: model-wide expert ids on a layer that holds experts [first, first + E)"""
    import torch
    D, F, E, K, T = 1024, 512, 6, 4, 9
    first, total = 10, 24
    types = (synth.Q2_K, synth.Q2_K, synth.Q3_K)
    rng = synth.rng_for(31, 0)
    wg = to_dev(synth.expert_weights(types[0], E, F, D, rng), dev)
    wu = to_dev(synth.expert_weights(types[1], E, F, D, rng), dev)
    wd = to_dev(synth.expert_weights(types[2], E, D, F, rng), dev)
    x = to_dev(synth.activations(T, D, rng), dev)
    ids = np.stack([rng.permutation(total)[:K] for _ in range(T)]).astype(np.int32)
    ids[1, 0] = -1                                       # an inactive route stays inactive
    wts = to_dev(rng.uniform(0.05, 0.3, size=(T, K)).astype(np.float32), dev)
    local = np.where((ids >= first) & (ids < first + E), ids - first, -1).astype(np.int32)
    assert (local >= 0).sum() > 4
    ctx = zlib.Context(16, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, wg, wu, wd)
    layer.set_routes(x, to_dev(local, dev), wts)
    a = torch.full((T, D), float("nan"), device=dev)
    layer.expert_ffn(a)
    layer.set_routes_window(x, to_dev(ids, dev), wts, first)
    b = torch.full((T, D), float("nan"), device=dev)
    layer.expert_ffn(b)
    _sync()
    ctx.check()
    got_ids, _ = ctx.routes(T, K)
    assert np.array_equal(got_ids, local)
    assert torch.equal(a, b)


def test_deepseek_shaped_layer_with_shared_expert(zlib, oracle, dev):
    """fourth benchmark configuration, scaled down in expert count only: hidden 7168, ffn 2048,
    sigmoid gating, 8 groups with the top 4 kept, top-8, normalised weights, Q4_K, one shared expert"""
    import torch
    D, F, E, K, T = 7168, 2048, 64, 8, 3
    types = (synth.Q4_K,) * 3
    rng = synth.rng_for(29, 0)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    sg = synth.expert_weights(types[0], 1, F, D, rng)
    su = synth.expert_weights(types[1], 1, F, D, rng)
    sd = synth.expert_weights(types[2], 1, D, F, rng)
    bias = (rng.standard_normal(E) * 0.02).astype(np.float32)
    wr, x, probs, ids_ref, w_ref = routed_inputs(oracle, 29, T, D, E, K, gating=1, normalize=1, weight_scale=2.5,
                                                 bias=bias, n_groups=8, n_groups_used=4)
    ctx = zlib.Context(16, D, F, E, K)
    routed = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev),
                        router_w=to_dev(wr, dev), router_bias=to_dev(bias, dev), gating=1, weights_norm=1,
                        weights_scale=2.5, n_groups=8, n_groups_used=4)
    shared = zlib.Layer(ctx, D, F, 1, 1, types, to_dev(sg, dev), to_dev(su, dev), to_dev(sd, dev))
    xd = to_dev(x, dev)
    out = torch.empty((T, D), device=dev)
    routed.forward(xd, out)
    _sync()
    ids, wts = ctx.routes(T, K)
    assert np.array_equal(ids, ids_ref)
    # every token stays inside its 4 kept groups
    assert all(len({int(e) // (E // 8) for e in row}) <= 4 for row in ids)
    shared.dense_ffn(xd, out, accumulate=1)
    _sync()
    ctx.check()
    ref = oracle.moe_ffn(oracle.make_layer(D, F, E, K, types, wg, wu, wd), x, ids_ref, w_ref)
    ref += oracle.moe_ffn(oracle.make_layer(D, F, 1, 1, types, sg, su, sd), x, np.zeros((T, 1), np.int32),
                          np.ones((T, 1), np.float32))
    assert rel_to_norm(out.cpu().numpy(), ref) < REL_TO_NORM


def test_shared_expert_with_scalar_gate(zlib, oracle, dev):
    """shared = sigmoid(W_gi . x) * FFN(x), added to what the output holds (reference
    models/graph/ggml_moe_graph_builder.cpp:120-124)"""
    import torch
    D, F, T = 2048, 768, 6
    types = (synth.Q4_K,) * 3
    rng = synth.rng_for(31, 0)
    sg = synth.expert_weights(types[0], 1, F, D, rng)
    su = synth.expert_weights(types[1], 1, F, D, rng)
    sd = synth.expert_weights(types[2], 1, D, F, rng)
    x = synth.activations(T, D, rng)
    gw = (rng.standard_normal(D) * 0.05).astype(np.float32)
    base = rng.standard_normal((T, D)).astype(np.float32)
    ctx = zlib.Context(16, D, F, 1, 1)
    shared = zlib.Layer(ctx, D, F, 1, 1, types, to_dev(sg, dev), to_dev(su, dev), to_dev(sd, dev))
    out = to_dev(base.copy(), dev)
    shared.dense_ffn_gated(to_dev(x, dev), to_dev(gw, dev), out, accumulate=1)
    _sync()
    ctx.check()
    raw = oracle.moe_ffn(oracle.make_layer(D, F, 1, 1, types, sg, su, sd), x, np.zeros((T, 1), np.int32),
                         np.ones((T, 1), np.float32))
    gate = 1.0 / (1.0 + np.exp(-(x.astype(np.float64) @ gw.astype(np.float64))))
    ref = base + raw * gate[:, None].astype(np.float32)
    assert rel_to_norm(out.cpu().numpy() - base, ref - base) < REL_TO_NORM
    assert zlib.load().zmoe_dense_ffn_gated(shared.h, None, zlib.ptr(out), zlib.ptr(out), T, 0, None) == -1


@pytest.mark.parametrize("T", [3, 300])
def test_moe_forward_bf16_activations(zlib, oracle, dev, T):
    """bf16 activations (the third configuration's input type) give exactly what their f32 widening gives, on the
    decode kernels (3 tokens) and on the tensor-core path (300 tokens, 75 pairs per expert)"""
    import torch
    D, F, E, K = 1024, 512, 16, 4
    types = (synth.Q4_K,) * 3
    rng = synth.rng_for(37, T)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    wr = synth.router_weights(E, D, rng, sigma=0.05)
    xb = torch.from_numpy(synth.activations(T, D, rng)).to(dev).to(torch.bfloat16)
    xf = xb.to(torch.float32)
    ctx = zlib.Context(512, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev), router_w=to_dev(wr, dev))
    out_b = torch.zeros((T, D), device=dev)
    out_f = torch.zeros((T, D), device=dev)
    layer.forward(xf, out_f)
    _sync()
    ids_f, _ = ctx.routes(T, K)
    layer.forward_bf16(xb, out_b)
    _sync()
    ctx.check()
    ids_b, w_b = ctx.routes(T, K)
    assert np.array_equal(ids_f, ids_b)
    assert torch.equal(out_b, out_f)
    ref = oracle.moe_ffn(oracle.make_layer(D, F, E, K, types, wg, wu, wd), xf.cpu().numpy(), ids_b, w_b, fast=True)[0]
    assert rel_to_norm(out_b.cpu().numpy(), ref) < REL_TO_NORM


def test_moe_forward_host_buffers(zlib, oracle, dev):
    import torch
    D, F, E, K, T = 1024, 512, 16, 4, 4
    types = (synth.Q4_K,) * 3
    rng = synth.rng_for(19, 0)
    wg = synth.expert_weights(types[0], E, F, D, rng)
    wu = synth.expert_weights(types[1], E, F, D, rng)
    wd = synth.expert_weights(types[2], E, D, F, rng)
    wr, x, probs, ids_ref, w_ref = routed_inputs(oracle, 19, T, D, E, K)
    ctx = zlib.Context(8, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev),
                       router_w=to_dev(wr, dev))
    xh = torch.from_numpy(x).pin_memory()
    oh = torch.empty((T, D), dtype=torch.float32).pin_memory()
    layer.forward_host(xh, oh)
    Lr = oracle.make_layer(D, F, E, K, types, wg, wu, wd)
    ref = oracle.moe_ffn(Lr, x, ids_ref, w_ref)
    assert rel_to_norm(oh.numpy(), ref) < REL_TO_NORM
    first = oh.numpy().copy()
    # the same pinned buffers again
    for _ in range(3):
        oh.zero_()
        layer.forward_host(xh, oh)
        assert np.array_equal(oh.numpy().view(np.uint32), first.view(np.uint32))
    # new contents in the same buffers, another layer on the same context
    wr2, x2, _, ids2, w2 = routed_inputs(oracle, 23, T, D, E, K)
    assert wr2.shape == wr.shape
    layer2 = zlib.Layer(ctx, D, F, E, K, types, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev),
                        router_w=to_dev(wr2, dev))
    xh.copy_(torch.from_numpy(x2))
    for _ in range(3):
        layer2.forward_host(xh, oh)
        assert rel_to_norm(oh.numpy(), oracle.moe_ffn(Lr, x2, ids2, w2)) < REL_TO_NORM
    # pageable buffers
    xp, op = torch.from_numpy(x.copy()), torch.empty((T, D), dtype=torch.float32)
    for _ in range(3):
        layer.forward_host(xp, op)
        assert np.array_equal(op.numpy().view(np.uint32), first.view(np.uint32))


def test_capacity_and_state_errors(zlib, dev):
    import torch
    D, F, E, K = 512, 256, 8, 2
    rng = synth.rng_for(20, 0)
    w = to_dev(synth.expert_weights(synth.Q4_K, E, F, D, rng), dev)
    wd = to_dev(synth.expert_weights(synth.Q4_K, E, D, F, rng), dev)
    ctx = zlib.Context(4, D, F, E, K)
    layer = zlib.Layer(ctx, D, F, E, K, (synth.Q4_K,) * 3, w, w, wd,
                       router_w=torch.zeros((E, D), device=dev))
    x = torch.zeros((5, D), device=dev)
    with pytest.raises(zlib.ZmoeError) as e:
        layer.route(x)
    assert e.value.code == -6
    out = torch.zeros((2, D), device=dev)
    with pytest.raises(zlib.ZmoeError) as e:
        layer.expert_ffn(out)           # no routing for two tokens yet
    assert e.value.code == -8
    with pytest.raises(zlib.ZmoeError) as e:
        zlib.Layer(ctx, D, F, E, K, (synth.Q4_K, synth.Q4_K, 7), w, w, wd)   # a type without a kernel
    assert e.value.code == -2


# ---------------------------------------------------------------------------
# MUL_MAT_ID through the backend-op hook
# ---------------------------------------------------------------------------
def _hook_tensors(zlib, qtype, slab, off, I, O, E, stride, xd, K, T, x_per_route, ids_d, y):
    import torch
    rb = I // 256 * zlib.BLOCK_BYTES.get(qtype, 34)
    w = zlib.Tensor()
    w.type = qtype
    w.ne[:] = [I, O, E, 1]
    w.nb[:] = [0, rb, stride, stride * E]
    w.data = slab.data_ptr() + off
    x = zlib.Tensor()
    x.type = zlib.GGML_F32
    xr = K if x_per_route else 1
    x.ne[:] = [I, xr, T, 1]
    x.nb[:] = [4, 4 * I, 4 * I * xr, 4 * I * xr * T]
    x.data = xd.data_ptr()
    ids = zlib.Tensor()
    ids.type = zlib.GGML_I32
    ids.ne[:] = [K, T, 1, 1]
    ids.nb[:] = [4, 4 * K, 4 * K * T, 4 * K * T]
    ids.data = ids_d.data_ptr()
    yt = zlib.Tensor()
    yt.type = zlib.GGML_F32
    yt.ne[:] = [O, K, T, 1]
    yt.nb[:] = [4, 4 * O, 4 * O * K, 4 * O * K * T]
    yt.data = y.data_ptr()
    return w, x, ids, yt


@pytest.mark.parametrize("T", [1, 19])
def test_hook_mul_mat_id_strided_slab(zlib, oracle, dev, T):
    """gate|up|down slabs per expert viewed in place: each projection equals the planar
    layout bit for bit, ids -1 give zero rows, ids >= E give NaN rows, weights untouched"""
    import torch
    D, F, E, K = 256, 256, 9, 6
    qg, qd = synth.Q2_K, synth.Q3_K
    rng = synth.rng_for(21, T)
    wg = synth.expert_weights(qg, E, F, D, rng)
    wu = synth.expert_weights(qg, E, F, D, rng)
    wd = synth.expert_weights(qd, E, D, F, rng)
    gb, db = wg[0].size, wd[0].size
    stride = (2 * gb + db + 15) // 16 * 16
    slab = np.zeros((E, stride), dtype=np.uint8)
    slab[:, :gb] = wg.reshape(E, -1)
    slab[:, gb:2 * gb] = wu.reshape(E, -1)
    slab[:, 2 * gb:2 * gb + db] = wd.reshape(E, -1)
    slab_d = to_dev(slab, dev)
    keep = slab_d.clone()
    x = synth.activations(T, D, rng)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    ids[0, 1] = -1
    if T > 1:
        ids[3, 2] = E + 5
    xd, ids_d = to_dev(x, dev), to_dev(ids, dev)
    L = zlib.load()
    y_slab = torch.full((T, K, F), 7.0, device=dev)
    args = _hook_tensors(zlib, qg, slab_d, gb, D, F, E, stride, xd, K, T, False, ids_d, y_slab)   # the "up" plane
    assert L.zmoe_f32_quant_hook(*[C.byref(a) for a in args], None, False)     # support query
    assert torch.all(y_slab == 7.0)                                             # ... has no side effect
    assert L.zmoe_f32_quant_hook(*[C.byref(a) for a in args], None, True)
    planar = to_dev(wu, dev)
    y_planar = torch.full((T, K, F), 7.0, device=dev)
    args2 = _hook_tensors(zlib, qg, planar, 0, D, F, E, wu[0].size, xd, K, T, False, ids_d, y_planar)
    assert L.zmoe_f32_quant_hook(*[C.byref(a) for a in args2], None, True)
    _sync()
    a, b = y_slab.cpu().numpy(), y_planar.cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    ref = oracle.mul_mat_id(qg, x, wu, wu[0].size, ids, T, K, E, D, F, 0)
    valid = (ids >= 0) & (ids < E)
    assert rel_to_norm(a[valid], ref[valid]) < REL_TO_NORM
    assert np.all(a[0, 1] == 0.0)
    if T > 1:
        assert np.all(np.isnan(a[3, 2]))
    # each valid pair equals the stand-alone dense launch on that expert, bit for bit
    t, k = (T - 1, K - 1)
    dense = zlib.dense_matmul(qg, xd[t:t + 1].contiguous(), to_dev(wu[ids[t, k]], dev), F).cpu().numpy()
    assert np.array_equal(dense[0].view(np.uint32), a[t, k].view(np.uint32))
    assert torch.equal(slab_d, keep)
    # unsupported nodes are declined, not mis-computed
    bad = _hook_tensors(zlib, 8, slab_d, 0, D, F, E, stride, xd, K, T, False, ids_d, y_slab)    # Q8_0
    assert not L.zmoe_f32_quant_hook(*[C.byref(a) for a in bad], None, False)
