"""GPU parity at the sizes the benchmark times: the third configuration as `bench.py` runs it
(128 experts, 4096 tokens, Zipf-skewed load, tensor-core grouped GEMM chosen by the library), one
rank's shard of the fourth configuration (32 of 256 experts, 7168 / 2048, Q4_K, sigmoid gating with 8
groups of which 4 are used, shared expert) at 64 tokens (decode kernels) and 1024 tokens (grouped
GEMM), and the reporting paths for device-side problems.

The CPU side is the oracle's AVX2 twin (bit-identical to the scalar oracle, see
tests/test_oracle_pins.py); tolerances as everywhere: expert ids exact, f32 outputs within 1e-3
max-abs relative to the norm of the reference output.  Shapes follow the reference's own large
cases: tests/native/tests_basic_cuda.cpp:301-320 (long rows), tests/test_dsv41_cache_graph.cpp:60-185
(hundreds of tokens through MUL_MAT_ID).
"""
import numpy as np
import pytest

from helpers import REL_TO_NORM, rel_to_norm, to_dev
from zeromoe_b200 import synth

pytestmark = pytest.mark.gpu


def _sync():
    import torch
    torch.cuda.synchronize()


def test_prefill_configuration_full_size(zlib, oracle, dev):
    """hidden 4096, 128 experts top-8, ffn 1536, IQ2_XXS, 4096 tokens, Zipf(1.1) expert load: the head
    expert holds thousands of pairs (many pair blocks), the tail a few tens (a ragged single block)"""
    import torch
    D, F, E, K, T = 4096, 1536, 128, 8, 4096
    ty = synth.IQ2_XXS
    rng = synth.rng_for(31, 3)
    wg = synth.expert_weights(ty, E, F, D, rng)
    wu = synth.expert_weights(ty, E, F, D, rng)
    wd = synth.expert_weights(ty, E, D, F, rng)
    wr = synth.router_weights(E, D, rng, sigma=0.02)
    x = synth.activations(T, D, rng)
    # Zipf(1.1) over a random expert ranking as a selection bias on the router probabilities
    rank = rng.permutation(E).astype(np.float64) + 1.0
    pz = rank ** -1.1
    bias = (2.0 * pz / pz.sum()).astype(np.float32)

    ctx = zlib.Context(T, D, F, E, K)
    tg, tu, td = to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev)
    layer = zlib.Layer(ctx, D, F, E, K, (ty,) * 3, tg, tu, td, router_w=to_dev(wr, dev), router_bias=to_dev(bias, dev))
    out = torch.full((T, D), float("nan"), device=dev)
    layer.forward(to_dev(x, dev), out)      # path 0: the library picks the grouped GEMM at 256 pairs per expert
    _sync()
    ctx.check()
    ids, wts = ctx.routes(T, K)
    freq = ctx.expert_freq(E)
    assert freq.sum() == T * K and freq.max() >= 2048 and freq.min() < 64, (freq.max(), freq.min())

    # router: the same experts as the oracle for every token whose selection is not a near tie
    logits = oracle.router_logits(x, wr)
    _, ids_ref, w_ref, _ = oracle.router_select(logits, K, bias=bias)
    same = (ids == ids_ref).all(axis=1)
    assert same.mean() > 0.995, same.mean()
    assert np.allclose(wts[same], w_ref[same], atol=1e-5)

    # expert FFN + combine on the routes the device chose
    Lr = oracle.make_layer(D, F, E, K, (ty,) * 3, wg, wu, wd)
    ref, _ = oracle.moe_ffn(Lr, x, ids, wts, fast=True)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_to_norm(got, ref) < REL_TO_NORM
    assert ctx.bad_counts() == (0, 0)


def _shard_inputs(oracle, T, rank_id):
    D, F, E_all, E_loc, K = 7168, 2048, 256, 32, 8
    ty = synth.Q4_K
    rng = synth.rng_for(32, 4, rank_id)
    wg = synth.expert_weights(ty, E_loc, F, D, rng)
    wu = synth.expert_weights(ty, E_loc, F, D, rng)
    wd = synth.expert_weights(ty, E_loc, D, F, rng)
    sg = synth.expert_weights(ty, 1, F, D, rng)
    su = synth.expert_weights(ty, 1, F, D, rng)
    sd = synth.expert_weights(ty, 1, D, F, rng)
    wr = synth.router_weights(E_all, D, rng, sigma=1.0 / np.sqrt(D))
    rbias = (rng.standard_normal(E_all) * 0.05).astype(np.float32)
    x = synth.activations(T, D, rng)
    logits = oracle.router_logits(x, wr)
    _, ids, w, _ = oracle.router_select(logits, K, gating=1, normalize=1, weight_scale=2.5, bias=rbias,
                                        n_groups=8, n_groups_used=4)
    return (D, F, E_all, E_loc, K, ty), (wg, wu, wd), (sg, su, sd), x, ids, w


@pytest.mark.parametrize("T", [64, 1024])
def test_expert_parallel_shard_of_the_fourth_configuration(zlib, oracle, dev, T):
    """rank 3 of 8: experts 96..127 of 256; routes of the whole model supplied through the window entry,
    shared expert added on top.  64 tokens take the decode kernels (4032-byte rows: the un-padded copy
    path), 1024 tokens the grouped GEMM."""
    import torch
    rank_id = 3
    (D, F, E_all, E_loc, K, ty), (wg, wu, wd), (sg, su, sd), x, ids, w = _shard_inputs(oracle, T, rank_id)
    first = rank_id * E_loc
    local = np.where((ids >= first) & (ids < first + E_loc), ids - first, -1).astype(np.int32)
    assert (local >= 0).sum() > 0

    ctx = zlib.Context(T, D, F, E_loc, K)
    layer = zlib.Layer(ctx, D, F, E_loc, K, (ty,) * 3, to_dev(wg, dev), to_dev(wu, dev), to_dev(wd, dev))
    sctx = zlib.Context(T, D, F, 1, 1)
    shared = zlib.Layer(sctx, D, F, 1, 1, (ty,) * 3, to_dev(sg, dev), to_dev(su, dev), to_dev(sd, dev))
    xd = to_dev(x, dev)
    out = torch.full((T, D), float("nan"), device=dev)
    layer.set_routes_window(xd, to_dev(ids, dev), to_dev(w, dev), first)
    layer.expert_ffn(out)
    _sync()
    ctx.check()
    got_ids, _ = ctx.routes(T, K)
    assert np.array_equal(got_ids, local)
    routed = out.cpu().numpy().copy()
    shared.dense_ffn(xd, out, accumulate=1)
    _sync()
    sctx.check()

    ref_routed, _ = oracle.moe_ffn(oracle.make_layer(D, F, E_loc, K, (ty,) * 3, wg, wu, wd), x, local, w, fast=True)
    ref_shared, _ = oracle.moe_ffn(oracle.make_layer(D, F, 1, 1, (ty,) * 3, sg, su, sd), x,
                                   np.zeros((T, 1), np.int32), np.ones((T, 1), np.float32), fast=True)
    assert rel_to_norm(routed, ref_routed) < REL_TO_NORM
    assert rel_to_norm(out.cpu().numpy(), ref_routed + ref_shared) < REL_TO_NORM
    # tokens none of whose routes are local get an exactly zero routed row
    none_local = (local < 0).all(axis=1)
    if none_local.any():
        assert np.all(routed[none_local] == 0.0)


def test_expired_device_wait_is_reported(zlib, dev):
    """a bounded wait that runs out on the handle-free entries becomes ZMOE_ERR_DEVICE_WAIT: the self-test
    warp waits on a barrier nothing arrives on, gives up after its poll limit, raises the error word and
    returns; the status call reports it once and clears it"""
    L = zlib.load()
    assert L.zmoe_device_status() == 0
    zlib.check(L.zmoe_selftest_wait_expiry(None), "zmoe_selftest_wait_expiry")
    assert L.zmoe_device_status() == -7
    assert L.zmoe_device_status() == 0
    # the device and the library stay usable
    import torch
    rng = synth.rng_for(33, 0)
    wq = synth.expert_weights(synth.Q4_K, 1, 8, 512, rng)[0]
    xq = synth.activations(3, 512, rng)
    y = zlib.dense_matmul(synth.Q4_K, to_dev(xq, dev), to_dev(wq, dev), 8)
    _sync()
    assert torch.isfinite(y).all()
    assert L.zmoe_device_status() == 0


def test_fused_swiglu_counts_non_finite_inputs(zlib, oracle, dev):
    """a NaN super-scale in one gate row and an infinite one in one up row turn that row's value non-finite
    for every pair routed to the expert: the fused epilogue counts them (reference
    kernels/math/expert_activation.cu:42-44), on the decode kernels and on the grouped GEMM"""
    import torch
    D, F, E, K, T = 512, 256, 4, 2, 48
    rng = synth.rng_for(34, 0)
    ty = synth.Q4_K
    wg, wu = synth.expert_weights(ty, E, F, D, rng), synth.expert_weights(ty, E, F, D, rng)
    wd = synth.expert_weights(ty, E, D, F, rng)
    x = synth.activations(T, D, rng)
    ids = np.stack([np.arange(T) % E, (np.arange(T) + 1) % E], axis=1).astype(np.int32)
    w = np.full((T, K), 0.5, dtype=np.float32)
    pairs_per_expert = T * K // E
    wg_nan = wg.copy()
    wg_nan[1, 5, 0:2] = (0x00, 0x7E)        # fp16 NaN in d of expert 1, gate row 5, first super-block
    wu_inf = wu.copy()
    wu_inf[2, 9, 144:146] = (0x00, 0x7C)    # fp16 +inf in d of expert 2, up row 9, second super-block
    ctx = zlib.Context(T, D, F, E, K)
    out = torch.empty((T, D), device=dev)
    xd, idd, wdv = to_dev(x, dev), to_dev(ids, dev), to_dev(w, dev)
    tdn = to_dev(wd, dev)

    def run(g, u, path):
        layer = zlib.Layer(ctx, D, F, E, K, (ty,) * 3, to_dev(g, dev), to_dev(u, dev), tdn)
        ctx.set_path(path)
        layer.set_routes(xd, idd, wdv)
        layer.expert_ffn(out)
        _sync()
        ctx.check()
        return ctx.bad_counts()

    for path in (1, 2):
        assert run(wg, wu, path) == (0, 0)
        assert run(wg_nan, wu, path) == (pairs_per_expert, 0), path
        assert ctx.bad_counts() == (0, 0)      # cleared by the read
    # an infinite scale stays an infinity only where the sums are integer (decode kernels); in the fp16
    # GEMM the row's products of both signs meet as inf - inf
    assert run(wg, wu_inf, 1) == (0, pairs_per_expert)
    n_nan, n_inf = run(wg, wu_inf, 2)
    assert n_nan + n_inf == pairs_per_expert
