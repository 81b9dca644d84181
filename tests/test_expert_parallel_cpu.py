"""Expert-parallel exchange on two CPU ranks (gloo): sharding the experts over ranks and
exchanging token rows must reproduce the single-rank layer.  The CPU oracle stands in for
the CUDA library as the per-rank compute."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

D, F, E, K, T = 512, 256, 8, 3, 4
TYPES = (12, 12, 11)


def _inputs():
    sys.path.insert(0, ROOT)
    from zeromoe_b200 import synth
    rng = synth.rng_for(31, 0)
    wg = synth.expert_weights(TYPES[0], E, F, D, rng)
    wu = synth.expert_weights(TYPES[1], E, F, D, rng)
    wd = synth.expert_weights(TYPES[2], E, D, F, rng)
    xs = [synth.activations(T, D, synth.rng_for(31, 10 + r)) for r in range(2)]
    ids = [np.stack([synth.rng_for(31, 20 + r, t).permutation(E)[:K] for t in range(T)]).astype(np.int32)
           for r in range(2)]
    ws = [synth.rng_for(31, 30 + r).uniform(0.1, 0.5, size=(T, K)).astype(np.float32) for r in range(2)]
    return wg, wu, wd, xs, ids, ws


def _worker_a2a(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    from zeromoe_b200 import expert_parallel as ep
    wg, wu, wd, xs, ids, ws = _inputs()
    e_lo, e_hi = ep.expert_range(rank, world, E)
    L = O.make_layer(D, F, e_hi - e_lo, K, TYPES, wg[e_lo:e_hi].copy(), wu[e_lo:e_hi].copy(), wd[e_lo:e_hi].copy())
    seen = {}

    def compute(x_recv, ids_recv, w_recv):
        seen["rows"] = x_recv.shape[0]
        local = ep.localise_ids(ids_recv, e_lo, e_hi)
        assert bool((local >= 0).any(dim=1).all()), "a row arrived that names no local expert"
        return torch.from_numpy(O.moe_ffn(L, x_recv.numpy(), local.numpy(), w_recv.numpy()))
    my_ids = ids[rank].copy()
    if rank == 1:
        my_ids[2, :] = -1            # a token with no active route: goes nowhere, output row is zero
    out = ep.exchange_forward_a2a(torch.from_numpy(xs[rank]), torch.from_numpy(my_ids), torch.from_numpy(ws[rank]), E,
                                  compute)
    results[rank] = (out.numpy(), seen.get("rows", 0))
    dist.destroy_process_group()


def test_two_rank_all_to_all_matches_single_rank(oracle):
    """token rows travel once to every rank that owns one of their experts and come back pre-reduced"""
    world = 2
    port = 31000 + os.getpid() % 2000
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker_a2a, args=(world, port, results), nprocs=world, join=True)
    wg, wu, wd, xs, ids, ws = _inputs()
    L = oracle.make_layer(D, F, E, K, TYPES, wg, wu, wd)
    ids[1][2, :] = -1
    total_rows = 0
    for r in range(world):
        ref = oracle.moe_ffn(L, xs[r], ids[r], ws[r])
        got, rows = results[r]
        total_rows += rows
        assert np.abs(got - ref).max() / np.linalg.norm(ref) < 1e-6
    assert np.all(results[1][0][2] == 0.0)
    # every (token, owning rank) pair is one row: no more than tokens x ranks, no fewer than routed tokens
    assert 2 * T - 1 <= total_rows <= 2 * world * T


def test_destination_plan_is_stable():
    from zeromoe_b200 import expert_parallel as ep
    ids = torch.tensor([[0, 5], [6, 7], [-1, 9], [3, 1]], dtype=torch.int32)
    mask, counts, tokens = ep.destination_plan(ids, 8, 2)       # ranks own experts 0..3 and 4..7; 9 is out of range
    assert mask.tolist() == [[True, True], [False, True], [False, False], [True, False]]
    assert counts == [2, 2]
    assert [t.tolist() for t in tokens] == [[0, 3], [0, 1]]


def _worker(rank, world, port, results, own_mapping=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    from zeromoe_b200 import expert_parallel as ep
    wg, wu, wd, xs, ids, ws = _inputs()
    e_lo, e_hi = ep.expert_range(rank, world, E)
    L = O.make_layer(D, F, e_hi - e_lo, K, TYPES, wg[e_lo:e_hi].copy(), wu[e_lo:e_hi].copy(), wd[e_lo:e_hi].copy())

    def compute(x_all, ids_local, w_all):
        return torch.from_numpy(O.moe_ffn(L, x_all.numpy(), ids_local.numpy(), w_all.numpy()))
    if own_mapping:
        # the backend maps model-wide ids into its window itself (what zmoe_set_routes_window does on the GPU)
        # and the result lands in the caller's tensor
        def compute_global(x_all, ids_all, w_all):
            return compute(x_all, ep.localise_ids(ids_all, e_lo, e_hi), w_all)
        out = torch.full((T, D), float("nan"))
        ret = ep.exchange_forward(torch.from_numpy(xs[rank]), torch.from_numpy(ids[rank]), torch.from_numpy(ws[rank]),
                                  e_lo, e_hi, compute_global, out=out, localise=False)
        assert ret is out
    else:
        out = ep.exchange_forward(torch.from_numpy(xs[rank]), torch.from_numpy(ids[rank]), torch.from_numpy(ws[rank]),
                                  e_lo, e_hi, compute)
    results[rank] = out.numpy()
    dist.destroy_process_group()


@pytest.mark.parametrize("own_mapping", [False, True])
def test_two_rank_exchange_matches_single_rank(oracle, own_mapping):
    world = 2
    port = 29000 + (os.getpid() + 7 * own_mapping) % 2000
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results, own_mapping), nprocs=world, join=True)
    wg, wu, wd, xs, ids, ws = _inputs()
    L = oracle.make_layer(D, F, E, K, TYPES, wg, wu, wd)
    for r in range(world):
        ref = oracle.moe_ffn(L, xs[r], ids[r], ws[r])
        got = results[r]
        # the only difference is the order in which the two ranks' partial sums are added
        assert np.abs(got - ref).max() / np.linalg.norm(ref) < 1e-6


def test_localise_ids():
    from zeromoe_b200 import expert_parallel as ep
    ids = torch.tensor([[0, 5, 7], [4, 3, -1]], dtype=torch.int32)
    assert ep.localise_ids(ids, 4, 8).tolist() == [[-1, 1, 3], [0, -1, -1]]
    assert [ep.expert_range(r, 8, 256) for r in (0, 7)] == [(0, 32), (224, 256)]
