"""Expert parallelism on real GPUs: two ranks, each with half of the experts, must reproduce the
single-GPU layer.  Needs two CUDA devices; skipped otherwise."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
D, F, E, K, T = 1024, 512, 16, 4, 6
TYPES = (10, 10, 11)


def _weights():
    from zeromoe_b200 import synth
    rng = synth.rng_for(41, 0)
    return (synth.expert_weights(TYPES[0], E, F, D, rng), synth.expert_weights(TYPES[1], E, F, D, rng),
            synth.expert_weights(TYPES[2], E, D, F, rng), synth.router_weights(E, D, rng, sigma=1.0 / 32))


def _worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from zeromoe_b200 import expert_parallel as ep, lib, synth
    wg, wu, wd, wr = _weights()
    lo, hi = ep.expert_range(rank, world, E)
    w = [(torch.from_numpy(wg[lo:hi].copy()).to(dev), torch.from_numpy(wu[lo:hi].copy()).to(dev),
          torch.from_numpy(wd[lo:hi].copy()).to(dev), torch.from_numpy(wr).to(dev))]
    ctx = lib.Context(max(16, world * T), D, F, E, K)
    shard = ep.ExpertShard(ctx, rank, world, E, K, D, F, TYPES, w, dev)
    x = torch.from_numpy(synth.activations(T, D, synth.rng_for(41, 10 + rank))).to(dev)
    out = torch.empty((T, D), device=dev)
    shard.forward(0, x, out)
    torch.cuda.synchronize()
    ctx.check()
    results[rank] = out.cpu().numpy()
    dist.destroy_process_group()


def test_two_gpu_expert_parallel_matches_single_gpu(zlib, dev):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from zeromoe_b200 import synth
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, 29300 + os.getpid() % 500, results), nprocs=2, join=True)
    wg, wu, wd, wr = _weights()
    ctx = zlib.Context(16, D, F, E, K)
    t = [torch.from_numpy(a).to(dev) for a in (wg, wu, wd, wr)]
    layer = zlib.Layer(ctx, D, F, E, K, TYPES, t[0], t[1], t[2], router_w=t[3])
    for r in range(2):
        x = torch.from_numpy(synth.activations(T, D, synth.rng_for(41, 10 + r))).to(dev)
        ref = torch.empty((T, D), device=dev)
        layer.forward(x, ref)
        torch.cuda.synchronize()
        ref = ref.cpu().numpy()
        assert np.abs(results[r] - ref).max() / np.linalg.norm(ref) < 1e-6


# ---------------------------------------------------------------------------
# all-to-all exchange (zmoe_ep_forward) with the fourth configuration's router: sigmoid gating, groups,
# selection bias, weight scale, shared expert
# ---------------------------------------------------------------------------
D2, F2, E2, K2, T2 = 1024, 512, 16, 4, 40
TYPES2 = (12, 12, 12)
ROUTER2 = dict(gating=1, weights_norm=1, weights_scale=2.5, n_groups=4, n_groups_used=2)


def _weights2():
    from zeromoe_b200 import synth
    rng = synth.rng_for(43, 0)
    ws = [synth.expert_weights(TYPES2[0], E2, F2, D2, rng), synth.expert_weights(TYPES2[1], E2, F2, D2, rng),
          synth.expert_weights(TYPES2[2], E2, D2, F2, rng)]
    shared = [synth.expert_weights(TYPES2[0], 1, F2, D2, rng), synth.expert_weights(TYPES2[1], 1, F2, D2, rng),
              synth.expert_weights(TYPES2[2], 1, D2, F2, rng)]
    wr = synth.router_weights(E2, D2, rng, sigma=1.0 / 32)
    bias = (rng.standard_normal(E2) * 0.05).astype(np.float32)
    return ws, shared, wr, bias


def _worker_a2a(rank, world, port, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from zeromoe_b200 import expert_parallel as ep, lib, synth
    ws, sh, wr, bias = _weights2()
    lo, hi = ep.expert_range(rank, world, E2)
    w = [tuple(torch.from_numpy(a[lo:hi].copy()).to(dev) for a in ws) + (torch.from_numpy(wr).to(dev),)]
    shared = [tuple(torch.from_numpy(a).to(dev) for a in sh)]
    ctx = lib.Context(world * T2, D2, F2, E2, K2)
    shard = ep.ExpertShard(ctx, rank, world, E2, K2, D2, F2, TYPES2, w, dev,
                           router=dict(ROUTER2, bias=[torch.from_numpy(bias).to(dev)]), shared=shared, max_tokens=T2)
    x = torch.from_numpy(synth.activations(T2, D2, synth.rng_for(43, 10 + rank))).to(dev)
    outs = {}
    for mode in ("a2a", "gather", "a2a"):
        out = torch.full((T2, D2), float("nan"), device=dev)
        shard.forward(0, x, out, mode=mode)
        torch.cuda.synchronize()
        ctx.check()
        outs.setdefault(mode, []).append(out.cpu().numpy())
    sent, recv = shard.last_rows()
    results[rank] = (outs["a2a"][0], outs["gather"][0], outs["a2a"][1], sent, recv)
    shard.close()
    dist.destroy_process_group()


def test_two_gpu_all_to_all_matches_single_gpu(zlib, dev):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from zeromoe_b200 import synth
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker_a2a, args=(2, 29800 + os.getpid() % 500, results), nprocs=2, join=True)
    ws, sh, wr, bias = _weights2()
    ctx = zlib.Context(T2, D2, F2, E2, K2)
    sctx = zlib.Context(T2, D2, F2, 1, 1)
    t = [torch.from_numpy(a).to(dev) for a in ws]
    layer = zlib.Layer(ctx, D2, F2, E2, K2, TYPES2, t[0], t[1], t[2], router_w=torch.from_numpy(wr).to(dev),
                       router_bias=torch.from_numpy(bias).to(dev), **ROUTER2)
    ts = [torch.from_numpy(a).to(dev) for a in sh]
    shared = zlib.Layer(sctx, D2, F2, 1, 1, TYPES2, ts[0], ts[1], ts[2])
    total_sent = 0
    for r in range(2):
        x = torch.from_numpy(synth.activations(T2, D2, synth.rng_for(43, 10 + r))).to(dev)
        ref = torch.empty((T2, D2), device=dev)
        layer.forward(x, ref)
        shared.dense_ffn(x, ref, accumulate=1)
        torch.cuda.synchronize()
        ref = ref.cpu().numpy()
        a2a, gather, a2a_again, sent, recv = results[r]
        # the ranks' partial sums are added in another order than the single GPU's k order
        assert np.abs(a2a - ref).max() / np.linalg.norm(ref) < 1e-6
        assert np.abs(gather - ref).max() / np.linalg.norm(ref) < 1e-6
        assert np.array_equal(a2a.view(np.uint32), a2a_again.view(np.uint32))     # reproducible
        assert T2 <= sent <= 2 * T2
        total_sent += sent
    assert total_sent == results[0][4] + results[1][4]      # every row sent was received
