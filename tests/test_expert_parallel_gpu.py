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
