"""GPU test of zmoe_matmul_noalloc, the matmul entry point for callers that cannot
allocate device memory (engines that own the whole GPU through a pool of their own,
code inside another framework's stream capture, real-time loops).  Its scratch is a
fixed array inside the library instead of cudaMalloc'ed buffers, so the checks are:
same bits as the allocating entry points, correct when called twice in a row on
different problems (the array keeps the previous call's contents), and a clean
refusal beyond the fixed size.  Collected last on purpose (file name)."""
import numpy as np
import pytest

from helpers import to_dev
from zeromoe_b200 import synth

pytestmark = pytest.mark.gpu

LIMIT = 1 << 20


def _run(zlib, dev, qtype, I, O, S, seed):
    import torch
    rng = synth.rng_for(77, qtype, seed)
    w = to_dev(synth.expert_weights(qtype, 1, O, I, rng)[0], dev)
    x = to_dev(synth.activations(S, I, rng), dev)
    y = torch.full((S, O), float("nan"), device=dev)
    zlib.check(zlib.load().zmoe_matmul_noalloc(qtype, zlib.ptr(y), zlib.ptr(x), zlib.ptr(w), S, I, O, None),
               "zmoe_matmul_noalloc")
    ref = zlib.dense_matmul(qtype, x, w, O)
    torch.cuda.synchronize()
    return y.cpu().numpy(), ref.cpu().numpy()


def test_noalloc_matches_allocating_entry_twice_in_a_row(zlib, dev):
    # first call: a large problem that fills much of the array; second: a small one of another
    # type right behind it, which must not see what the first left there
    for qtype, I, O, S, seed in ((synth.Q4_K, 4096, 96, 120, 1), (synth.Q3_K, 768, 20, 3, 2),
                                 (synth.Q2_K, 2048, 64, 7, 3)):
        got, ref = _run(zlib, dev, qtype, I, O, S, seed)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (qtype, I, O, S)


def test_noalloc_refuses_what_does_not_fit(zlib, dev):
    import torch
    I, S, O = 4096, 400, 8           # 400 rows of 4096 need more than the fixed megabyte
    x = torch.zeros((S, I), device=dev)
    w = torch.zeros(O * (I // 256) * 144, dtype=torch.uint8, device=dev)
    y = torch.zeros((S, O), device=dev)
    rc = zlib.load().zmoe_matmul_noalloc(synth.Q4_K, zlib.ptr(y), zlib.ptr(x), zlib.ptr(w), S, I, O, None)
    assert rc == -6
    assert zlib.load().zmoe_matmul_noalloc(synth.Q4_K, None, zlib.ptr(x), zlib.ptr(w), 1, I, O, None) == -1
    assert zlib.load().zmoe_matmul_noalloc(5, zlib.ptr(y), zlib.ptr(x), zlib.ptr(w), 1, I, O, None) == -2
