"""GPU parity of the dense kernels around the MoE block and of the decoder step built from them, against
the CPU restatement in oracle/decoder_ref.py: Q8_0 matmul (activation bytes' effect exact per block, f32
within 1e-3 of the output norm), RMSNorm, and a small decoder (prompt of several tokens, then greedy steps):
logits within 1e-3 of their norm after every step, the same greedy tokens.  Shapes follow the reference's
Q8_0 cases in tests/native/tests_basic_cuda.cpp:301-320 (long rows, few outputs; S > 1)."""
import numpy as np
import pytest

from helpers import REL_TO_NORM, rel_to_norm, to_dev
from zeromoe_b200 import synth

pytestmark = pytest.mark.gpu


def q8_0_weights(rows, cols, rng, d_sigma):
    nb = cols // 32
    blk = np.frombuffer(rng.bytes(rows * nb * 34), dtype=np.uint8).reshape(rows * nb, 34).copy()
    blk[:, 2:][blk[:, 2:] == 0x80] = 0x81          # int8 -128 does not occur in ggml's Q8_0 (values are in +-127)
    d = np.abs(rng.standard_normal(rows * nb, dtype=np.float32) * d_sigma).astype(np.float16)
    blk[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    return blk.reshape(rows, nb * 34)


@pytest.mark.parametrize("shape", [(512, 8, 3), (2048, 40, 1), (4096, 64, 5), (2048, 515, 9), (96, 7, 2), (7168, 16, 11)])
def test_q8_0_matmul_vs_oracle(zlib, oracle, dev, shape):
    import torch
    I, O, S = shape
    rng = synth.rng_for(51, I, O)
    w = q8_0_weights(O, I, rng, 0.01)
    x = synth.activations(S, I, rng)
    x[0, :32] = 0.0                           # an all-zero activation block
    if S > 1:
        x[1, 5] = 63.5                        # products that land on .5 exactly (round half away from zero)
        x[1, 6] = 127.0
    y = zlib.q8_0_matmul(to_dev(x, dev), to_dev(w, dev), O)
    torch.cuda.synchronize()
    ref = oracle.matmul_q8_0(x, w, S, I, O)
    assert rel_to_norm(y.cpu().numpy(), ref) < 1e-5       # integer block sums are exact: only the f32 order differs


def test_rmsnorm_vs_oracle(zlib, dev):
    import torch
    from oracle import decoder_ref as R
    rng = synth.rng_for(52, 0)
    x = synth.activations(5, 2048, rng) * 3.0
    w = (1.0 + 0.1 * rng.standard_normal(2048)).astype(np.float32)
    y = torch.empty((5, 2048), device=dev)
    xd, wd = to_dev(x, dev), to_dev(w, dev)
    zlib.load().launch_rmsnorm(zlib.ptr(y), zlib.ptr(xd), zlib.ptr(wd), 5, 2048, 1e-6)
    torch.cuda.synchronize()
    assert zlib.load().zmoe_last_status() == 0
    assert np.allclose(y.cpu().numpy(), R.rmsnorm(x, w, 1e-6), rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("hd", [64, 128])
def test_decoder_steps_vs_oracle(zlib, oracle, dev, hd):
    import torch
    from oracle import decoder_ref as R
    D, H, KV, F, E, K, V, NL = 256, 4, 2, 256, 8, 2, 512, 2
    ty = synth.Q4_K
    rng = synth.rng_for(53, hd)
    ctx = zlib.Context(16, D, F, E, K)
    glayers, rlayers, keep = [], [], []
    for l in range(NL):
        wg, wu = synth.expert_weights(ty, E, F, D, rng), synth.expert_weights(ty, E, F, D, rng)
        wd = synth.expert_weights(ty, E, D, F, rng)
        wr = synth.router_weights(E, D, rng, sigma=1.0 / 16)
        an = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        fn = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        wqkv = q8_0_weights((H + 2 * KV) * hd, D, rng, 0.0015)
        wo = q8_0_weights(D, H * hd, rng, 0.0015)
        dv = [to_dev(a, dev) for a in (wg, wu, wd, wr, an, fn, wqkv, wo)]
        keep.append(dv)
        moe = zlib.Layer(ctx, D, F, E, K, (ty,) * 3, dv[0], dv[1], dv[2], router_w=dv[3])
        glayers.append(dict(attn_norm=dv[4], ffn_norm=dv[5], wqkv=dv[6], wo=dv[7], moe=moe))
        rlayers.append(dict(attn_norm=an, ffn_norm=fn, wqkv=wqkv, wo=wo,
                            moe=dict(D=D, F=F, E=E, K=K, types=(ty,) * 3, wg=wg, wu=wu, wd=wd, wr=wr)))
    embd = q8_0_weights(V, D, rng, 0.02)
    head = q8_0_weights(V, D, rng, 0.002)
    on = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    d_embd, d_head, d_on = to_dev(embd, dev), to_dev(head, dev), to_dev(on, dev)
    dec = zlib.Decoder(glayers, d_embd, d_on, d_head, D, H, KV, hd, V, max_ctx=32, max_tokens=16)
    ref = R.Decoder(rlayers, embd, on, head, D, H, KV, hd, V)
    prompt = np.array([3, 141, 59, 26, 500, 358, 97], dtype=np.int32)
    dec.step(to_dev(prompt, dev))
    tok, pos, lg = dec.read(V)
    rtok, rlg = ref.step(prompt)
    ctx.check()
    assert pos == len(prompt)
    assert rel_to_norm(lg, rlg) < REL_TO_NORM
    for _ in range(4):
        # the same token goes into both, so one near-tie in the arg-max cannot make the runs diverge
        top2 = np.sort(rlg)[-2:]
        if top2[1] - top2[0] > 1e-3 * np.abs(rlg).max():
            assert tok == rtok
        dec.step(to_dev(np.array([rtok], dtype=np.int32), dev))
        tok, pos, lg = dec.read(V)
        rtok, rlg = ref.step([rtok])
        assert rel_to_norm(lg, rlg) < REL_TO_NORM
    # the device-resident loop: feeding back the sampled token without a host round trip gives the same tokens
    dec.reset()
    dec.step(to_dev(prompt, dev))
    first = dec.read()[0]
    dec.step()
    dec.step()
    chain = dec.read()
    dec.reset()
    dec.step(to_dev(prompt, dev))
    t1 = dec.read()[0]
    dec.step(to_dev(np.array([t1], dtype=np.int32), dev))
    t2 = dec.read()[0]
    dec.step(to_dev(np.array([t2], dtype=np.int32), dev))
    assert first == t1 and chain[0] == dec.read()[0] and chain[1] == len(prompt) + 2
