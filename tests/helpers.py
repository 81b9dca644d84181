"""shared helpers of the parity tests"""
import numpy as np

from zeromoe_b200 import synth

TYPES = (synth.Q2_K, synth.Q3_K, synth.Q4_K, synth.IQ2_XXS)
# tolerance the path is specified to: max-abs error relative to the norm of the reference output
REL_TO_NORM = 1e-3


def rel_to_norm(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / (np.linalg.norm(ref) + 1e-30))


def to_dev(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def routed_inputs(oracle, seed, T, D, E, K, gating=0, min_margin=2e-5, sigma=None, **kw):
    """router weights and activations whose top-k has no near tie (re-drawn until so)"""
    if sigma is None:
        sigma = 1.0 / np.sqrt(D)   # logits ~ N(0, 1): no saturated gates
    for attempt in range(200):
        rng = synth.rng_for(seed, 1000 + attempt)
        wr = synth.router_weights(E, D, rng, sigma=sigma)
        x = synth.activations(T, D, rng)
        logits = oracle.router_logits(x, wr)
        probs, ids, w, margin = oracle.router_select(logits, K, gating=gating, **kw)
        if margin > min_margin:
            return wr, x, probs, ids, w
    raise AssertionError("could not draw tie-free router inputs")
