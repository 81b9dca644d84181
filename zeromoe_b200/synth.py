"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations: random quantised super-blocks (uniform random quants
and packed scale fields, fp16 super-scales |N(0, 0.01)|), router weights
N(0, 0.02), activations N(0, 1).  Stands in for real checkpoints.
"""
import numpy as np

Q2_K, Q3_K, Q4_K, IQ2_XXS = 10, 11, 12, 16
BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, IQ2_XXS: 66}
TYPE_NAMES = {Q2_K: "Q2_K", Q3_K: "Q3_K", Q4_K: "Q4_K", IQ2_XXS: "IQ2_XXS"}
# byte offsets of the fp16 super-scales inside a block
_HALF_FIELDS = {Q2_K: (80, 82), Q3_K: (108,), Q4_K: (0, 2), IQ2_XXS: (0,)}


def rng_for(seed, *stream):
    """one independent Philox stream per (seed, tensor id...)"""
    key = [int(seed) & 0xFFFFFFFFFFFFFFFF, 0]
    for i, s in enumerate(stream):
        key[1] = (key[1] * 1000003 + int(s) + 1 + i) & 0xFFFFFFFFFFFFFFFF
    return np.random.Generator(np.random.Philox(key=key))


def random_blocks(qtype, n_blocks, rng, d_sigma=0.01):
    """uint8 [n_blocks, block_bytes]"""
    bb = BLOCK_BYTES[qtype]
    blocks = np.frombuffer(rng.bytes(n_blocks * bb), dtype=np.uint8).reshape(n_blocks, bb).copy()
    for off in _HALF_FIELDS[qtype]:
        h = np.abs(rng.standard_normal(n_blocks, dtype=np.float32) * d_sigma).astype(np.float16)
        blocks[:, off:off + 2] = h.view(np.uint8).reshape(n_blocks, 2)
    return blocks


def expert_weights(qtype, E, O, I, rng, d_sigma=0.01):
    """uint8 [E, O, I/256*block_bytes]: E experts of O packed rows of I elements"""
    assert I % 256 == 0
    nb = I // 256
    return random_blocks(qtype, E * O * nb, rng, d_sigma).reshape(E, O, nb * BLOCK_BYTES[qtype])


def router_weights(E, D, rng, sigma=0.02):
    return (rng.standard_normal((E, D), dtype=np.float32) * sigma).astype(np.float32)


def activations(T, D, rng):
    return rng.standard_normal((T, D), dtype=np.float32)


def exact_activations(T, D, rng):
    """Integers in [-127, 127] with +-127 present in every 256-block, so Q8_K
    quantisation is lossless (the reference's EXACT_INPUTS recipe,
    tests/test_phase_alias_numerics.cpp:104-107)."""
    x = rng.integers(-127, 128, size=(T, D)).astype(np.float32)
    x[:, ::256] = -127.0
    return x


def zipf_logit_bias(E, s, rng):
    """log of a Zipf(s) distribution over a random expert ranking; added to the
    router logits it skews expert load the way the prefill configuration asks."""
    rank = rng.permutation(E).astype(np.float64) + 1.0
    p = rank ** (-s)
    p /= p.sum()
    return np.log(p).astype(np.float32)
