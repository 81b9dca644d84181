"""CPU restatement of the decoder step around the MoE block (numpy + the C oracle).

TEST INFRASTRUCTURE ONLY: imported by tests/ and by the benchmark's check, never by the
zeromoe_b200 package.

What it restates (reference files): RMSNorm kernels/math/rmsnorm.cu:6-78; RoPE with interleaved
pairs and the angle built by repeated f32 multiplication, models/base/rope.hpp:52-118 with
rope_ext_factor = 0; grouped-query attention with scores q.k / sqrt(head_dim) and a
max-subtracted softmax, core/attention_layer.cpp:2633-2690, over a KV cache that holds fp16 values;
dense Q8_0 matmuls as ggml's CPU MUL_MAT does them (oracle/zmoe_oracle_dense.c); the MoE block is the
oracle's router + expert FFN; sampling is the arg-max with the lowest index on ties.
Parity unpinned: the reference's attention code needs its engine (GGUF model, ggml) to run, so there
is no executable or golden reference for this composition in the checkout; each piece follows the
cited formula.
"""
import numpy as np

from . import oracle as O

f32 = np.float32


def rmsnorm(x, w, eps):
    x = x.astype(f32)
    ms = (x * x).sum(axis=-1, dtype=f32) / f32(x.shape[-1])
    inv = f32(1.0) / np.sqrt(ms + f32(eps), dtype=f32)
    return (x * inv[..., None] * w).astype(f32)


def rope(v, positions, theta):
    """v [T, heads, hd] -> rotated copy; pairs (2j, 2j+1); angle_j = pos * scale * scale ... (j factors) in f32"""
    T, Hh, hd = v.shape
    scale = f32(np.power(f32(theta), f32(-2.0) / f32(hd)))
    out = v.astype(f32).copy()
    for t in range(T):
        ang = f32(positions[t])
        for j in range(hd // 2):
            c, s = f32(np.cos(ang, dtype=f32)), f32(np.sin(ang, dtype=f32))
            a, b = out[t, :, 2 * j].copy(), out[t, :, 2 * j + 1].copy()
            out[t, :, 2 * j] = a * c - b * s
            out[t, :, 2 * j + 1] = a * s + b * c
            ang = f32(ang * scale)
    return out


class Decoder:
    """layers: list of dicts(attn_norm, wqkv (uint8 Q8_0 rows), wo, ffn_norm, moe=dict(D, F, E, K, types, wg, wu, wd,
    wr, router kwargs))"""

    def __init__(self, layers, tok_embd, out_norm, lm_head, d_model, n_heads, n_kv_heads, head_dim, vocab, rms_eps=1e-6,
                 rope_theta=10000.0):
        self.L, self.embd, self.out_norm, self.head = layers, tok_embd, out_norm, lm_head
        self.D, self.H, self.KV, self.hd, self.V = d_model, n_heads, n_kv_heads, head_dim, vocab
        self.eps, self.theta = rms_eps, rope_theta
        self.kc = [np.zeros((0, n_kv_heads, head_dim), np.float16) for _ in layers]
        self.vc = [np.zeros((0, n_kv_heads, head_dim), np.float16) for _ in layers]
        self.pos = 0
        self.moe = [O.make_layer(m["D"], m["F"], m["E"], m["K"], m["types"], m["wg"], m["wu"], m["wd"])
                    for m in (l["moe"] for l in layers)]

    def step(self, tokens):
        """returns (next token, logits [vocab]) for the last of the given tokens"""
        T = len(tokens)
        D, H, KV, hd = self.D, self.H, self.KV, self.hd
        h = O.dequantize_q8_0(self.embd[np.asarray(tokens)], D)
        positions = np.arange(self.pos, self.pos + T)
        for l, lay in enumerate(self.L):
            xn = rmsnorm(h, lay["attn_norm"], self.eps)
            qkv = O.matmul_q8_0(xn, lay["wqkv"], T, D, (H + 2 * KV) * hd)
            q = rope(qkv[:, :H * hd].reshape(T, H, hd), positions, self.theta)
            k = rope(qkv[:, H * hd:(H + KV) * hd].reshape(T, KV, hd), positions, self.theta)
            v = qkv[:, (H + KV) * hd:].reshape(T, KV, hd)
            self.kc[l] = np.concatenate([self.kc[l], k.astype(np.float16)])
            self.vc[l] = np.concatenate([self.vc[l], v.astype(np.float16)])
            ao = np.zeros((T, H, hd), f32)
            G = H // KV
            for t in range(T):
                n = self.pos + t + 1
                K_, V_ = self.kc[l][:n].astype(f32), self.vc[l][:n].astype(f32)
                for hh in range(H):
                    s = (K_[:, hh // G, :] @ q[t, hh]).astype(f32) * f32(1.0 / np.sqrt(f32(hd)))
                    p = np.exp(s - s.max(), dtype=f32)
                    p = p / p.sum(dtype=f32)
                    ao[t, hh] = p @ V_[:, hh // G, :]
            h = (h + O.matmul_q8_0(ao.reshape(T, H * hd), lay["wo"], T, H * hd, D)).astype(f32)
            xn = rmsnorm(h, lay["ffn_norm"], self.eps)
            m = lay["moe"]
            logits = O.router_logits(xn, m["wr"])
            _, ids, w, _ = O.router_select(logits, m["K"], **m.get("router", {}))
            h = (h + O.moe_ffn(self.moe[l], xn, ids, w)).astype(f32)
        self.pos += T
        hn = rmsnorm(h[-1:], self.out_norm, self.eps)
        lg = O.matmul_q8_0(hn, self.head, 1, D, self.V)[0]
        return int(np.argmax(lg)), lg
