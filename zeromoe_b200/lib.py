"""ctypes binding of libzmoe_b200.so.  Device memory and streams come from
torch; every compute call goes through the C ABI."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libzmoe_b200.so")

Q2_K, Q3_K, Q4_K, IQ2_XXS = 10, 11, 12, 16
BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, IQ2_XXS: 66}
GGML_F32, GGML_I32 = 0, 26

ERRORS = {0: "OK", -1: "ARG", -2: "TYPE", -3: "SHAPE", -4: "ALIGN", -5: "CUDA", -6: "CAPACITY",
          -7: "DEVICE_WAIT", -8: "STATE", -9: "COMM"}

# every symbol include/zmoe_b200.h declares
EXPORTS = [
    "launch_q2_K_matmul", "launch_q2_K_matmul_stream", "launch_q3_K_matmul", "launch_q3_K_matmul_stream",
    "launch_q4_K_matmul", "launch_iq2_xxs_matmul", "launch_expert_swiglu", "launch_expert_scatter_accum",
    "launch_expert_scatter_add", "launch_glm5next_router_topk", "zmoe_matmul_noalloc", "zmoe_reserve", "zmoe_last_status",
    "zmoe_f32_quant_hook", "zeromoe_install_f32_quant_graph_hook", "zeromoe_f32_quant_graph_launches",
    "zmoe_ctx_create", "zmoe_ctx_destroy", "zmoe_layer_create", "zmoe_layer_destroy", "zmoe_route",
    "zmoe_set_routes", "zmoe_set_routes_strided", "zmoe_set_routes_window", "zmoe_expert_ffn", "zmoe_expert_ffn_events", "zmoe_dense_ffn", "zmoe_dense_ffn_gated", "zmoe_moe_forward", "zmoe_moe_forward_bf16", "zmoe_moe_forward_host", "zmoe_get_routes",
    "zmoe_get_expert_freq", "zmoe_copy_routes", "zmoe_get_probs", "zmoe_get_act", "zmoe_ctx_set_path", "zmoe_ctx_check", "zmoe_kernel_launches",
    "zmoe_quantize_q8_K", "zmoe_block_isums", "zmoe_block_isums_pairs",
    "zmoe_device_status", "zmoe_selftest_wait_expiry", "zmoe_ctx_bad_counts", "zmoe_gemm_min_pairs_per_expert",
    "zmoe_debug_gemm_cycles",
    "zmoe_ep_unique_id", "zmoe_ep_comm_init", "zmoe_ep_comm_destroy", "zmoe_ep_create", "zmoe_ep_destroy",
    "zmoe_ep_forward", "zmoe_ep_forward_routed", "zmoe_ep_last_rows",
    "launch_q8_0_matmul", "launch_q8_0_matmul_stream", "launch_rmsnorm",
    "zmoe_decoder_create", "zmoe_decoder_destroy", "zmoe_decoder_reset", "zmoe_decoder_step", "zmoe_decoder_read",
    "launch_ggml_moe_unpack", "launch_ggml_moe_unpack_scatter", "zmoe_moe_pack", "zmoe_gguf_open", "zmoe_gguf_close",
    "zmoe_gguf_tensor_count", "zmoe_gguf_find", "zmoe_gguf_read", "zmoe_gguf_load_experts",
]


class ZmoeError(RuntimeError):
    def __init__(self, code, where):
        super().__init__("%s failed: ZMOE_ERR_%s (%d)" % (where, ERRORS.get(code, "?"), code))
        self.code = code


class Weight(C.Structure):
    _fields_ = [("data_dev", C.c_void_p), ("expert_stride", C.c_size_t), ("bytes", C.c_size_t), ("type", C.c_int)]


class LayerDesc(C.Structure):
    _fields_ = [("d_model", C.c_int), ("d_ff", C.c_int), ("n_experts", C.c_int), ("topk", C.c_int),
                ("gate", Weight), ("up", Weight), ("down", Weight),
                ("router_w_dev", C.c_void_p), ("router_bias_dev", C.c_void_p),
                ("gating", C.c_int), ("weights_norm", C.c_int), ("weights_scale", C.c_float),
                ("n_groups", C.c_int), ("n_groups_used", C.c_int),
                ("swiglu_clamp", C.c_float), ("swiglu_clamp_fused", C.c_int)]


class DecoderDesc(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("d_model", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("vocab", C.c_int), ("max_ctx", C.c_int), ("max_tokens", C.c_int),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("attn_norm_w", C.POINTER(C.c_void_p)), ("wqkv", C.POINTER(C.c_void_p)), ("wo", C.POINTER(C.c_void_p)),
                ("ffn_norm_w", C.POINTER(C.c_void_p)), ("moe", C.POINTER(C.c_void_p)),
                ("tok_embd", C.c_void_p), ("out_norm_w", C.c_void_p), ("lm_head", C.c_void_p)]


class GgufTensor(C.Structure):
    _fields_ = [("type", C.c_int), ("n_dims", C.c_int), ("ne", C.c_int64 * 4), ("file_offset", C.c_uint64),
                ("bytes", C.c_uint64)]


class Tensor(C.Structure):
    _fields_ = [("type", C.c_int), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("data", C.c_void_p)]


_lib = None


def load():
    """Load the shared library; raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("libzmoe_b200.so is not built (run `python -m zeromoe_b200.build`); "
                          "there is no fallback path")
    L = C.CDLL(LIB_PATH)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    for name in ("launch_q2_K_matmul", "launch_q3_K_matmul", "launch_q4_K_matmul", "launch_iq2_xxs_matmul"):
        getattr(L, name).argtypes = [vp, vp, vp, i, i, i]
        getattr(L, name).restype = None
    for name in ("launch_q2_K_matmul_stream", "launch_q3_K_matmul_stream"):
        getattr(L, name).argtypes = [vp, vp, vp, i, i, i, vp]
        getattr(L, name).restype = None
    L.launch_expert_swiglu.argtypes = [vp, vp, vp, i, f, i, vp, vp]
    L.launch_expert_swiglu.restype = None
    L.launch_expert_scatter_accum.argtypes = [vp, vp, vp, vp, i, i, i, vp]
    L.launch_expert_scatter_accum.restype = None
    L.launch_expert_scatter_add.argtypes = [vp, vp, vp, i, i, i, vp]
    L.launch_expert_scatter_add.restype = None
    L.launch_glm5next_router_topk.argtypes = [vp, vp, vp, vp, i, i, i, i, i, f, vp]
    L.launch_glm5next_router_topk.restype = None
    L.zmoe_matmul_noalloc.argtypes = [i, vp, vp, vp, i, i, i, vp]
    L.zmoe_reserve.argtypes = [i, i]
    L.zmoe_f32_quant_hook.argtypes = [C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor),
                                      vp, C.c_bool]
    L.zmoe_f32_quant_hook.restype = C.c_bool
    L.zeromoe_install_f32_quant_graph_hook.restype = C.c_bool
    L.zeromoe_f32_quant_graph_launches.restype = C.c_uint64
    L.zmoe_kernel_launches.restype = C.c_uint64
    L.zmoe_ctx_create.argtypes = [i, i, i, i, i, C.POINTER(vp)]
    L.zmoe_ctx_destroy.argtypes = [vp]
    L.zmoe_ctx_destroy.restype = None
    L.zmoe_layer_create.argtypes = [vp, C.POINTER(LayerDesc), C.POINTER(vp)]
    L.zmoe_layer_destroy.argtypes = [vp]
    L.zmoe_layer_destroy.restype = None
    L.zmoe_route.argtypes = [vp, vp, i, vp]
    L.zmoe_set_routes.argtypes = [vp, vp, vp, vp, i, vp]
    L.zmoe_set_routes_window.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.zmoe_block_isums_pairs.argtypes = [i, vp, vp, vp, i, i, vp]
    L.zmoe_set_routes_strided.argtypes = [vp, vp, vp, C.c_size_t, vp, C.c_size_t, i, vp]
    L.zmoe_expert_ffn.argtypes = [vp, vp, i, i, vp]
    L.zmoe_expert_ffn_events.argtypes = [vp, vp, i, i, vp, vp, vp]
    L.zmoe_dense_ffn.argtypes = [vp, vp, vp, i, i, vp]
    L.zmoe_dense_ffn_gated.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.zmoe_moe_forward_bf16.argtypes = [vp, vp, vp, i, vp]
    L.zmoe_moe_forward.argtypes = [vp, vp, vp, i, vp]
    L.zmoe_moe_forward_host.argtypes = [vp, vp, vp, i]
    L.zmoe_get_routes.argtypes = [vp, i, i, vp, vp]
    L.zmoe_get_expert_freq.argtypes = [vp, i, vp]
    L.zmoe_copy_routes.argtypes = [vp, i, i, vp, vp, vp]
    L.zmoe_get_probs.argtypes = [vp, i, i, vp]
    L.zmoe_get_act.argtypes = [vp, i, i, vp]
    L.zmoe_ctx_check.argtypes = [vp]
    L.zmoe_ctx_set_path.argtypes = [vp, i]
    L.zmoe_quantize_q8_K.argtypes = [vp, vp, i, i, i, vp]
    L.zmoe_block_isums.argtypes = [i, vp, vp, vp, vp, i, i, vp]
    L.zmoe_selftest_wait_expiry.argtypes = [vp]
    L.zmoe_ctx_bad_counts.argtypes = [vp, vp, i]
    L.zmoe_debug_gemm_cycles.argtypes = [vp]
    L.zmoe_ep_unique_id.argtypes = [vp]
    L.zmoe_ep_comm_init.argtypes = [vp, i, i, C.POINTER(vp)]
    L.zmoe_ep_comm_destroy.argtypes = [vp]
    L.zmoe_ep_create.argtypes = [vp, i, i, i, i, i, i, C.POINTER(vp)]
    L.zmoe_ep_destroy.argtypes = [vp]
    L.zmoe_ep_destroy.restype = None
    L.zmoe_ep_forward.argtypes = [vp, vp, vp, vp, vp, vp, i, vp]
    L.zmoe_ep_forward_routed.argtypes = [vp, vp, vp, i, vp, vp, vp, vp, i, vp]
    L.zmoe_ep_last_rows.argtypes = [vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    L.launch_q8_0_matmul.argtypes = [vp, vp, vp, i, i, i]
    L.launch_q8_0_matmul.restype = None
    L.launch_q8_0_matmul_stream.argtypes = [vp, vp, vp, i, i, i, vp]
    L.launch_q8_0_matmul_stream.restype = None
    L.launch_rmsnorm.argtypes = [vp, vp, vp, i, i, f]
    L.launch_rmsnorm.restype = None
    L.zmoe_decoder_create.argtypes = [C.POINTER(DecoderDesc), C.POINTER(vp)]
    L.zmoe_decoder_destroy.argtypes = [vp]
    L.zmoe_decoder_destroy.restype = None
    L.zmoe_decoder_reset.argtypes = [vp, vp]
    L.zmoe_decoder_step.argtypes = [vp, vp, i, vp]
    L.zmoe_decoder_read.argtypes = [vp, vp, vp, vp, i]
    sz = C.c_size_t
    L.launch_ggml_moe_unpack.argtypes = [vp, vp, vp, vp, i, sz, sz, sz, sz, sz, sz, sz, vp]
    L.launch_ggml_moe_unpack_scatter.argtypes = [vp, vp, vp, vp, vp, i, sz, sz, sz, sz, sz, sz, sz, vp]
    L.zmoe_moe_pack.argtypes = [vp, vp, vp, vp, i, sz, sz, sz, sz, sz, sz, sz, vp]
    L.zmoe_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.zmoe_gguf_close.argtypes = [vp]
    L.zmoe_gguf_close.restype = None
    L.zmoe_gguf_tensor_count.argtypes = [vp]
    L.zmoe_gguf_find.argtypes = [vp, C.c_char_p, C.POINTER(GgufTensor)]
    L.zmoe_gguf_read.argtypes = [vp, C.POINTER(GgufTensor), vp, C.c_uint64, C.c_uint64]
    L.zmoe_gguf_load_experts.argtypes = [vp, i, vp, vp, vp, C.POINTER(GgufTensor), vp]
    _lib = L
    return L


def check(rc, where):
    if rc != 0:
        raise ZmoeError(rc, where)


def _stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class Context:
    """Per-device scratch (zmoe_ctx)."""

    def __init__(self, max_tokens, max_d_model, max_d_ff, max_experts, max_topk):
        self.h = C.c_void_p()
        check(load().zmoe_ctx_create(max_tokens, max_d_model, max_d_ff, max_experts, max_topk, C.byref(self.h)),
              "zmoe_ctx_create")
        self.max_tokens = max_tokens

    def check(self):
        check(load().zmoe_ctx_check(self.h), "zmoe_ctx_check")

    def set_path(self, path):
        """0 auto, 1 decode kernels, 2 tensor-core GEMM, 3 decode kernels one pair at a time"""
        check(load().zmoe_ctx_set_path(self.h, path), "zmoe_ctx_set_path")

    def routes(self, T, K):
        ids = np.zeros((T, K), dtype=np.int32)
        w = np.zeros((T, K), dtype=np.float32)
        check(load().zmoe_get_routes(self.h, T, K, ids.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p)),
              "zmoe_get_routes")
        return ids, w

    def copy_routes(self, ids_dev, weights_dev, stream=None):
        T, K = ids_dev.shape
        check(load().zmoe_copy_routes(self.h, T, K, ptr(ids_dev), ptr(weights_dev), _stream_ptr(stream)),
              "zmoe_copy_routes")

    def expert_freq(self, E):
        f = np.zeros(E, dtype=np.int32)
        check(load().zmoe_get_expert_freq(self.h, E, f.ctypes.data_as(C.c_void_p)), "zmoe_get_expert_freq")
        return f

    def bad_counts(self, clear=True):
        """(pairs with a NaN, pairs with an infinity) seen by the fused SwiGLU epilogues"""
        c = np.zeros(2, dtype=np.int32)
        check(load().zmoe_ctx_bad_counts(self.h, c.ctypes.data_as(C.c_void_p), 1 if clear else 0),
              "zmoe_ctx_bad_counts")
        return int(c[0]), int(c[1])

    def probs(self, T, E):
        p = np.zeros((T, E), dtype=np.float32)
        check(load().zmoe_get_probs(self.h, T, E, p.ctypes.data_as(C.c_void_p)), "zmoe_get_probs")
        return p

    def act(self, P, F):
        a = np.zeros((P, F), dtype=np.float32)
        check(load().zmoe_get_act(self.h, P, F, a.ctypes.data_as(C.c_void_p)), "zmoe_get_act")
        return a

    def close(self):
        if self.h:
            load().zmoe_ctx_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Layer:
    """One MoE layer over borrowed device weights (torch uint8 tensors [E, rows, row_bytes])."""

    def __init__(self, ctx, d_model, d_ff, n_experts, topk, types, w_gate, w_up, w_down, router_w=None,
                 router_bias=None, gating=0, weights_norm=1, weights_scale=0.0, n_groups=0, n_groups_used=0,
                 clamp=0.0, clamp_fused=0):
        self.ctx = ctx
        self.keep = (w_gate, w_up, w_down, router_w, router_bias)
        self.d_model, self.d_ff, self.n_experts, self.topk = d_model, d_ff, n_experts, topk
        d = LayerDesc()
        d.d_model, d.d_ff, d.n_experts, d.topk = d_model, d_ff, n_experts, topk
        for wt, t, ty in ((d.gate, w_gate, types[0]), (d.up, w_up, types[1]), (d.down, w_down, types[2])):
            wt.data_dev = t.data_ptr()
            wt.expert_stride = t.stride(0) * t.element_size()
            wt.bytes = 0
            wt.type = ty
        d.router_w_dev = router_w.data_ptr() if router_w is not None else None
        d.router_bias_dev = router_bias.data_ptr() if router_bias is not None else None
        d.gating, d.weights_norm, d.weights_scale = gating, weights_norm, weights_scale
        d.n_groups, d.n_groups_used = n_groups, n_groups_used
        d.swiglu_clamp, d.swiglu_clamp_fused = clamp, clamp_fused
        self.desc = d
        self.h = C.c_void_p()
        check(load().zmoe_layer_create(ctx.h, C.byref(d), C.byref(self.h)), "zmoe_layer_create")

    def route(self, x, stream=None):
        check(load().zmoe_route(self.h, ptr(x), x.shape[0], _stream_ptr(stream)), "zmoe_route")

    def set_routes(self, x, ids, weights, stream=None):
        check(load().zmoe_set_routes(self.h, ptr(x), ptr(ids), ptr(weights), x.shape[0], _stream_ptr(stream)),
              "zmoe_set_routes")

    def set_routes_window(self, x, ids, weights, first_expert, stream=None):
        """ids number the experts of a larger model; this layer holds [first_expert, first_expert + n_experts)"""
        check(load().zmoe_set_routes_window(self.h, ptr(x), ptr(ids), ptr(weights), x.shape[0], first_expert,
                                            _stream_ptr(stream)), "zmoe_set_routes_window")

    def expert_ffn(self, out, accumulate=0, stream=None):
        check(load().zmoe_expert_ffn(self.h, ptr(out), out.shape[0], accumulate, _stream_ptr(stream)),
              "zmoe_expert_ffn")

    def expert_ffn_timed(self, out, ev0, ev1, stream=None):
        """expert_ffn with two torch.cuda.Event recorded around the gate/up matmul"""
        for ev in (ev0, ev1):
            if not ev.cuda_event:      # torch creates the handle on first record
                ev.record()
        check(load().zmoe_expert_ffn_events(self.h, ptr(out), out.shape[0], 0, _stream_ptr(stream),
                                            C.c_void_p(ev0.cuda_event), C.c_void_p(ev1.cuda_event)),
              "zmoe_expert_ffn_events")

    def dense_ffn(self, x, out, accumulate=0, stream=None):
        """single-expert layer applied to every token (shared expert)"""
        check(load().zmoe_dense_ffn(self.h, ptr(x), ptr(out), x.shape[0], accumulate, _stream_ptr(stream)),
              "zmoe_dense_ffn")

    def dense_ffn_gated(self, x, gate_w, out, accumulate=0, stream=None):
        """dense_ffn with every token's row scaled by sigmoid(gate_w . x[t])"""
        check(load().zmoe_dense_ffn_gated(self.h, ptr(x), ptr(gate_w), ptr(out), x.shape[0], accumulate, _stream_ptr(stream)),
              "zmoe_dense_ffn_gated")

    def forward(self, x, out, stream=None):
        check(load().zmoe_moe_forward(self.h, ptr(x), ptr(out), x.shape[0], _stream_ptr(stream)), "zmoe_moe_forward")

    def forward_bf16(self, x_bf16, out, stream=None):
        """forward for a torch.bfloat16 activation tensor [T, d_model]"""
        check(load().zmoe_moe_forward_bf16(self.h, ptr(x_bf16), ptr(out), x_bf16.shape[0], _stream_ptr(stream)),
              "zmoe_moe_forward_bf16")

    def forward_host(self, x_host, out_host):
        """x_host / out_host: host tensors or arrays [T, d_model] f32 (pinned for full speed)"""
        T = x_host.shape[0]
        xp = x_host.data_ptr() if hasattr(x_host, "data_ptr") else x_host.ctypes.data
        op = out_host.data_ptr() if hasattr(out_host, "data_ptr") else out_host.ctypes.data
        check(load().zmoe_moe_forward_host(self.h, C.c_void_p(xp), C.c_void_p(op), T), "zmoe_moe_forward_host")

    def close(self):
        if self.h:
            load().zmoe_layer_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Decoder:
    """A decoder over borrowed device tensors (zmoe_decoder).  layers: list of dicts with attn_norm [D] f32, wqkv
    and wo (uint8 Q8_0 rows), ffn_norm [D] f32 and moe (a Layer on a context of >= max_tokens tokens)."""

    def __init__(self, layers, tok_embd, out_norm, lm_head, d_model, n_heads, n_kv_heads, head_dim, vocab, max_ctx,
                 max_tokens, rms_eps=1e-6, rope_theta=10000.0):
        self.keep = (layers, tok_embd, out_norm, lm_head)
        n = len(layers)
        arr = lambda key: (C.c_void_p * n)(*[l[key].data_ptr() for l in layers])
        self._arrays = [arr("attn_norm"), arr("wqkv"), arr("wo"), arr("ffn_norm"),
                        (C.c_void_p * n)(*[l["moe"].h.value for l in layers])]
        d = DecoderDesc()
        d.n_layers, d.d_model, d.n_heads, d.n_kv_heads, d.head_dim = n, d_model, n_heads, n_kv_heads, head_dim
        d.vocab, d.max_ctx, d.max_tokens = vocab, max_ctx, max_tokens
        d.rms_eps, d.rope_theta = rms_eps, rope_theta
        d.attn_norm_w, d.wqkv, d.wo, d.ffn_norm_w, d.moe = [C.cast(a, C.POINTER(C.c_void_p)) for a in self._arrays]
        d.tok_embd, d.out_norm_w, d.lm_head = tok_embd.data_ptr(), out_norm.data_ptr(), lm_head.data_ptr()
        self.desc = d
        self.vocab = vocab
        self.h = C.c_void_p()
        check(load().zmoe_decoder_create(C.byref(d), C.byref(self.h)), "zmoe_decoder_create")

    def reset(self, stream=None):
        check(load().zmoe_decoder_reset(self.h, _stream_ptr(stream)), "zmoe_decoder_reset")

    def step(self, tokens=None, stream=None):
        """tokens: int32 device tensor [T], or None = continue with the token the last step sampled"""
        T = 1 if tokens is None else tokens.shape[0]
        check(load().zmoe_decoder_step(self.h, ptr(tokens), T, _stream_ptr(stream)), "zmoe_decoder_step")

    def read(self, n_logits=0):
        """(next token, position, logits[:n_logits]) after a synchronisation"""
        import torch
        torch.cuda.synchronize()
        tok, pos = C.c_int32(), C.c_int32()
        lg = np.zeros(max(n_logits, 1), dtype=np.float32)
        check(load().zmoe_decoder_read(self.h, C.byref(tok), C.byref(pos), lg.ctypes.data_as(C.c_void_p), n_logits),
              "zmoe_decoder_read")
        return tok.value, pos.value, lg[:n_logits]

    def close(self):
        if self.h:
            load().zmoe_decoder_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def q8_0_matmul(x, w, O, stream=None):
    """y[S, O] = x[S, I] . W^T, W uint8 rows of Q8_0 blocks (launch_q8_0_matmul_stream)"""
    import torch
    S, I = x.shape
    y = torch.empty((S, O), dtype=torch.float32, device=x.device)
    L = load()
    L.launch_q8_0_matmul_stream(ptr(y), ptr(x), ptr(w), S, I, O, _stream_ptr(stream))
    check(L.zmoe_last_status(), "launch_q8_0_matmul_stream")
    return y


def dense_matmul(qtype, x, w, O, stream=None):
    """y[S,O] = x[S,I] . W^T through the reference's launch_*_matmul symbols (torch tensors on the device)"""
    import torch
    S, I = x.shape
    y = torch.empty((S, O), dtype=torch.float32, device=x.device)
    L = load()
    if qtype == Q2_K:
        L.launch_q2_K_matmul_stream(ptr(y), ptr(x), ptr(w), S, I, O, _stream_ptr(stream))
    elif qtype == Q3_K:
        L.launch_q3_K_matmul_stream(ptr(y), ptr(x), ptr(w), S, I, O, _stream_ptr(stream))
    else:
        # these two symbols have no stream variant in the reference: legacy default stream
        torch.cuda.current_stream().synchronize()
        (L.launch_q4_K_matmul if qtype == Q4_K else L.launch_iq2_xxs_matmul)(ptr(y), ptr(x), ptr(w), S, I, O)
        torch.cuda.synchronize()
    check(L.zmoe_last_status(), "launch_*_matmul")
    return y


def make_tensor(t, qtype, ne, nb):
    T = Tensor()
    T.type = qtype
    for k in range(4):
        T.ne[k] = ne[k]
        T.nb[k] = nb[k]
    T.data = t.data_ptr()
    return T
