"""Expert-parallel execution of one MoE layer over the ranks of a torch.distributed group.

Rank r owns the experts [r*E/N, (r+1)*E/N) of every layer; the router is replicated; every
rank brings its own tokens.  Two exchanges:

* small batches (decode): all-gather activations and routes, run the local experts over all
  ranks' tokens with the ids of experts owned elsewhere mapped to -1 (the inactive-route rule of
  the single-GPU op, reference backends/ggml/mmid_route_skip.hpp:60-67), reduce-scatter the
  partial outputs.  Latency-bound: three small collectives, no host synchronisation.
* large batches (prefill): all-to-all.  A token row travels once to every rank that owns one of
  its experts, by per-destination counts; the rank's experts produce one pre-weighted,
  pre-reduced row per (token, rank); the rows travel back and are added in ascending rank
  order.  On GPUs this is the library's zmoe_ep_forward (device kernels + grouped
  ncclSend / ncclRecv); `exchange_forward_a2a` below is the same algorithm on torch
  collectives, used with CPU ranks (gloo) to test the exchange logic.

The reference has no collective anywhere (its multi-GPU support is placement plus
cudaMemcpyPeer, core/gpu_topology.cpp:1644); these exchanges are new.  Remote rows always
land in local memory through the collective before any kernel reads them.
"""
import ctypes as C

import torch
import torch.distributed as dist


def expert_range(rank, world, n_experts):
    return rank * n_experts // world, (rank + 1) * n_experts // world


def localise_ids(ids_all, e_lo, e_hi):
    """global expert ids -> ids inside this rank's shard, -1 for experts owned elsewhere"""
    owned = (ids_all >= e_lo) & (ids_all < e_hi)
    return torch.where(owned, ids_all - e_lo, torch.full_like(ids_all, -1))


def exchange_forward(x, ids, weights, e_lo, e_hi, compute, group=None, out=None, localise=True):
    """All-gather / reduce-scatter exchange.  x [T, D], ids [T, K] int32 (global), weights [T, K] -> out [T, D].

    compute(x_all [N*T, D], ids [N*T, K], w_all [N*T, K]) -> partial [N*T, D] sums the local experts'
    contributions for every token of every rank.  It is handed ids inside this rank's shard (-1 for experts
    owned elsewhere), or with localise=False the gathered global ids (a backend that maps them itself)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T = x.shape[0]
    x_all = torch.empty((world * T, x.shape[1]), dtype=x.dtype, device=x.device)
    ids_all = torch.empty((world * T, ids.shape[1]), dtype=ids.dtype, device=ids.device)
    w_all = torch.empty((world * T, weights.shape[1]), dtype=weights.dtype, device=weights.device)
    dist.all_gather_into_tensor(x_all, x.contiguous(), group=group)
    dist.all_gather_into_tensor(ids_all, ids.contiguous(), group=group)
    dist.all_gather_into_tensor(w_all, weights.contiguous(), group=group)
    partial = compute(x_all, localise_ids(ids_all, e_lo, e_hi) if localise else ids_all, w_all)
    if out is None:
        out = torch.empty_like(x)
    if dist.get_backend(group) == "gloo":       # gloo has no reduce-scatter: reduce, then take this rank's rows
        dist.all_reduce(partial, group=group)
        out.copy_(partial[rank * T:(rank + 1) * T])
    else:
        dist.reduce_scatter_tensor(out, partial, group=group)
    return out


def destination_plan(ids, n_experts, world):
    """Which ranks a token goes to and where: mask [T, N] bool (rank d owns one of the token's experts; ids
    outside [0, n_experts) are inactive routes), counts [N], and per destination the token indices in
    ascending order -- the same stable order the device kernels of the library produce."""
    per_rank = n_experts // world
    valid = (ids >= 0) & (ids < n_experts)
    owner = torch.where(valid, ids // per_rank, torch.zeros_like(ids)).long()
    mask = torch.zeros((ids.shape[0], world), dtype=torch.bool, device=ids.device)
    for k in range(ids.shape[1]):
        mask[valid[:, k], owner[valid[:, k], k]] = True
    tokens = [torch.nonzero(mask[:, d], as_tuple=False).flatten() for d in range(world)]
    counts = [int(t.numel()) for t in tokens]
    return mask, counts, tokens


def exchange_forward_a2a(x, ids, weights, n_experts, compute, group=None, out=None):
    """All-to-all exchange on torch collectives (the algorithm of zmoe_ep_forward).

    compute(x_recv [R, D], ids_recv [R, K] (global ids), w_recv [R, K]) -> [R, D]: the local experts'
    weighted sum for every received row (experts owned elsewhere contribute nothing)."""
    world = dist.get_world_size(group)
    T, D = x.shape
    K = ids.shape[1]
    mask, s_cnt, tokens = destination_plan(ids, n_experts, world)
    order = torch.cat(tokens) if sum(s_cnt) else torch.zeros(0, dtype=torch.long, device=x.device)
    sx, sids, sw = x[order].contiguous(), ids[order].contiguous(), weights[order].contiguous()
    cnt = torch.tensor(s_cnt, dtype=torch.int64, device=x.device)
    cnt_all = [torch.zeros_like(cnt) for _ in range(world)]
    dist.all_gather(cnt_all, cnt, group=group)
    rank = dist.get_rank(group)
    r_cnt = [int(c[rank]) for c in cnt_all]
    R = sum(r_cnt)
    rx = torch.empty((R, D), dtype=x.dtype, device=x.device)
    rids = torch.empty((R, K), dtype=ids.dtype, device=x.device)
    rw = torch.empty((R, K), dtype=weights.dtype, device=x.device)
    dist.all_to_all_single(rx, sx, r_cnt, s_cnt, group=group)
    dist.all_to_all_single(rids, sids, r_cnt, s_cnt, group=group)
    dist.all_to_all_single(rw, sw, r_cnt, s_cnt, group=group)
    ry = compute(rx, rids, rw) if R else torch.empty((0, D), dtype=x.dtype, device=x.device)
    yb = torch.empty((sum(s_cnt), D), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(yb, ry.contiguous(), s_cnt, r_cnt, group=group)
    if out is None:
        out = torch.empty_like(x)
    out.zero_()
    first = torch.ones(T, dtype=torch.bool, device=x.device)
    off = 0
    for d in range(world):                      # ascending rank order, the first contribution is copied, not added
        tk = tokens[d]
        rows = yb[off:off + s_cnt[d]]
        f = first[tk]
        out[tk[f]] = rows[f]
        out[tk[~f]] = out[tk[~f]] + rows[~f]
        first[tk] = False
        off += s_cnt[d]
    return out


class ExpertShard:
    """The CUDA backend: one rank's experts of a stack of layers.

    weights: list over layers of (w_gate, w_up, w_down, router_w); the expert tensors hold only this rank's
    experts, router_w all of them.  router: dict of the router's settings for lib.Layer (gating, weights_norm,
    weights_scale, n_groups, n_groups_used) plus optional "bias": list over layers of [E] tensors.  shared: list
    over layers of (w_gate, w_up, w_down) of the shared expert ([1, rows, row_bytes] each), or None.
    max_tokens: tokens a rank brings per call."""

    def __init__(self, ctx, rank, world, n_experts, topk, d_model, d_ff, types, weights, device, router=None,
                 shared=None, group=None, max_tokens=None):
        from . import lib
        self.lib = lib
        self.rank, self.world = rank, world
        self.E, self.K, self.D, self.F = n_experts, topk, d_model, d_ff
        self.e_lo, self.e_hi = expert_range(rank, world, n_experts)
        n_local = self.e_hi - self.e_lo
        self.ctx = ctx                                     # sized for the tokens a rank may process
        self.group = group
        self.max_tokens = max_tokens or max(1, ctx.max_tokens // world)
        router = dict(router or {})
        biases = router.pop("bias", None)
        # routing runs over all experts on a context of its own; its layer borrows the local
        # expert tensors only to satisfy the descriptor, it never runs the expert FFN
        self.route_ctx = lib.Context(max(self.max_tokens, 16), d_model, d_ff, n_experts, topk)
        self.routers, self.layers, self.shared = [], [], []
        self.shared_ctx = lib.Context(max(self.max_tokens, 16), d_model, d_ff, 1, 1) if shared else None
        for l, (wg, wu, wd, wr) in enumerate(weights):
            self.layers.append(lib.Layer(ctx, d_model, d_ff, n_local, topk, types, wg, wu, wd))
            self.routers.append(_router_only(lib, self.route_ctx, d_model, d_ff, n_experts, topk, types, wg, wu, wd, wr,
                                             biases[l] if biases else None, router))
            if shared:
                sg, su, sd = shared[l]
                self.shared.append(lib.Layer(self.shared_ctx, d_model, d_ff, 1, 1, types, sg, su, sd))
        self.device = device
        self._bufs = {}
        self._ep = None
        self._comm = None
        self.gemm_min = lib.load().zmoe_gemm_min_pairs_per_expert()

    # ---- small batches: all-gather / reduce-scatter -------------------------------------------------------
    def _buffers(self, T):
        if T not in self._bufs:
            dev, N = self.device, self.world
            self._bufs[T] = (torch.empty((2, T, self.K), dtype=torch.int32, device=dev),       # ids | weight bits
                             torch.empty((N, 2, T, self.K), dtype=torch.int32, device=dev),    # the same of all ranks
                             torch.empty((N * T, self.D), dtype=torch.float32, device=dev),    # x of all ranks
                             torch.empty((N * T, self.D), dtype=torch.float32, device=dev))    # partial sums
        return self._bufs[T]

    def forward_gather(self, l, x, out):
        """ids and weights travel in one all-gather, buffers are kept, the library maps model-wide ids into this
        rank's window (zmoe_set_routes_window) and the reduce-scatter writes the caller's rows."""
        T, N = x.shape[0], self.world
        routes, routes_all, x_all, partial = self._buffers(T)
        self.routers[l].route(x)
        self.route_ctx.copy_routes(routes[0], routes[1].view(torch.float32))
        dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(routes_all, routes, group=self.group)
        ids_all = routes_all[:, 0].reshape(N * T, self.K)                     # one small copy each
        w_all = routes_all[:, 1].reshape(N * T, self.K).view(torch.float32)
        # Only 1 / world of the gathered routes name a local expert, which the library cannot see from the
        # host: choose its kernels by the pairs per expert of the whole batch (the single-GPU rule)
        self.ctx.set_path(2 if N * T * self.K >= self.gemm_min * self.E else 1)
        self.layers[l].set_routes_window(x_all, ids_all, w_all, self.e_lo)
        self.layers[l].expert_ffn(partial)
        self.ctx.set_path(0)
        if out.is_contiguous():
            dist.reduce_scatter_tensor(out, partial, group=self.group)
        else:
            own = torch.empty_like(x)
            dist.reduce_scatter_tensor(own, partial, group=self.group)
            out.copy_(own)
        if self.shared:
            self.shared[l].dense_ffn(x, out, accumulate=1)

    # ---- large batches: all-to-all through the library ---------------------------------------------------
    def _ensure_ep(self):
        if self._ep is not None:
            return
        L = self.lib.load()
        ident = torch.zeros(128, dtype=torch.uint8, device=self.device)
        if self.rank == 0:
            buf = (C.c_ubyte * 128)()
            self.lib.check(L.zmoe_ep_unique_id(buf), "zmoe_ep_unique_id")
            ident.copy_(torch.tensor(list(buf), dtype=torch.uint8))
        dist.broadcast(ident, src=0 if self.group is None else dist.get_global_rank(self.group, 0), group=self.group)
        raw = (C.c_ubyte * 128)(*ident.cpu().tolist())
        comm = C.c_void_p()
        self.lib.check(L.zmoe_ep_comm_init(raw, self.rank, self.world, C.byref(comm)), "zmoe_ep_comm_init")
        self._comm = comm
        ep = C.c_void_p()
        self.lib.check(L.zmoe_ep_create(comm, self.rank, self.world, self.max_tokens, self.ctx.max_tokens, self.D, self.K,
                                        C.byref(ep)), "zmoe_ep_create")
        self._ep = ep

    def forward_a2a(self, l, x, out):
        self._ensure_ep()
        L = self.lib.load()
        sh = self.shared[l].h if self.shared else None
        self.lib.check(L.zmoe_ep_forward(self._ep, self.routers[l].h, self.layers[l].h, sh, self.lib.ptr(x),
                                         self.lib.ptr(out), x.shape[0], self.lib._stream_ptr()), "zmoe_ep_forward")

    def last_rows(self):
        """(rows sent, rows received) by this rank in its last all-to-all"""
        s, r = C.c_int64(), C.c_int64()
        self.lib.check(self.lib.load().zmoe_ep_last_rows(self._ep, C.byref(s), C.byref(r)), "zmoe_ep_last_rows")
        return s.value, r.value

    def forward(self, l, x, out, mode=None):
        """mode: "gather", "a2a" or None = by size: the all-to-all from the batch at which experts hold enough pairs
        for the tensor-core path (its host synchronisation is then a small part of the layer)"""
        if mode is None:
            mode = "a2a" if self.world * x.shape[0] * self.K >= self.gemm_min * self.E else "gather"
        if mode == "a2a":
            self.forward_a2a(l, x, out)
        else:
            self.forward_gather(l, x, out)

    def close(self):
        L = self.lib.load()
        if self._ep is not None:
            L.zmoe_ep_destroy(self._ep)
            self._ep = None
        if self._comm is not None:
            L.zmoe_ep_comm_destroy(self._comm)
            self._comm = None


def _router_only(lib, ctx, d_model, d_ff, n_experts, topk, types, wg, wu, wd, wr, bias=None, spec=None):
    """a layer object used for zmoe_route only: all experts in the router, expert tensors unused"""
    spec = spec or {}
    layer = lib.Layer.__new__(lib.Layer)
    layer.ctx = ctx
    layer.keep = (wg, wu, wd, wr, bias)
    layer.d_model, layer.d_ff, layer.n_experts, layer.topk = d_model, d_ff, n_experts, topk
    d = lib.LayerDesc()
    d.d_model, d.d_ff, d.n_experts, d.topk = d_model, d_ff, n_experts, topk
    for wt, t, ty in ((d.gate, wg, types[0]), (d.up, wu, types[1]), (d.down, wd, types[2])):
        wt.data_dev = t.data_ptr()
        wt.expert_stride = t.stride(0) * t.element_size()
        wt.bytes = t.numel() * t.element_size()          # what is really addressable
        wt.type = ty
    d.router_w_dev = wr.data_ptr()
    d.router_bias_dev = bias.data_ptr() if bias is not None else None
    d.gating = spec.get("gating", 0)
    d.weights_norm = spec.get("weights_norm", 1)
    d.weights_scale = spec.get("weights_scale", 0.0)
    d.n_groups, d.n_groups_used = spec.get("n_groups", 0), spec.get("n_groups_used", 0)
    d.swiglu_clamp, d.swiglu_clamp_fused = 0.0, 0
    layer.desc = d
    layer.h = C.c_void_p()
    lib.check(lib.load().zmoe_layer_create(ctx.h, C.byref(d), C.byref(layer.h)), "zmoe_layer_create")
    return layer
