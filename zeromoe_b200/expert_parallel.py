"""Expert-parallel execution of one MoE layer over the ranks of a torch.distributed group.

Rank r owns the experts [r*E/N, (r+1)*E/N) of every layer; the router is replicated; every
rank brings its own tokens.  Per layer: route locally, all-gather activations and routes,
run the local experts over all ranks' tokens with the ids of experts owned elsewhere mapped
to -1 (the inactive-route rule of the single-GPU op, reference
backends/ggml/mmid_route_skip.hpp:60-67), reduce-scatter the partial outputs.

The reference has no collective anywhere (its multi-GPU support is placement plus
cudaMemcpyPeer, core/gpu_topology.cpp:1644); this exchange is new.  Remote rows always
land in local memory through the collective before any kernel reads them.

The exchange logic is independent of the compute backend so it can be tested on CPU ranks
(gloo) with the CPU oracle standing in for the CUDA library.
"""
import torch
import torch.distributed as dist


def expert_range(rank, world, n_experts):
    return rank * n_experts // world, (rank + 1) * n_experts // world


def localise_ids(ids_all, e_lo, e_hi):
    """global expert ids -> ids inside this rank's shard, -1 for experts owned elsewhere"""
    owned = (ids_all >= e_lo) & (ids_all < e_hi)
    return torch.where(owned, ids_all - e_lo, torch.full_like(ids_all, -1))


def exchange_forward(x, ids, weights, e_lo, e_hi, compute, group=None, out=None, localise=True):
    """x [T, D], ids [T, K] int32 (global), weights [T, K] -> out [T, D].

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


class ExpertShard:
    """The CUDA backend: one rank's experts of a stack of layers.

    weights: list over layers of (w_gate, w_up, w_down, router_w); the expert tensors hold only
    this rank's experts, router_w all of them."""

    def __init__(self, ctx, rank, world, n_experts, topk, d_model, d_ff, types, weights, device):
        from . import lib
        self.lib = lib
        self.rank, self.world = rank, world
        self.E, self.K, self.D, self.F = n_experts, topk, d_model, d_ff
        self.e_lo, self.e_hi = expert_range(rank, world, n_experts)
        n_local = self.e_hi - self.e_lo
        self.ctx = ctx                                     # sized for world * T tokens
        # routing runs over all experts on a context of its own; its layer borrows the local
        # expert tensors only to satisfy the descriptor, it never runs the expert FFN
        self.route_ctx = lib.Context(ctx.max_tokens, d_model, d_ff, n_experts, topk)
        self.routers, self.layers = [], []
        for wg, wu, wd, wr in weights:
            self.layers.append(lib.Layer(ctx, d_model, d_ff, n_local, topk, types, wg, wu, wd))
            self.routers.append(_router_only(lib, self.route_ctx, d_model, d_ff, n_experts, topk, types, wg, wu, wd, wr))
        self.device = device
        self._bufs = {}

    def _buffers(self, T):
        if T not in self._bufs:
            dev, N = self.device, self.world
            self._bufs[T] = (torch.empty((2, T, self.K), dtype=torch.int32, device=dev),       # ids | weight bits
                             torch.empty((N, 2, T, self.K), dtype=torch.int32, device=dev),    # the same of all ranks
                             torch.empty((N * T, self.D), dtype=torch.float32, device=dev),    # x of all ranks
                             torch.empty((N * T, self.D), dtype=torch.float32, device=dev))    # partial sums
        return self._bufs[T]

    def forward(self, l, x, out):
        """Same exchange as exchange_forward, with fewer launches: ids and weights travel in one all-gather,
        buffers are kept, the library maps model-wide ids into this rank's window
        (zmoe_set_routes_window) and the reduce-scatter writes the caller's rows."""
        T, N = x.shape[0], self.world
        routes, routes_all, x_all, partial = self._buffers(T)
        self.routers[l].route(x)
        self.route_ctx.copy_routes(routes[0], routes[1].view(torch.float32))
        dist.all_gather_into_tensor(x_all, x.contiguous())
        dist.all_gather_into_tensor(routes_all, routes)
        ids_all = routes_all[:, 0].reshape(N * T, self.K)                     # one small copy each
        w_all = routes_all[:, 1].reshape(N * T, self.K).view(torch.float32)
        # Only 1 / world of the gathered routes name a local expert, which the library cannot see from the
        # host: choose its kernels by the pairs per expert of the whole batch (the single-GPU rule)
        self.ctx.set_path(2 if N * T * self.K >= 24 * self.E else 1)
        self.layers[l].set_routes_window(x_all, ids_all, w_all, self.e_lo)
        self.layers[l].expert_ffn(partial)
        if out.is_contiguous():
            dist.reduce_scatter_tensor(out, partial)
        else:
            own = torch.empty_like(x)
            dist.reduce_scatter_tensor(own, partial)
            out.copy_(own)


def _router_only(lib, ctx, d_model, d_ff, n_experts, topk, types, wg, wu, wd, wr):
    """a layer object used for zmoe_route only: all experts in the router, expert tensors unused"""
    import ctypes as C
    layer = lib.Layer.__new__(lib.Layer)
    layer.ctx = ctx
    layer.keep = (wg, wu, wd, wr)
    layer.d_model, layer.d_ff, layer.n_experts, layer.topk = d_model, d_ff, n_experts, topk
    d = lib.LayerDesc()
    d.d_model, d.d_ff, d.n_experts, d.topk = d_model, d_ff, n_experts, topk
    for wt, t, ty in ((d.gate, wg, types[0]), (d.up, wu, types[1]), (d.down, wd, types[2])):
        wt.data_dev = t.data_ptr()
        wt.expert_stride = t.stride(0) * t.element_size()
        wt.bytes = t.numel() * t.element_size()          # what is really addressable
        wt.type = ty
    d.router_w_dev = wr.data_ptr()
    d.router_bias_dev = None
    d.gating, d.weights_norm, d.weights_scale = 0, 1, 0.0
    d.n_groups, d.n_groups_used = 0, 0
    d.swiglu_clamp, d.swiglu_clamp_fused = 0.0, 0
    layer.desc = d
    layer.h = C.c_void_p()
    lib.check(lib.load().zmoe_layer_create(ctx.h, C.byref(d), C.byref(layer.h)), "zmoe_layer_create")
    return layer
