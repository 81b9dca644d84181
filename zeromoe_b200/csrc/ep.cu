// ep.cu -- expert parallelism over the GPUs of one node: all-to-all token dispatch and combine.
//
// The reference has no collective anywhere (its multi-GPU support is placement plus
// cudaMemcpyPeer, reference core/gpu_topology.cpp:1644); this exchange is new.  What it keeps of
// the reference is the ownership convention of its hot / cold expert split: every rank sees the
// model-wide expert numbers of a token's routes and maps the experts it does not hold to -1
// (reference backends/ggml/moe_partial_route_ggml.hpp:13-35, backends/ggml/mmid_route_skip.hpp:60-67),
// so the per-rank operator is the single-GPU layer unchanged, and the ranks' partial outputs are
// summed (combine_hot_cold, reference backends/ggml/moe_partial_route_ggml.hpp:40-58).
//
// Rank r holds the experts [r * E / N, (r + 1) * E / N).  Per layer, for the T tokens a rank brings:
//   1. route (replicated router over all E experts);
//   2. destinations: token t goes ONCE to every rank that owns at least one of its experts, with all K
//      route ids and weights (device kernels: destination masks, stable positions, send offsets);
//   3. the per-destination counts are all-gathered and read by the host (one stream synchronisation
//      per layer: NCCL needs the sizes), rows are packed by destination and exchanged with grouped
//      ncclSend / ncclRecv;
//   4. the rank runs its experts over the rows it received (routes of experts held elsewhere are
//      inactive and contribute zero rows), which gives ONE pre-weighted, pre-reduced row per
//      (token, destination rank);
//   5. those rows travel back the same way and the home rank adds them in ascending rank order, then
//      adds the shared expert where the model has one.
// Remote rows always land in this GPU's own memory through NCCL before a kernel reads them.
// NCCL is looked up with dlopen at first use, so the library loads (and every other entry point works)
// on machines without it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "zmoe_common.cuh"
#include "zmoe_internal.h"

using namespace zmoe;

namespace {

// ---------------------------------------------------------------------------
// NCCL entry points, resolved at run time
// ---------------------------------------------------------------------------
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    bool ok = false;
};

const NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // a copy the process already holds (the one a framework brought along) comes first
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        auto sym = [&](const char *n) { return dlsym(h, n); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Send && api.Recv &&
                 api.GroupStart && api.GroupEnd;
    });
    return api;
}

inline int nc(ncclResult_t r) { return r == ncclSuccess ? ZMOE_OK : ZMOE_ERR_COMM; }
inline int cu(cudaError_t e) { return e == cudaSuccess ? ZMOE_OK : ZMOE_ERR_CUDA; }

constexpr int EP_MAX_WORLD = 32;   // destination masks are one 32-bit word per token

// ---------------------------------------------------------------------------
// device side of the exchange
// ---------------------------------------------------------------------------
// mask[t]: bit d set when rank d owns an expert of token t (ids outside [0, E) are inactive routes)
__global__ void ep_mask_kernel(const int32_t *__restrict__ ids, uint32_t *__restrict__ mask, int T, int K, int per_rank,
                               int E) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    uint32_t m = 0;
    for (int k = 0; k < K; ++k) {
        const int e = ids[(size_t)t * K + k];
        if (e >= 0 && e < E) m |= 1u << (e / per_rank);
    }
    mask[t] = m;
}

// One CTA.  pos[t * N + d]: how many tokens before t also go to rank d (-1 when t does not go there);
// counts[d]; send_off[d]: first row of rank d's block in the packed send buffers (exclusive prefix of counts).
// Stable (token order inside every destination), so the exchange is reproducible.
__global__ void __launch_bounds__(1024) ep_positions_kernel(const uint32_t *__restrict__ mask, int *__restrict__ pos,
                                                            int *__restrict__ counts, int *__restrict__ send_off, int T,
                                                            int N) {
    __shared__ int warp_tot[32];
    __shared__ int base_s;
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int d = 0; d < N; ++d) {
        if (tid == 0) base_s = 0;
        __syncthreads();
        for (int t0 = 0; t0 < T; t0 += 1024) {
            const int t = t0 + tid;
            const bool on = t < T && ((mask[t] >> d) & 1u);
            const unsigned b = __ballot_sync(0xffffffffu, on);
            const int before = __popc(b & ((1u << lane) - 1u));
            if (lane == 0) warp_tot[warp] = __popc(b);
            __syncthreads();
            int wbase = 0;
            for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
            const int base = base_s;
            if (t < T) pos[(size_t)t * N + d] = on ? base + wbase + before : -1;
            __syncthreads();
            if (tid == 1023) base_s = base + wbase + __popc(b);
            __syncthreads();
        }
        if (tid == 0) counts[d] = base_s;
        __syncthreads();
    }
    if (tid == 0) {
        int run = 0;
        for (int d = 0; d < N; ++d) {
            send_off[d] = run;
            run += counts[d];
        }
        send_off[N] = run;
    }
}

// packs rows by destination: CTA (t, d) copies x[t, :] and the token's K routes to row send_off[d] + pos[t, d]
__global__ void __launch_bounds__(256) ep_pack_kernel(const float *__restrict__ x, const int32_t *__restrict__ ids,
                                                      const float *__restrict__ w, const int *__restrict__ pos,
                                                      const int *__restrict__ send_off, float *__restrict__ sx,
                                                      int32_t *__restrict__ sids, float *__restrict__ sw, int T, int N,
                                                      int D, int K) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x / N, d = blockIdx.x % N;
    if (t >= T) return;
    const int ps = pos[(size_t)t * N + d];
    if (ps < 0) return;
    const size_t row = (size_t)send_off[d] + ps;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)t * D);
    float4 *dst = reinterpret_cast<float4 *>(sx + row * D);
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) dst[i] = src[i];
    if (threadIdx.x < K) {
        sids[row * K + threadIdx.x] = ids[(size_t)t * K + threadIdx.x];
        sw[row * K + threadIdx.x] = w[(size_t)t * K + threadIdx.x];
    }
}

// out[t, :] = sum over the ranks d the token went to, in ascending d, of yb[send_off[d] + pos[t, d], :]
__global__ void __launch_bounds__(256) ep_combine_kernel(const float *__restrict__ yb, const int *__restrict__ pos,
                                                         const int *__restrict__ send_off, float *__restrict__ out,
                                                         int T, int N, int D) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int D4 = D / 4;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)T * D4; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / D4), d4 = (int)(i % D4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        bool first = true;
        for (int d = 0; d < N; ++d) {
            const int ps = pos[(size_t)t * N + d];
            if (ps < 0) continue;
            const float4 v = reinterpret_cast<const float4 *>(yb + ((size_t)send_off[d] + ps) * D)[d4];
            if (first) { acc = v; first = false; }
            else acc = make_float4(__fadd_rn(acc.x, v.x), __fadd_rn(acc.y, v.y), __fadd_rn(acc.z, v.z), __fadd_rn(acc.w, v.w));
        }
        reinterpret_cast<float4 *>(out + (size_t)t * D)[d4] = acc;
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// handle
// ---------------------------------------------------------------------------
struct zmoe_ep {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, max_t = 0, D = 0, K = 0, fan = 1;
    size_t cap_send = 0, cap_recv = 0;   // rows
    uint32_t *mask = nullptr;
    int *pos = nullptr, *counts = nullptr, *send_off = nullptr, *all_counts = nullptr;
    int *all_counts_host = nullptr;      // pinned
    float *sx = nullptr, *sw = nullptr, *rx = nullptr, *rw = nullptr, *ry = nullptr, *yb = nullptr;
    int32_t *sids = nullptr, *rids = nullptr;
    // sizes of the last exchange, for callers that report traffic
    long last_sent_rows = 0, last_recv_rows = 0;
};

extern "C" {

int zmoe_ep_unique_id(void *id128) {
    if (!id128) return ZMOE_ERR_ARG;
    if (!nccl().ok) return ZMOE_ERR_COMM;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId");
    return nc(nccl().GetUniqueId(static_cast<ncclUniqueId *>(id128)));
}

int zmoe_ep_comm_init(const void *id128, int rank, int world, void **comm_out) {
    if (!id128 || !comm_out || world <= 0 || rank < 0 || rank >= world) return ZMOE_ERR_ARG;
    if (!nccl().ok) return ZMOE_ERR_COMM;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    const int rc = nc(nccl().CommInitRank(&c, world, id, rank));
    *comm_out = c;
    return rc;
}

int zmoe_ep_comm_destroy(void *comm) {
    if (!comm) return ZMOE_ERR_ARG;
    if (!nccl().ok) return ZMOE_ERR_COMM;
    return nc(nccl().CommDestroy(static_cast<ncclComm_t>(comm)));
}

void zmoe_ep_destroy(zmoe_ep *ep) {
    if (!ep) return;
    cudaFree(ep->mask); cudaFree(ep->pos); cudaFree(ep->counts); cudaFree(ep->send_off); cudaFree(ep->all_counts);
    cudaFree(ep->sx); cudaFree(ep->sw); cudaFree(ep->rx); cudaFree(ep->rw); cudaFree(ep->ry); cudaFree(ep->yb);
    cudaFree(ep->sids); cudaFree(ep->rids);
    if (ep->all_counts_host) cudaFreeHost(ep->all_counts_host);
    delete ep;
}

int zmoe_ep_create(void *nccl_comm, int rank, int world, int max_tokens, int max_recv_tokens, int d_model, int topk,
                   zmoe_ep **out) {
    if (!out || !nccl_comm || world <= 0 || world > EP_MAX_WORLD || rank < 0 || rank >= world || max_tokens <= 0 ||
        max_recv_tokens <= 0 || d_model <= 0 || d_model % 4 || topk <= 0 || topk > 256)
        return ZMOE_ERR_ARG;
    if (!nccl().ok) return ZMOE_ERR_COMM;
    zmoe_ep *ep = new (std::nothrow) zmoe_ep();
    if (!ep) return ZMOE_ERR_ARG;
    ep->comm = static_cast<ncclComm_t>(nccl_comm);
    ep->rank = rank; ep->world = world; ep->max_t = max_tokens; ep->D = d_model; ep->K = topk;
    ep->fan = world < topk ? world : topk;           // ranks one token can go to
    ep->cap_send = (size_t)max_tokens * ep->fan;
    ep->cap_recv = (size_t)max_recv_tokens;
    auto A = [](auto **p, size_t n) { return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(**p)) == cudaSuccess ? 0 : 1; };
    int bad = 0;
    bad |= A(&ep->mask, (size_t)max_tokens);
    bad |= A(&ep->pos, (size_t)max_tokens * world);
    bad |= A(&ep->counts, (size_t)world);
    bad |= A(&ep->send_off, (size_t)world + 1);
    bad |= A(&ep->all_counts, (size_t)world * world);
    bad |= A(&ep->sx, ep->cap_send * d_model);
    bad |= A(&ep->sids, ep->cap_send * topk);
    bad |= A(&ep->sw, ep->cap_send * topk);
    bad |= A(&ep->yb, ep->cap_send * d_model);
    bad |= A(&ep->rx, ep->cap_recv * d_model);
    bad |= A(&ep->rids, ep->cap_recv * topk);
    bad |= A(&ep->rw, ep->cap_recv * topk);
    bad |= A(&ep->ry, ep->cap_recv * d_model);
    bad |= cudaHostAlloc(reinterpret_cast<void **>(&ep->all_counts_host), (size_t)world * world * sizeof(int),
                         cudaHostAllocDefault) != cudaSuccess;
    if (bad) {
        zmoe_ep_destroy(ep);
        return ZMOE_ERR_CUDA;
    }
    *out = ep;
    return ZMOE_OK;
}

int zmoe_ep_forward_routed(zmoe_ep *ep, zmoe_layer *local, zmoe_layer *shared, int n_experts_total, const float *x_dev,
                           const int32_t *ids_dev, const float *weights_dev, float *out_dev, int T, void *stream) {
    if (!ep || !local || !x_dev || !ids_dev || !weights_dev || !out_dev || T <= 0 || n_experts_total <= 0)
        return ZMOE_ERR_ARG;
    if (T > ep->max_t) return ZMOE_ERR_CAPACITY;
    const int N = ep->world, D = ep->D, K = ep->K;
    if (n_experts_total % N) return ZMOE_ERR_ARG;
    const int per_rank = n_experts_total / N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const NcclApi &nc_api = nccl();

    // ---- destinations ----
    int rc = cu(launch_pdl(ep_mask_kernel, dim3((T + 255) / 256), dim3(256), 0, st, ids_dev, ep->mask, T, K, per_rank,
                           n_experts_total));
    if (!rc) rc = cu(launch_pdl(ep_positions_kernel, dim3(1), dim3(1024), 0, st, (const uint32_t *)ep->mask, ep->pos,
                                ep->counts, ep->send_off, T, N));
    if (!rc) rc = cu(launch_pdl(ep_pack_kernel, dim3((unsigned)T * N), dim3(256), 0, st, x_dev, ids_dev, weights_dev,
                                (const int *)ep->pos, (const int *)ep->send_off, ep->sx, ep->sids, ep->sw, T, N, D, K));
    count_launches(3);
    if (rc) return rc;
    // ---- sizes: every rank learns every count; the host needs them for the transfers ----
    rc = nc(nc_api.AllGather(ep->counts, ep->all_counts, (size_t)N, ncclInt32, ep->comm, st));
    if (!rc) rc = cu(cudaMemcpyAsync(ep->all_counts_host, ep->all_counts, (size_t)N * N * sizeof(int),
                                     cudaMemcpyDeviceToHost, st));
    if (!rc) rc = cu(cudaStreamSynchronize(st));
    if (rc) return rc;
    std::vector<size_t> s_cnt(N), s_off(N + 1, 0), r_cnt(N), r_off(N + 1, 0);
    for (int d = 0; d < N; ++d) {
        s_cnt[d] = (size_t)ep->all_counts_host[ep->rank * N + d];
        r_cnt[d] = (size_t)ep->all_counts_host[d * N + ep->rank];
        s_off[d + 1] = s_off[d] + s_cnt[d];
        r_off[d + 1] = r_off[d] + r_cnt[d];
    }
    const size_t n_recv = r_off[N];
    ep->last_sent_rows = (long)s_off[N];
    ep->last_recv_rows = (long)n_recv;
    if (s_off[N] > ep->cap_send || n_recv > ep->cap_recv) return ZMOE_ERR_CAPACITY;
    // ---- dispatch ----
    rc = nc(nc_api.GroupStart());
    for (int peer = 0; peer < N && !rc; ++peer) {
        if (s_cnt[peer]) {
            rc |= nc(nc_api.Send(ep->sx + s_off[peer] * D, s_cnt[peer] * D, ncclFloat, peer, ep->comm, st));
            rc |= nc(nc_api.Send(ep->sids + s_off[peer] * K, s_cnt[peer] * K, ncclInt32, peer, ep->comm, st));
            rc |= nc(nc_api.Send(ep->sw + s_off[peer] * K, s_cnt[peer] * K, ncclFloat, peer, ep->comm, st));
        }
        if (r_cnt[peer]) {
            rc |= nc(nc_api.Recv(ep->rx + r_off[peer] * D, r_cnt[peer] * D, ncclFloat, peer, ep->comm, st));
            rc |= nc(nc_api.Recv(ep->rids + r_off[peer] * K, r_cnt[peer] * K, ncclInt32, peer, ep->comm, st));
            rc |= nc(nc_api.Recv(ep->rw + r_off[peer] * K, r_cnt[peer] * K, ncclFloat, peer, ep->comm, st));
        }
    }
    const int rc_end = nc(nc_api.GroupEnd());
    if (!rc) rc = rc_end;
    if (rc) return ZMOE_ERR_COMM;
    // ---- this rank's experts over what arrived: one pre-weighted, pre-reduced row per received token ----
    if (n_recv) {
        // Most routes of the received tokens name experts held elsewhere, which the layer entry cannot see from
        // the host when it picks its kernels: choose by the pairs per expert of the whole exchange (every rank
        // brings about T tokens, so about T * K pairs land on each rank's E / N experts)
        zmoe_ctx *lctx = layer_context(local);
        const int prev_path = context_path(lctx);
        if (prev_path == 0)
            zmoe_ctx_set_path(lctx, (long)T * K >= (long)zmoe_gemm_min_pairs_per_expert() * per_rank ? 2 : 1);
        rc = zmoe_set_routes_window(local, ep->rx, ep->rids, ep->rw, (int)n_recv, ep->rank * per_rank, stream);
        if (!rc) rc = zmoe_expert_ffn(local, ep->ry, (int)n_recv, 0, stream);
        if (prev_path == 0) zmoe_ctx_set_path(lctx, 0);
        if (rc) return rc;
    }
    // ---- combine: the rows go back where they came from ----
    rc = nc(nc_api.GroupStart());
    for (int peer = 0; peer < N && !rc; ++peer) {
        if (r_cnt[peer]) rc |= nc(nc_api.Send(ep->ry + r_off[peer] * D, r_cnt[peer] * D, ncclFloat, peer, ep->comm, st));
        if (s_cnt[peer]) rc |= nc(nc_api.Recv(ep->yb + s_off[peer] * D, s_cnt[peer] * D, ncclFloat, peer, ep->comm, st));
    }
    const int rc_end2 = nc(nc_api.GroupEnd());
    if (!rc) rc = rc_end2;
    if (rc) return ZMOE_ERR_COMM;
    const long n4 = (long)T * (D / 4);
    long grid = (n4 + 255) / 256;
    const long cap = 8L * device_sm_count();
    if (grid > cap) grid = cap;
    rc = cu(launch_pdl(ep_combine_kernel, dim3((unsigned)grid), dim3(256), 0, st, (const float *)ep->yb,
                       (const int *)ep->pos, (const int *)ep->send_off, out_dev, T, N, D));
    count_launches(1);
    // the shared expert runs on the tokens' home rank and is added to the routed sum
    if (!rc && shared) rc = zmoe_dense_ffn(shared, x_dev, out_dev, T, 1, stream);
    return rc;
}

int zmoe_ep_forward(zmoe_ep *ep, zmoe_layer *router, zmoe_layer *local, zmoe_layer *shared, const float *x_dev,
                    float *out_dev, int T, void *stream) {
    if (!ep || !router || !local) return ZMOE_ERR_ARG;
    int rc = zmoe_route(router, x_dev, T, stream);
    if (rc) return rc;
    const int32_t *ids = nullptr;
    const float *w = nullptr;
    int n_total = 0;
    rc = layer_route_table(router, &ids, &w, &n_total);
    if (rc) return rc;
    return zmoe_ep_forward_routed(ep, local, shared, n_total, x_dev, ids, w, out_dev, T, stream);
}

int zmoe_ep_last_rows(zmoe_ep *ep, int64_t *sent_rows, int64_t *recv_rows) {
    if (!ep) return ZMOE_ERR_ARG;
    if (sent_rows) *sent_rows = ep->last_sent_rows;
    if (recv_rows) *recv_rows = ep->last_recv_rows;
    return ZMOE_OK;
}

}  // extern "C"
