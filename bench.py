"""Benchmark of the MoE expert hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

Workload (`config.workload`): the decode sweep configuration -- a stack of 8 MoE
layers, hidden 4096, 128 experts, top-8 softmax routing, expert FFN dim 1536,
gate/up weights Q2_K and down weights Q3_K (random super-blocks), T tokens of
N(0,1) activations per layer.  One "step" is one pass of T tokens through the 8
layers: router top-k, grouping, gate/up matmul + SwiGLU, down matmul, weighted
combine.  Weights of the 8 layers (7 GB) cycle through HBM every step, so the
inputs are far larger than L2.

Printed JSON (rank 0): `value` = tokens/s with inputs resident in HBM; `e2e` =
the same through the host-buffer entry (pinned host -> device copy of the
activations and device -> host read of the output inside the timed region, per
layer, as the reference's layer call does); `roofline` = achieved HBM GB/s of
the dominant kernel (gate/up matmul) against the measured copy bandwidth;
`cpu_baseline` = the CPU restatement of the reference path timed on this box.
Further keys report the other benchmark configurations on the same GPUs: `sweep`
(batches 1 / 4 / 16 / 64 of the stack), `cfg1` (one Q4_K layer 2048 / 768, 1 and 64
tokens), `prefill` (IQ2_XXS, 4096 tokens, Zipf-skewed load, tensor-core grouped
GEMM), `cfg4` (DeepSeek-V3-shaped layer, 256 experts + shared expert, 64 and 8192
tokens), `cfg5` (the full 48-layer decoder: prompt of 512 tokens, 256 greedy steps, one GPU) and, with N > 1,
`strong` (the stack at a fixed global batch of 128).

With N > 1 (torchrun) the experts of every layer are sharded over the ranks
(expert parallel).  The headline keeps every rank's T tokens (weak scaling);
`prefill`, `cfg4` and `strong` split a fixed global batch over the ranks.  Small
batches exchange rows with all-gather / reduce-scatter, large ones with the
library's all-to-all (zmoe_ep_forward).  Rank 0 checks a sample of its output
rows against the CPU oracle outside the timed regions.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q2_K, Q3_K, Q4_K, IQ2_XXS = 10, 11, 12, 16
BB = {Q2_K: 84, Q3_K: 110, Q4_K: 144, IQ2_XXS: 66}
HALF_OFFS = {Q2_K: (80, 82), Q3_K: (108,), Q4_K: (0, 2), IQ2_XXS: (0,)}
METRIC = "moe_layer_stack_decode_tokens_per_s"
UNIT = "tokens/s"

# the benchmark configurations (BASELINE.json `configs`), one dict each
CFG2 = dict(name="decode sweep: 8 MoE layers, hidden 4096, 128 experts top-8 softmax, ffn 1536, "
                 "gate/up Q2_K + down Q3_K random blocks",
            D=4096, F=1536, E=128, K=8, types=(Q2_K, Q2_K, Q3_K), layers=8, router={}, sigma=0.02)
CFG1 = dict(name="single MoE layer: hidden 2048, 128 experts top-8 softmax, ffn 768, Q4_K",
            D=2048, F=768, E=128, K=8, types=(Q4_K,) * 3, layers=8, router={}, sigma=0.02)   # 8 weight sets in turn: past L2
CFG3 = dict(name="prefill grouped GEMM: hidden 4096, 128 experts top-8, ffn 1536, IQ2_XXS, Zipf(1.1) expert load",
            D=4096, F=1536, E=128, K=8, types=(IQ2_XXS,) * 3, layers=1, router={}, sigma=0.02, zipf=1.1)
CFG4 = dict(name="DeepSeek-V3-shaped layer: hidden 7168, 256 experts + 1 shared, ffn 2048, top-8 sigmoid gating, "
                 "8 groups of which 4 used, Q4_K",
            D=7168, F=2048, E=256, K=8, types=(Q4_K,) * 3, layers=1, sigma=0.012, shared=True, bias_sigma=0.05,
            router=dict(gating=1, weights_norm=1, weights_scale=2.5, n_groups=8, n_groups_used=4))
D, F, E, K = CFG2["D"], CFG2["F"], CFG2["E"], CFG2["K"]
TYPES = CFG2["types"]


def workload_name(T):
    return CFG2["name"] + ", batch %d tokens" % T


def config_dict(T, world):
    """the `config` of the JSON line; identical in both arms"""
    return {"workload": workload_name(T), "tokens_per_step_per_gpu": T, "layers": CFG2["layers"],
            "parallelism": "ep%d" % world if world > 1 else "single"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def row_bytes(qtype, cols):
    return cols // 256 * BB[qtype]


def expert_bytes(cfg):
    """bytes of one expert's gate, up and down tensors"""
    t = cfg["types"]
    return (cfg["F"] * row_bytes(t[0], cfg["D"]), cfg["F"] * row_bytes(t[1], cfg["D"]),
            cfg["D"] * row_bytes(t[2], cfg["F"]))


# ---------------------------------------------------------------------------
# synthetic weights: every tensor of every expert has its own generator stream, so
# any shard (and the CPU check of a few experts) sees the same bytes
# ---------------------------------------------------------------------------
def torch_blocks(qtype, n_blocks, gen, device):
    """uint8 [n_blocks, block_bytes]: uniform random bytes, fp16 super-scales |N(0, 0.01)|"""
    import torch
    bb = BB[qtype]
    blocks = torch.randint(0, 256, (n_blocks, bb), dtype=torch.uint8, device=device, generator=gen)
    for off in HALF_OFFS[qtype]:
        h = (torch.randn(n_blocks, device=device, generator=gen) * 0.01).abs().to(torch.float16)
        blocks[:, off:off + 2] = h.view(torch.uint8).reshape(n_blocks, 2)
    return blocks


def expert_tensors(cfg, seed, layer, e, gen, device):
    """(gate, up, down) of expert e of a layer: uint8 [rows, row_bytes] each; e = -1 is the shared expert"""
    Dm, Ff, t = cfg["D"], cfg["F"], cfg["types"]
    gen.manual_seed(seed * 1000003 + layer * 1009 + (e + 1) + 7919 * (cfg["D"] + cfg["E"]))
    g = torch_blocks(t[0], Ff * (Dm // 256), gen, device).reshape(Ff, -1)
    u = torch_blocks(t[1], Ff * (Dm // 256), gen, device).reshape(Ff, -1)
    d = torch_blocks(t[2], Dm * (Ff // 256), gen, device).reshape(Dm, -1)
    return g, u, d


def router_tensors(cfg, seed, layer, device):
    """router matrix [E, D] and the selection bias [E] (None where the configuration has none)"""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 7919 + layer + 31 * cfg["E"] + cfg["D"])
    wr = torch.randn((cfg["E"], cfg["D"]), device=device, generator=gen) * cfg["sigma"]
    bias = None
    if cfg.get("zipf"):
        # Zipf(s) over a random expert ranking, as a selection bias on the router probabilities
        rank = torch.randperm(cfg["E"], device=device, generator=gen).double() + 1.0
        pz = rank.pow(-cfg["zipf"])
        bias = (2.0 * pz / pz.sum()).float()
    elif cfg.get("bias_sigma"):
        bias = torch.randn(cfg["E"], device=device, generator=gen) * cfg["bias_sigma"]
    return wr, bias


def make_inputs(cfg, seed, T, device, rank=0):
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 31 + 17 + 1000 * rank + cfg["D"])
    return [torch.randn((T, cfg["D"]), device=device, generator=gen) for _ in range(cfg["layers"])]


class Stack:
    """The layers of one configuration on this rank: all experts (one GPU) or this rank's shard."""

    def __init__(self, lib, cfg, seed, dev, rank, world, tokens_per_rank, path=0):
        import torch
        self.lib, self.cfg, self.dev, self.rank, self.world, self.seed = lib, cfg, dev, rank, world, seed
        Dm, Ff, En, Kk, t = cfg["D"], cfg["F"], cfg["E"], cfg["K"], cfg["types"]
        self.e_lo, self.e_hi = rank * En // world, (rank + 1) * En // world
        ne = self.e_hi - self.e_lo
        self.T = tokens_per_rank
        gen = torch.Generator(device=dev)
        rbs = [row_bytes(t[0], Dm), row_bytes(t[1], Dm), row_bytes(t[2], Ff)]
        self.weights, self.routers, self.shared_w = [], [], []
        for l in range(cfg["layers"]):
            wg = torch.empty((ne, Ff, rbs[0]), dtype=torch.uint8, device=dev)
            wu = torch.empty((ne, Ff, rbs[1]), dtype=torch.uint8, device=dev)
            wd = torch.empty((ne, Dm, rbs[2]), dtype=torch.uint8, device=dev)
            for e in range(self.e_lo, self.e_hi):
                wg[e - self.e_lo], wu[e - self.e_lo], wd[e - self.e_lo] = expert_tensors(cfg, seed, l, e, gen, dev)
            wr, bias = router_tensors(cfg, seed, l, dev)
            self.weights.append((wg, wu, wd, wr))
            self.routers.append((wr, bias))
            if cfg.get("shared"):
                self.shared_w.append(tuple(a.unsqueeze(0).contiguous() for a in expert_tensors(cfg, seed, l, -1, gen, dev)))
        # capacity: a rank may be handed every token of every rank
        self.ctx = lib.Context(max(self.T * world, 64), Dm, Ff, ne, Kk)
        if path:
            self.ctx.set_path(path)
        self.layers, self.shared, self.shard = [], [], None
        if world == 1:
            for l, (wg, wu, wd, wr) in enumerate(self.weights):
                self.layers.append(lib.Layer(self.ctx, Dm, Ff, ne, Kk, t, wg, wu, wd, router_w=wr,
                                             router_bias=self.routers[l][1], **cfg["router"]))
            if self.shared_w:
                self.sctx = lib.Context(max(self.T, 64), Dm, Ff, 1, 1)
                self.shared = [lib.Layer(self.sctx, Dm, Ff, 1, 1, t, *sw) for sw in self.shared_w]
        else:
            from zeromoe_b200 import expert_parallel as ep
            spec = dict(cfg["router"])
            if self.routers[0][1] is not None:
                spec["bias"] = [b for _, b in self.routers]
            self.shard = ep.ExpertShard(self.ctx, rank, world, En, Kk, Dm, Ff, t, self.weights, dev, router=spec,
                                        shared=self.shared_w or None, max_tokens=max(self.T, 1))

    def forward_layer(self, l, x, out, stream=None):
        if self.world == 1:
            self.layers[l].forward(x, out, stream)
            if self.shared:
                self.shared[l].dense_ffn(x, out, accumulate=1, stream=stream)
        else:
            self.shard.forward(l, x, out)

    def step(self, xs, outs):
        for l in range(self.cfg["layers"]):
            self.forward_layer(l, xs[l], outs[l])

    def routes_of_layer0(self, x):
        """(ids, weights) [T, K] the device router gives for x on layer 0 (host arrays)"""
        import torch
        if self.world == 1:
            self.layers[0].route(x)
            torch.cuda.synchronize()
            return self.ctx.routes(x.shape[0], self.cfg["K"])
        self.shard.routers[0].route(x)
        torch.cuda.synchronize()
        return self.shard.route_ctx.routes(x.shape[0], self.cfg["K"])

    def check_layer0(self, x, out, sample=None):
        """max-abs error of `sample` output rows of layer 0 against the CPU oracle, relative to the norm of the
        reference rows.  Only the experts the sampled tokens use are rebuilt on the host."""
        import torch
        from oracle import oracle as O
        cfg = self.cfg
        if sample is None:                       # keep the host copy of the used experts near a gigabyte
            sample = 32 if sum(expert_bytes(cfg)) < (8 << 20) else 6
        ids, w = self.routes_of_layer0(x)
        n = min(sample, x.shape[0])
        ids, w = ids[:n], w[:n]
        used = sorted(set(int(e) for e in ids.flatten() if 0 <= e < cfg["E"]))
        remap = {e: i for i, e in enumerate(used)}
        gen = torch.Generator(device=self.dev)
        parts = [expert_tensors(cfg, self.seed, 0, e, gen, self.dev) for e in used]
        wg = torch.stack([p[0] for p in parts]).cpu().numpy()
        wu = torch.stack([p[1] for p in parts]).cpu().numpy()
        wd = torch.stack([p[2] for p in parts]).cpu().numpy()
        cid = np.vectorize(lambda e: remap.get(int(e), -1))(ids).astype(np.int32)
        xh = x[:n].cpu().numpy()
        L = O.make_layer(cfg["D"], cfg["F"], len(used), cfg["K"], cfg["types"], wg, wu, wd)
        ref, _ = O.moe_ffn(L, xh, cid, w, fast=True)
        if cfg.get("shared"):
            sg, su, sd = (a.cpu().numpy()[None] for a in expert_tensors(cfg, self.seed, 0, -1, gen, self.dev))
            Ls = O.make_layer(cfg["D"], cfg["F"], 1, 1, cfg["types"], sg, su, sd)
            rs, _ = O.moe_ffn(Ls, xh, np.zeros((n, 1), np.int32), np.ones((n, 1), np.float32), fast=True)
            ref = ref + rs
        got = out[:n].cpu().numpy()
        return float(np.abs(got - ref).max() / (np.linalg.norm(ref) + 1e-30))

    def distinct_local_experts(self):
        """experts of this rank's shard the last expert FFN call touched"""
        return int((self.ctx.expert_freq(self.e_hi - self.e_lo) > 0).sum())

    def close(self):
        if self.shard is not None:
            self.shard.close()


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.idx = gpu_index
        self.t0 = self.t1 = None

    def mark(self, begin):
        """the timed region begins / ends now: only samples taken inside it count"""
        if begin:
            self.t0 = time.perf_counter()
        else:
            self.t1 = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment to come up: wait for its first line so that the timed region is covered
            deadline = time.perf_counter() + 2.0
            while not self.rows and time.perf_counter() < deadline:
                time.sleep(0.01)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.perf_counter()] + [c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r[1:] for r in self.rows
                if self.t0 is None or self.t1 is None or self.t0 <= r[0] <= self.t1 + 0.03]
        if not rows:                       # region shorter than one sampling period: the nearest samples
            rows = [r[1:] for r in self.rows]
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU leg (the oracle's SIMD + OpenMP twin); used by --impl reference and by cpu_baseline
# ---------------------------------------------------------------------------
def cpu_model_name():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_layers(seed, n_layers):
    """host copies of the first layers of the decode stack and a runner f(l, x) -> (out, threads used)"""
    import torch
    from oracle import oracle as O
    gen = torch.Generator(device="cpu")
    layers = []
    for l in range(n_layers):
        parts = [expert_tensors(CFG2, seed, l, e, gen, "cpu") for e in range(E)]
        wg = torch.stack([p[0] for p in parts]).numpy()
        wu = torch.stack([p[1] for p in parts]).numpy()
        wd = torch.stack([p[2] for p in parts]).numpy()
        wr = router_tensors(CFG2, seed, l, "cpu")[0].numpy()
        layers.append((O.make_layer(D, F, E, K, TYPES, wg, wu, wd), wr))

    def run(l, x):
        L, wr = layers[l]
        logits = O.router_logits(x, wr)
        _, ids, w, _ = O.router_select(logits, K)
        return O.moe_ffn(L, x, ids, w, fast=True, threads=0)
    return run


def cpu_dot_kind():
    from oracle import oracle as O
    try:
        return O.fast_kind()
    except AttributeError:
        return "AVX2"


def run_reference_arm(args, rank, world):
    """the CPU restatement of the reference's ggml path on this box's host cores: all host threads, the
    whole job's tokens per step, a bounded sample of the stack's layers scaled to 8"""
    if rank != 0:
        return
    # one OpenMP thread per core, spread over the cores (read by the OpenMP runtime when it starts, so set
    # before anything loads it); torchrun's default of one thread per rank does not apply to this arm
    os.environ["OMP_PROC_BIND"] = "spread"
    os.environ["OMP_PLACES"] = "cores"
    os.environ.pop("OMP_NUM_THREADS", None)
    cores = os.cpu_count() or 1
    T = args.tokens * world
    nl = 2
    run = cpu_layers(args.seed, nl)
    # rotating inputs: a different batch (hence different routed experts) every repetition
    xsets = [[x.numpy() for x in make_inputs(CFG2, args.seed, T, "cpu", rank=r)[:nl]] for r in range(4)]
    used = 1

    def step(i):
        nonlocal used
        for l in range(nl):
            _, used = run(l, xsets[i % 4][l])
    for i in range(max(args.warmup, 1)):
        step(i)
    # at least about a second of timed work, in whole multiples of the requested steps
    reps, t0 = 0, time.perf_counter()
    while reps < args.steps or time.perf_counter() - t0 < 1.0:
        step(reps)
        reps += 1
    dt = (time.perf_counter() - t0) / reps * (CFG2["layers"] / nl)
    val = T / dt
    sample = ("%d of 8 layers per step, scaled to 8; %d timed steps over 4 rotating input batches; %s dots, "
              "OpenMP over rows grouped by expert, threads spread over the cores (OMP_PROC_BIND)" % (nl, reps, cpu_dot_kind()))
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int2/int3 dot, f32 accumulate", "data": "synthetic",
            "config": config_dict(args.tokens, world),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": used, "kind": "port", "sample": sample,
                             "host_cores": cores, "cpu": cpu_model_name(), "tokens_per_step": T},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# timing helpers
# ---------------------------------------------------------------------------
class Timer:
    def __init__(self, dev, world):
        import torch
        self.torch, self.dev, self.world = torch, dev, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps):
        """ms per step: CUDA events on the launching stream, barrier + synchronise on both sides, max over ranks"""
        torch = self.torch
        self.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(self.stream)
        for _ in range(steps):
            fn()
        ev1.record(self.stream)
        self.barrier()
        ms = ev0.elapsed_time(ev1)
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def sum_over_ranks(self, v):
        if self.world == 1:
            return v
        import torch.distributed as dist
        t = self.torch.tensor([float(v)], device=self.dev, dtype=self.torch.float64)
        dist.all_reduce(t)
        return float(t.item())


def run_case(lib, tm, cfg, seed, dev, rank, world, tokens_global, steps, warmup=3, check=True, peaks=None):
    """one configuration at a fixed global batch: tokens/s of the whole job, per-GPU traffic of the decode-shaped
    calls, tensor throughput of the prefill-shaped ones, error of a sample against the oracle"""
    import torch
    T = max(1, tokens_global // world)
    st = Stack(lib, cfg, seed, dev, rank, world, T)
    xs = make_inputs(cfg, seed, T, dev, rank)
    outs = [torch.empty((T, cfg["D"]), device=dev) for _ in range(cfg["layers"])]
    for _ in range(warmup):
        st.step(xs, outs)
    ms = tm.timed(lambda: st.step(xs, outs), steps)
    st.ctx.check()
    calls = cfg["layers"]
    res = {"workload": cfg["name"], "tokens_global": T * world, "tokens_per_gpu": T, "ms_per_call": ms / calls,
           "tokens_per_s": T * world / (ms / calls * 1e-3)}
    pairs = T * world * cfg["K"]
    gemm = pairs >= lib.load().zmoe_gemm_min_pairs_per_expert() * cfg["E"]
    if gemm:
        flops = pairs * 3 * 2 * cfg["D"] * cfg["F"] * (1 + (1.0 / cfg["K"] if cfg.get("shared") else 0))
        tf = flops / (ms / calls * 1e-3) / 1e12
        res.update({"bound": "tensor", "tflops": tf, "tflops_per_gpu": tf / world,
                    "frac_per_gpu": tf / world / peaks["bf16_tflops"], "peak_tflops": peaks["bf16_tflops"]})
    else:
        # bytes this rank streamed in its last call: the distinct local experts it touched
        n_loc = st.distinct_local_experts()
        eb = sum(expert_bytes(cfg)) * (n_loc + (1 if cfg.get("shared") else 0)) + cfg["E"] * cfg["D"] * 4
        tot = tm.sum_over_ranks(eb)
        gbs = tot / world / (ms / calls * 1e-3) / 1e9
        res.update({"bound": "hbm", "distinct_local_experts_rank0": n_loc, "gbs_per_gpu": gbs,
                    "frac_per_gpu": gbs / peaks["hbm_gbs"], "peak_gbs": peaks["hbm_gbs"]})
    if world > 1 and st.shard._ep is not None:
        s, r = st.shard.last_rows()
        res["a2a_rows_sent_recv_rank0"] = [s, r]
        res["exchange"] = "all-to-all (zmoe_ep_forward)"
    elif world > 1:
        res["exchange"] = "all-gather / reduce-scatter"
    if check and rank == 0:
        st.forward_layer(0, xs[0], outs[0])
        torch.cuda.synchronize()
        res["max_abs_err_rel_to_norm"] = st.check_layer0(xs[0], outs[0])
    elif check:
        st.forward_layer(0, xs[0], outs[0])          # collectives need every rank
        torch.cuda.synchronize()
    freq = None
    if world == 1:
        st.layers[0].route(xs[0])
        torch.cuda.synchronize()
        freq = st.ctx.expert_freq(cfg["E"])
        res["pairs_per_expert"] = {"max": int(freq.max()), "median": float(np.median(freq)), "min": int(freq.min())}
    st.close()
    del st, xs, outs
    torch.cuda.empty_cache()
    return res


CFG5 = dict(name="full random-init MoE decoder: 48 layers, hidden 2048, GQA 32 query / 4 KV heads of 128, RoPE, f16 KV "
                 "cache (4096 positions), 128 experts top-8 ffn 768 Q4_K, Q8_0 attention and output head, vocab 151552; "
                 "prompt 512 tokens, 256 generated",
            layers=48, D=2048, H=32, KV=4, hd=128, F=768, E=128, K=8, V=151552, ctx=4096, prompt=512, gen=256)


def q8_0_rows(rows, cols, gen, device, d_sigma):
    """uint8 [rows, cols / 32 * 34]: random int8 quants, fp16 scales |N(0, d_sigma)|"""
    import torch
    nb = rows * (cols // 32)
    blk = torch.randint(0, 256, (nb, 34), dtype=torch.uint8, device=device, generator=gen)
    h = (torch.randn(nb, device=device, generator=gen) * d_sigma).abs().to(torch.float16)
    blk[:, 0:2] = h.view(torch.uint8).reshape(nb, 2)
    return blk.reshape(rows, -1)


def run_decoder_case(lib, dev, seed, peaks, cfg=CFG5):
    """The fifth configuration on one GPU: the prompt in one step, then `gen` greedy steps of one token each, the
    sampled token and the position staying on the device (a step captured once as a CUDA graph and replayed).
    Reports decode tokens/s and the HBM fraction of the bytes a decode step has to stream."""
    import torch
    c = cfg
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed * 101 + 5)
    D, F, E, K, H, KV, hd, V = c["D"], c["F"], c["E"], c["K"], c["H"], c["KV"], c["hd"], c["V"]
    ctx = lib.Context(c["prompt"], D, F, E, K)
    layers = []
    for l in range(c["layers"]):
        wg = torch_blocks(Q4_K, E * F * (D // 256), gen, dev).reshape(E, F, -1)
        wu = torch_blocks(Q4_K, E * F * (D // 256), gen, dev).reshape(E, F, -1)
        wd = torch_blocks(Q4_K, E * D * (F // 256), gen, dev).reshape(E, D, -1)
        wr = torch.randn((E, D), device=dev, generator=gen) * 0.02
        moe = lib.Layer(ctx, D, F, E, K, (Q4_K,) * 3, wg, wu, wd, router_w=wr)
        layers.append(dict(attn_norm=torch.ones(D, device=dev), ffn_norm=torch.ones(D, device=dev),
                           wqkv=q8_0_rows((H + 2 * KV) * hd, D, gen, dev, 2e-4), wo=q8_0_rows(D, H * hd, gen, dev, 2e-4),
                           moe=moe, keep=(wg, wu, wd, wr)))
    embd = q8_0_rows(V, D, gen, dev, 0.01)
    head = q8_0_rows(V, D, gen, dev, 2e-4)
    dec = lib.Decoder(layers, embd, torch.ones(D, device=dev), head, D, H, KV, hd, V, max_ctx=c["ctx"],
                      max_tokens=c["prompt"])
    prompt = torch.randint(0, V, (c["prompt"],), dtype=torch.int32, device=dev, generator=gen)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    dec.step(prompt)                       # warm-up of the prompt path
    dec.reset()
    torch.cuda.synchronize()
    ev[0].record()
    dec.step(prompt)
    ev[1].record()
    torch.cuda.synchronize()
    ctx.check()
    prefill_ms = ev[0].elapsed_time(ev[1])
    # one decode step as a graph; the position and the token live on the device, so replays continue the sequence
    for _ in range(3):
        dec.step()
    torch.cuda.synchronize()
    graph, launch = None, "eager"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dec.step()
        launch = "cuda graph replay"
    except Exception as exc:
        graph = None
        sys.stderr.write("decoder step capture failed, timing eager launches: %r\n" % (exc,))
    dec.reset()
    dec.step(prompt)
    torch.cuda.synchronize()
    toks = []
    ev[2].record()
    for i in range(c["gen"]):
        if graph is not None:
            graph.replay()
        else:
            dec.step()
    ev[3].record()
    torch.cuda.synchronize()
    ctx.check()
    tok, pos, lg = dec.read(64)
    decode_ms = ev[2].elapsed_time(ev[3])
    eb = F * row_bytes(Q4_K, D) * 2 + D * row_bytes(Q4_K, F)
    attn_b = ((H + 2 * KV) * hd + D) * (D // 32) * 34 if H * hd == D else ((H + 2 * KV) * hd * (D // 32) + D * (H * hd // 32)) * 34
    kv_b = 2 * (c["prompt"] + c["gen"] / 2) * KV * hd * 2
    per_tok = c["layers"] * (K * eb + attn_b + E * D * 4 + kv_b) + V * (D // 32) * 34
    res = {"workload": c["name"], "decode_tokens_per_s": c["gen"] / (decode_ms * 1e-3), "ms_per_token": decode_ms / c["gen"],
           "prompt_ms": prefill_ms, "prompt_tokens_per_s": c["prompt"] / (prefill_ms * 1e-3), "launch": launch,
           "bytes_per_token": per_tok, "frac_of_hbm_peak": per_tok / (decode_ms / c["gen"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
           "final_position": pos, "last_token": tok, "logits_finite": bool(np.isfinite(lg).all()),
           "check": "tokens in range and logits finite; parity of the step against the CPU restatement is tested at "
                    "small shapes (tests/test_gpu_decoder.py)",
           "n_gpus_note": "one GPU; the decoder step has no expert-parallel form yet"}
    assert pos == c["prompt"] + c["gen"] and 0 <= tok < V
    dec.close()
    del dec, layers, embd, head
    torch.cuda.empty_cache()
    return res


def gemm_cycles(lib, calls):
    """per-role cycle sums of the grouped GEMM's CTA 0 (only a profiling build of the library has them)"""
    import ctypes as C
    cyc = (C.c_uint64 * 32)()
    if lib.load().zmoe_debug_gemm_cycles(cyc) != 0:
        return None
    names = ["stages", "conv_wait_raw", "conv_wait_stage", "conv_work", "conv_fence_arrive", "mma_wait_full",
             "mma_issue", "mma_wait_acc", "drain_wait", "drain_work", "load_wait", "load_issue", "tiles"]
    return {k: {nm: cyc[16 * j + i] / max(calls, 1) for i, nm in enumerate(names)}
            for j, k in enumerate(("gate_up", "down"))}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=16, help="tokens per step per GPU (1, 4 or 16 in the sweep)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the extra batch sizes and configurations")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill-shaped configuration")
    ap.add_argument("--path", type=int, default=0, help="zmoe_ctx_set_path for the decode stack (0 = the library's choice)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the prefill-shaped configuration (profiler captures)")
    ap.add_argument("--prefill-experts", type=int, default=E)
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=8, help="layers in the stack (8 = the benchmark configuration; "
                    "fewer only for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    CFG2["layers"] = args.layers

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from zeromoe_b200 import lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib.load()
    peaks, which = measured_peaks()
    tm = Timer(dev, world)

    if args.prefill_only:
        cfg = dict(CFG3, E=args.prefill_experts)
        res = run_case(lib, tm, cfg, args.seed, dev, rank, world, args.prefill_tokens, 3, peaks=peaks)
        cyc = gemm_cycles(lib, 3 + 3 + 1)
        if cyc:
            res["gemm_cycles_cta0_per_call"] = cyc
        if rank == 0:
            print(json.dumps({"prefill": res}))
        return

    T = args.tokens
    t_all = T * world
    LAYERS = CFG2["layers"]
    stack = Stack(lib, CFG2, args.seed, dev, rank, world, T, path=args.path)
    ctx, layers = stack.ctx, stack.layers
    xs = make_inputs(CFG2, args.seed, T, dev, rank)
    outs = [torch.empty((T, D), device=dev) for _ in range(LAYERS)]
    stream = torch.cuda.current_stream()

    def step_eager():
        stack.step(xs, outs)
    step, graph = step_eager, None
    if world == 1 and not args.no_graph:
        # the library only enqueues kernels on the stream it is given, so a step can be
        # captured once and replayed (the reference replays its MoE graphs the same way)
        for _ in range(2):
            step_eager()
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_eager()
            step = graph.replay
        except Exception as exc:      # capture not possible: time eager launches, say so
            graph = None
            sys.stderr.write("graph capture failed, timing eager launches: %r\n" % (exc,))

    # kernels per step, counted by the library on an eager step (a graph replay launches the same nodes)
    launches0 = lib.load().zmoe_kernel_launches()
    step_eager()
    launches_per_step = lib.load().zmoe_kernel_launches() - launches0
    # warm-up: the requested steps, then as many more as take about half a second (clocks settle, the sampler
    # below has rows from a warm GPU even when the timed region is a few tens of milliseconds).  The count
    # comes from a step time that is the maximum over the ranks, so every rank runs the same number of steps.
    for _ in range(args.warmup):
        step()
    ms_probe = tm.timed(step, 3)
    extra = int(min(2000, max(0, 500.0 / max(ms_probe, 1e-3) - args.warmup - 3)))
    for i in range(extra):
        step()
        if i % 16 == 15:
            torch.cuda.synchronize()
    warm_run = args.warmup + 3 + extra
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.mark(True)
    ms_step = tm.timed(step, args.steps)
    if rank == 0:
        sampler.mark(False)
    clocks = sampler.stop() if rank == 0 else None
    launches = launches_per_step * args.steps
    ctx.check()
    value = t_all / (ms_step * 1e-3)
    # parity of this very stack: rank 0's first rows of layer 0 against the CPU oracle
    stack.forward_layer(0, xs[0], outs[0])
    torch.cuda.synchronize()
    err_main = stack.check_layer0(xs[0], outs[0]) if rank == 0 else None

    # ---- end to end through the host-buffer entry --------------------------------------
    xh = [x.cpu().pin_memory() for x in xs]
    oh = [torch.empty((T, D), dtype=torch.float32).pin_memory() for _ in range(LAYERS)]
    if world == 1:
        def step_host():
            for l in range(LAYERS):
                layers[l].forward_host(xh[l], oh[l])
        api = "zmoe_moe_forward_host per layer (pinned host in, host out, stream sync per layer)"
    else:
        # expert parallel: every rank copies its own tokens in and its own output rows out
        xdev = [torch.empty_like(x) for x in xs]

        def step_host():
            for l in range(LAYERS):
                xdev[l].copy_(xh[l], non_blocking=True)
                stack.forward_layer(l, xdev[l], outs[l])
                oh[l].copy_(outs[l], non_blocking=True)
                torch.cuda.current_stream().synchronize()
        api = "ExpertShard.forward per layer with pinned host activations in and host output back"
    for _ in range(3):
        step_host()
    tm.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    tm.barrier()
    dt = (time.perf_counter() - t0) / args.steps
    if world > 1:
        tt = torch.tensor([dt], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
    else:
        assert torch.equal(oh[0], outs[0].cpu()), "host entry and device entry disagree"
    e2e = {"value": t_all / dt, "unit": UNIT, "h2d_bytes_per_step": LAYERS * T * D * 4 * world,
           "d2h_bytes_per_step": LAYERS * T * D * 4 * world, "ms_per_step": dt * 1e3, "api": api}

    # ---- roofline of the dominant kernel (gate/up matmul + SwiGLU) ---------------------
    eb = expert_bytes(CFG2)
    roofline, layer_roofline = None, None
    if world == 1:
        # distinct experts hit per layer decide the algorithmic bytes
        nact = []
        for l in range(LAYERS):
            layers[l].route(xs[l], stream)
            torch.cuda.synchronize()
            nact.append(int((ctx.expert_freq(E) > 0).sum()))
        gu_bytes = [n * (eb[0] + eb[1]) for n in nact]
        dn_bytes = [n * eb[2] for n in nact]
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(LAYERS)]
        reps, gu_ms = max(5, args.steps // 5), 0.0
        for r in range(3 + reps):
            for l in range(LAYERS):
                layers[l].route(xs[l], stream)
                layers[l].expert_ffn_timed(outs[l], evs[l][0], evs[l][1], stream)
            torch.cuda.synchronize()
            if r >= 3:
                gu_ms += sum(a.elapsed_time(b) for a, b in evs)
        gu_ms /= reps * LAYERS
        ach = (sum(gu_bytes) / LAYERS) / (gu_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "mmid2_kernel<Q2_K, dual> (gate/up matmul + SwiGLU)", "achieved": ach,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_source": which,
                    "avg_launch_ms": gu_ms, "bytes_per_launch": sum(gu_bytes) / LAYERS,
                    # dram__bytes_read + write of this kernel from ncu on a 1-layer capture of the same
                    # batch: 342.9 MB read + 5.0 MB written for 342.8 MB of algorithmic bytes; traffic is
                    # proportional to the distinct experts streamed, so the ratio carries over to a full launch
                    "traffic": sum(gu_bytes) / LAYERS * (347.9 / 342.8),
                    "traffic_source": "scaled from the ncu capture of a 1-layer run of the same batch "
                                      "(profiles/mmid2_kernel_decode_cfg2.md), not measured in this run",
                    "distinct_experts_per_layer": nact}
        step_bytes = sum(gu_bytes) + sum(dn_bytes) + LAYERS * E * D * 4
        layer_roofline = {"algorithmic_bytes_per_step": step_bytes, "achieved": step_bytes / (ms_step * 1e-3) / 1e9,
                          "unit": "GB/s", "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "frac_of_8TBs_nominal": step_bytes / (ms_step * 1e-3) / 8e12}
    else:
        # per-GPU traffic of the sharded step: distinct local experts of the last layer's call, all layers alike
        n_loc = stack.distinct_local_experts()
        per_gpu = LAYERS * (n_loc * sum(eb) + E * D * 4)
        tot = tm.sum_over_ranks(per_gpu)
        gbs = tot / world / (ms_step * 1e-3) / 1e9
        layer_roofline = {"algorithmic_bytes_per_step_all_gpus": tot, "achieved_per_gpu": gbs, "unit": "GB/s",
                          "frac_per_gpu": gbs / peaks["hbm_gbs"], "distinct_local_experts_rank0": n_loc}

    # ---- the other batch sizes of the sweep, and the first configuration ------------------
    sweep, cfg1 = {}, None
    if world == 1 and not args.no_sweep:
        for t2 in (1, 4, 16, 64):   # 64: beyond the configuration's sweep, where experts hold several pairs
            if t2 == T:
                sweep[str(t2)] = {"tokens_per_s": value, "ms_per_step": ms_step}
                continue
            xs2 = make_inputs(CFG2, args.seed, t2, dev, rank)
            outs2 = [torch.empty((t2, D), device=dev) for _ in range(LAYERS)]

            def step2():
                stack.step(xs2, outs2)
            for _ in range(args.warmup):
                step2()
            fn2 = step2
            if graph is not None:
                torch.cuda.synchronize()
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2):
                    step2()
                fn2 = g2.replay
                fn2()
            ms2 = tm.timed(fn2, args.steps)
            # bytes of the distinct experts this batch touches, all layers
            nb = 0
            for l in range(LAYERS):
                layers[l].route(xs2[l], stream)
                torch.cuda.synchronize()
                nb += int((ctx.expert_freq(E) > 0).sum()) * sum(eb) + E * D * 4
            sweep[str(t2)] = {"tokens_per_s": t2 / (ms2 * 1e-3), "ms_per_step": ms2,
                              "frac_of_hbm_peak": nb / (ms2 * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    stack.close()
    del stack, layers, xs, outs
    torch.cuda.empty_cache()

    extra_steps = max(5, min(30, args.steps // 4))
    if world == 1 and not args.no_sweep:
        # first configuration: one Q4_K layer; eight weight sets take turns so that the 21 MB a token
        # touches do not stay in L2
        cfg1 = {}
        for t1 in (1, 64):
            r = run_case(lib, tm, CFG1, args.seed, dev, rank, world, t1, extra_steps, peaks=peaks)
            cfg1[str(t1)] = r

    # ---- prefill-shaped configuration (tensor-core path), fixed global batch -----------------
    prefill, cfg4, strong = None, None, None
    if not args.no_prefill and LAYERS == 8:
        prefill = run_case(lib, tm, CFG3, args.seed, dev, rank, world, 4096, 5, peaks=peaks)
        prefill["kernel"] = "gemm_sm100_kernel (tcgen05.mma kind::f16, fp16 operands, f32 TMEM accumulators)"
        # the keys the single-GPU line has always carried
        if "tflops" in prefill:
            prefill["frac"] = prefill["tflops"] / world / peaks["bf16_tflops"]
    if not args.no_sweep and LAYERS == 8:
        cfg4 = {"decode_64": run_case(lib, tm, CFG4, args.seed, dev, rank, world, 64, extra_steps, peaks=peaks),
                "prefill_8192": run_case(lib, tm, CFG4, args.seed, dev, rank, world, 8192, 3, peaks=peaks)}
        if world > 1:
            strong = run_case(lib, tm, CFG2, args.seed, dev, rank, world, 128, extra_steps, peaks=peaks)
            strong["note"] = "the 8-layer stack at a fixed global batch of 128 tokens (strong scaling)"

    cfg5 = None
    if world == 1 and not args.no_sweep and LAYERS == 8:
        cfg5 = run_decoder_case(lib, dev, args.seed, peaks)

    # ---- CPU baseline on a bounded sample -----------------------------------------------
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        run = cpu_layers(args.seed, 1)
        xsets = [make_inputs(CFG2, args.seed, T, "cpu", rank=r)[0].numpy() for r in range(4)]
        _, used = run(0, xsets[0])
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 4000):
            run(0, xsets[reps % 4])
            reps += 1
        dt = (time.perf_counter() - t0) / reps * CFG2["layers"]
        cpu = {"value": T / dt, "unit": UNIT, "cores": used, "kind": "port",
               "sample": "layer 0 of 8 (router + expert FFN), %d repetitions over 4 rotating input batches, scaled to "
                         "8 layers; %s dots, OpenMP over rows grouped by expert" % (reps, cpu_dot_kind()),
               "host_cores": os.cpu_count(), "cpu": cpu_model_name(),
               "gpu_vs_cpu_max_abs_err_rel_to_norm": err_main}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int8 x int2/int3 dot, f32 accumulate", "data": "synthetic",
                "config": config_dict(T, world),
                "notes": {"l2": "inputs larger than L2: 7.0 GB of expert weights cycle every step",
                          "launch": "cuda graph replay" if graph is not None else "eager",
                          "warmup_steps_run": warm_run,
                          "exchange": None if world == 1 else "all-gather / reduce-scatter (small batch)"},
                "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e, "roofline": roofline,
                "layer_stack_roofline": layer_roofline, "max_abs_err_rel_to_norm": err_main, "sweep": sweep,
                "cfg1": cfg1, "prefill": prefill, "cfg4": cfg4, "cfg5": cfg5, "strong": strong, "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
