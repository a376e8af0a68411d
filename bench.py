#!/usr/bin/env python
"""Benchmark of the MoE-layer hot path (ESMM / ESTMM / ESS + routing) through the MoE_Cascaded API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("c5-layer"): the d=2048 / hidden 8192 / 64 experts / top-2 bf16 MoE layer, GELU, both
biases, `--tokens` tokens per GPU (default 131072) ~ N(0,1), two such layers cascaded in one
MoE_Cascaded module so that the pipeline-shared cache has a next layer to prefetch.  A step is
forward + backward of both layers; the metric counts tokens through one layer:
value = tokens_per_gpu * n_gpus * layers / step_time.  With N > 1 the module runs in data-centric
mode (tokens sharded over ranks, expert weights sharded along the hidden dimension, all-gathered
per layer and their gradients reduce-scattered): weak scaling.

Prints ONE JSON line (rank 0).  `value` is measured with inputs resident in HBM; `e2e` repeats the
measurement with each step's input copied from pinned host memory (double-buffered: the upload of
step i+1 runs on a copy stream while step i computes, one upload per timed step) and the loss read
back to the host inside the timed region.  `roofline` is for the dominant kernel (the tcgen05 grouped GEMM),
from CUDA events recorded around its launches during the timed steps.  `cpu_baseline` times the
CPU oracle's restatement of the same layer on the host cores on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOP_K, LAYERS = 2, 2
WORKLOADS = {  # name -> (d_model, hidden, experts, default tokens per GPU)
    "c5": (2048, 8192, 64, 131072),
    "c2": (768, 3072, 32, 16384),
    "c5s": (2048, 8192, 8, 16384),      # the headline layer's d / hidden with 8 experts and 16384 tokens: same k-loop lengths
                                        # and tile shapes as c5 at ~3 GB resident (sized for ncu captures)
    "small": (256, 1024, 8, 8192),
    "c3": (1024, 4096, 64, 65536),      # operator sweep only (--ops): Zipf(1.2)-skewed routing, some experts empty
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU (default: the workload's)")
    ap.add_argument("--ops", action="store_true",
                    help="operator sweep instead of the module step: routing, ESMM forward (fc1 + GELU, fc2), ESMM input "
                         "gradient (x2), ESTMM (x2), ESS (x2), gather and combine timed separately on one GPU, each "
                         "with its roofline fraction (workloads c2: E=8 and E=32, uniform routing; c3: Zipf-skewed)")
    ap.add_argument("--workload", default="c5", choices=["c5", "c5s", "c2", "small", "c4", "c3"],
                    help="c5: the headline layer; c2: d=768/H=3072/E=32, 16384 tokens (operator-sweep config, sized for ncu "
                         "captures); small: d=256/H=1024/E=8, 8192 tokens (smoke); c4: the Swin-MoE-B-like network "
                         "(secondary: images/s through the whole synthetic model, 128 images of 192x192 per GPU)")
    ap.add_argument("--images", type=int, default=128, help="c4: images per GPU")
    ap.add_argument("--mode", default="data", choices=["data", "model"],
                    help="multi-GPU mode of the layer workloads: data-centric (tokens sharded, expert weights gathered "
                         "through the pipeline-shared cache) or model-centric (hidden dimension sharded, tokens gathered)")
    ap.add_argument("--hetero", action="store_true",
                    help="the heterogeneous model-centric case: hidden dimension split 0.2/0.2/0.15/0.15/0.1/0.1/0.05/0.05 "
                         "over 8 ranks (neighbouring shares merged for 4 and 2 ranks), 131072 tokens in total (strong "
                         "scaling), implies --mode model")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# dram bytes per launch / algorithmic bytes per launch of the GEMM kernels by launch type, from an ncu capture of one
# launch of each type at the headline d / hidden with 8 experts (same rows per expert, so traffic scales with the experts)
TRAFFIC_RATIO = {"esmm:fc1_forward_act": 1.27, "esmm:fc2_forward": 1.92, "estmm:dw2": 1.29, "esmm:fc2_dgrad_dact": 1.36,
                 "estmm:dw1": 1.29, "esmm:fc1_dgrad": 1.92}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops=float(p.get("bf16_tflops_sustained", p.get("bf16_tflops"))), burst=float(p["bf16_tflops"]),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1400.0, burst=1590.0, hbm=6650.0, source="fallback")


class InputPrefetcher:
    """Double-buffered host -> device feed for the end-to-end measurement: every call of next() returns the device
    buffer whose upload (from pinned host memory, on a copy stream) was started one step earlier and starts the
    upload of the following step's input into the other buffer, so each timed step contains exactly one upload,
    overlapped with the previous step's kernels."""

    def __init__(self, host, bufs):
        import torch
        self.torch, self.host, self.bufs = torch, host, bufs
        self.stream = torch.cuda.Stream(device=bufs[0].device)
        self.ready = [None, None]
        self.i = 0
        self._upload(0)

    def _upload(self, slot):
        torch = self.torch
        self.stream.wait_stream(torch.cuda.current_stream())      # the buffer's previous consumer has been enqueued
        with torch.cuda.stream(self.stream):
            self.bufs[slot].copy_(self.host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.ready[slot] = ev

    def next(self):
        slot = self.i & 1
        self.i += 1
        self.torch.cuda.current_stream().wait_event(self.ready[slot])
        self._upload(slot ^ 1)
        return self.bufs[slot]


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return None
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle's fp32 restatement on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_setup(d, H, E_sample, k, tokens):
    """Seeded synthetic inputs of one layer for the CPU pass (generated outside any timed region)."""
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(tokens, d, generator=g)
    w1 = torch.randn(E_sample, H, d, generator=g) / d ** 0.5
    w2 = torch.randn(E_sample, H, d, generator=g) / H ** 0.5
    b1 = torch.randn(E_sample, H, generator=g) * 0.02
    b2 = torch.randn(E_sample, d, generator=g) * 0.02
    dy = torch.randn(tokens, d, generator=g)
    ids = torch.topk(torch.randn(tokens, E_sample, generator=g), k, dim=1).indices.to(torch.int32)
    return x, ids, w1, w2, b1, b2, dy


def cpu_pass(data):
    """One fwd+bwd of the layer with the CPU oracle's grouped-matmul restatement; returns seconds."""
    from oracle import hexa_oracle as O
    t0 = time.perf_counter()
    O.moe_layer_fast(*data)
    return time.perf_counter() - t0


CPU_SAMPLE_TOKENS, CPU_SAMPLE_EXPERTS = 16384, 8


def cpu_sample(d, H, k):
    """The CPU arm's bounded sample, the same on every box: 16384 tokens (seed 0) routed top-k over 8 experts of the
    layer's own d and hidden size.  Per-token work (12*k*d*H flop forward + backward) is that of the full layer and
    does not depend on the expert count, so tokens/s of the sample is the rate of the full layer; nothing is
    extrapolated."""
    return cpu_setup(d, H, CPU_SAMPLE_EXPERTS, k, CPU_SAMPLE_TOKENS)


def cpu_sample_text(k, E):
    return (f"{CPU_SAMPLE_TOKENS} tokens (seed 0) top-{k} over {CPU_SAMPLE_EXPERTS} of the {E} experts, same d / hidden and "
            f"per-token work as the full layer, fp32, all host cores")


def layer_config(args, d, H, E, k, L, T, proportion):
    """The `config` object of the layer workloads: the same for this library's arm and for the reference arm."""
    return dict(workload=args.workload + "-layer", d_model=d, hidden=H, experts=E, hidden_split=proportion, top_k=k, layers=L,
                tokens_per_gpu=T, activation="gelu", mode=args.mode + "-centric",
                l2="inputs larger than L2 (expert weights %.1f GB per layer)" % (2 * E * H * d * 2 / 1e9))


def hetero_proportion(args, world):
    """(mode, hidden split, tokens per rank) of the heterogeneous model-centric case, else the arguments' own."""
    if not args.hetero:
        return None, None
    if 8 % world:
        raise SystemExit("--hetero needs 1, 2, 4 or 8 ranks")
    args.mode = "model"
    eighth = [0.2, 0.2, 0.15, 0.15, 0.1, 0.1, 0.05, 0.05]
    g = 8 // world
    return [round(sum(eighth[i * g:(i + 1) * g]), 6) for i in range(world)], world


def run_reference(args):
    """The reference has no CPU implementation of this path (its kernels are Triton / CUDA only), so this arm
    times the CPU oracle port of the same layer on the host cores, on a bounded token sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload not in WORKLOADS:      # the Swin harness is stock PyTorch around the layer; only the layer has a CPU arm
        print(json.dumps(dict(impl="reference", unavailable="no CPU arm for workload %s: use one of %s"
                                                            % (args.workload, ", ".join(WORKLOADS)))), flush=True)
        return
    d, H, EXPERTS, T_default = WORKLOADS[args.workload]
    k = TOP_K
    world = max(int(args.gpus), 1)
    proportion, _ = hetero_proportion(args, world)
    T = (args.tokens or T_default) // (world if args.hetero else 1)
    n = CPU_SAMPLE_TOKENS
    data = cpu_sample(d, H, k)
    for _ in range(min(args.warmup, 1)):
        cpu_pass(data)
    dt = sum(cpu_pass(data) for _ in range(args.steps)) / args.steps
    val = n / dt
    cores = os.cpu_count() or 1
    sample = cpu_sample_text(k, EXPERTS) + ", one fwd+bwd pass per step"
    line = dict(metric="moe_layer_fwd_bwd_tokens_per_s", value=val, unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", impl="reference",
                config=layer_config(args, d, H, EXPERTS, k, LAYERS, T, proportion),
                cpu_baseline=dict(value=val, unit="tokens/s", cores=cores, kind="port", sample=sample, extrapolated=False,
                                  note="CPU oracle port of the layer (fp32 grouped matmuls per expert): the reference ships "
                                       "no CPU path for these operators; one layer, one rank's host cores"),
                e2e=dict(value=val, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def run_ops(args, dev):
    """Operator sweep on one GPU: every operator of the layer timed alone (CUDA events on the launching stream, 3
    warm-up + `--steps` timed launches back to back; operands of one launch exceed L2 except at the `small` size).
    Tensor-bound operators are reported against the burst cuBLAS bf16 figure (kernels timed alone), HBM-bound ones
    against the measured copy bandwidth."""
    import torch
    from hexa_moe_b200 import _lib as L, ops
    d, H, E_default, T = WORKLOADS[args.workload]
    T = args.tokens or T
    k = TOP_K
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        pk = json.load(open(path))
        tf_peak, hbm_peak, src = float(pk["bf16_tflops"]), float(pk["hbm_gbs"]), "measured (burst cuBLAS bf16, copy bandwidth)"
    else:
        tf_peak, hbm_peak, src = 1590.0, 6650.0, "fallback"
    dt = torch.bfloat16
    results = []
    for E in ((8, 32) if args.workload == "c2" else (E_default,)):
        g = torch.Generator().manual_seed(0)
        if args.workload == "c3":       # Gumbel top-2 over Zipf(1.2) probabilities, the 4 least likely experts never chosen
            p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.2
            p = p[torch.randperm(E, generator=g)]
            p[torch.argsort(p)[:4]] = 0
            logit = torch.log(p / p.sum()).float().expand(T, E) - torch.log(-torch.log(torch.rand(T, E, generator=g)))
        else:
            logit = torch.randn(T, E, generator=g)
        ids = torch.topk(logit, k, dim=1).indices.to(torch.int32).to(dev)
        x = torch.randn(T, d, generator=g).to(dt).to(dev)
        dy = torch.randn(T, d, generator=g).to(dt).to(dev)
        w1 = (torch.randn(E, H, d, generator=g) / d ** 0.5).to(dt).to(dev)
        w2 = (torch.randn(E, H, d, generator=g) / H ** 0.5).to(dt).to(dev)
        b1 = (torch.randn(E, H, generator=g) * 0.02).to(dev)
        b2 = (torch.randn(E, d, generator=g) * 0.02).to(dev)
        r = ops.route(ids, E)
        xs, dys = ops.gather_rows(x, r), ops.gather_rows(dy, r)
        y1 = ops.sorted_buffer(r.row_capacity, H, dt, dev)
        h, dh = torch.empty_like(y1), torch.empty_like(y1)
        ys, dxs = torch.empty_like(xs), torch.empty_like(xs)
        dw = torch.empty(E, H, d, dtype=dt, device=dev)
        y = torch.empty(T, d, dtype=dt, device=dev)
        ops.esmm(xs, w1, L.B_NK, r, b1, L.EPI_ACT, L.ACT_GELU, aux=y1, out=h)
        N = T * k
        fl = 2.0 * N * d * H
        es = 2
        cases = [
            ("route", lambda: ops.route(ids, E), 0.0, 12.0 * N),
            ("gather x -> sorted rows", lambda: ops.gather_rows(x, r, out=xs), 0.0, 2.0 * N * d * es),
            ("ESMM fc1 + bias + GELU (forward)", lambda: ops.esmm(xs, w1, L.B_NK, r, b1, L.EPI_ACT, L.ACT_GELU, aux=y1, out=h), fl, 0.0),
            ("ESMM fc2 + bias (forward)", lambda: ops.esmm(h, w2, L.B_KN, r, b2, L.EPI_LINEAR, out=ys), fl, 0.0),
            ("combine routes (sum over k)", lambda: ops.combine_rows(ys, r, out=y), 0.0, (k + 1.0) * T * d * es),
            ("ESS db2", lambda: ops.ess(dys, r), 0.0, 1.0 * N * d * es),
            ("ESTMM dW2", lambda: ops.estmm(h, dys, r, out=dw), fl, 0.0),
            ("ESMM input gradient of fc2 x GELU'", lambda: ops.esmm(dys, w2, L.B_NK, r, None, L.EPI_DACT, L.ACT_GELU, aux=y1, out=dh), fl, 0.0),
            ("ESS db1", lambda: ops.ess(dh, r), 0.0, 1.0 * N * H * es),
            ("ESTMM dW1", lambda: ops.estmm(dh, xs, r, out=dw), fl, 0.0),
            ("ESMM input gradient of fc1", lambda: ops.esmm(dh, w1, L.B_KN, r, None, L.EPI_LINEAR, out=dxs), fl, 0.0),
        ]
        counts = r.counts.cpu()
        ops_out = {}
        for name, fn, flops, nbytes in cases:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / args.steps
            if flops:
                ach = flops / (ms * 1e-3) / 1e12
                ops_out[name] = dict(ms=round(ms, 4), bound="tensor", achieved=round(ach, 1), unit="TFLOP/s", frac=round(ach / tf_peak, 3))
            else:
                ach = nbytes / (ms * 1e-3) / 1e9
                ops_out[name] = dict(ms=round(ms, 4), bound="hbm", achieved=round(ach, 1), unit="GB/s", frac=round(ach / hbm_peak, 3))
        results.append(dict(experts=E, rows_per_expert_min=int(counts.min()), rows_per_expert_max=int(counts.max()),
                            empty_experts=int((counts == 0).sum()), ops=ops_out))
    esmm_fwd = [v for res in results for n_, v in res["ops"].items() if n_.startswith("ESMM fc")]
    value = 100.0 * sum(v["frac"] for v in esmm_fwd) / len(esmm_fwd)
    line = dict(metric="esmm_forward_pct_of_bf16_tensor_peak", value=value, unit="%", n_gpus=1, steps=args.steps, warmup=3,
                higher_is_better=True, vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload=args.workload + "-operator-sweep", tokens=T, d_model=d, hidden=H, top_k=k,
                            routing="zipf(1.2), 4 experts masked" if args.workload == "c3" else "uniform"),
                peaks=dict(tflops=tf_peak, hbm_gbs=hbm_peak, source=src), sweep=results)
    print(json.dumps(line), flush=True)


def run_swin(args, dev, rank, world, timed_factory=None):
    """Secondary workload: forward + backward of the synthetic Swin-MoE-B-like network (swin_moe_harness.py), bf16,
    data-centric at N > 1.  One JSON line with images/s and the MoE-layer token rate."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from hexa_moe_b200 import ops
    from swin_moe_harness import SwinMoEHarness
    torch.manual_seed(0)
    m = SwinMoEHarness().to(torch.bfloat16).to(dev).train()
    for g in m.cascaded_moe.gates:
        g.gate_noise = 0.0
    params = list(m.parameters())
    gen = torch.Generator().manual_seed(99 + rank)
    imgs_host = torch.randn(args.images, 3, 192, 192, generator=gen).to(torch.bfloat16).pin_memory()
    labels = torch.randint(0, 1000, (args.images,), generator=gen).to(dev)
    imgs_dev = imgs_host.to(dev)
    stage = torch.empty_like(imgs_dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step(x):
        for p in params:
            p.grad = None
        logits, aux = m(x)
        loss = F.cross_entropy(logits.float(), labels) + 0.01 * aux
        loss.backward()
        return loss

    loader = InputPrefetcher(imgs_host, [stage, torch.empty_like(imgs_dev)])

    def step_e2e():
        loss = step(loader.next())
        loss_host.copy_(loss.detach(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms / n

    for _ in range(max(args.warmup, 3)):
        step(imgs_dev)
    sampler = ClockSampler(dev.index or 0) if rank == 0 else None
    if sampler:
        sampler.start()
    l0 = ops.LAUNCHES
    ops.PROFILE = []
    ms = timed(lambda: step(imgs_dev), args.steps)
    prof, ops.PROFILE = ops.PROFILE, None
    launches = ops.LAUNCHES - l0
    clocks = sampler.stop() if sampler else None
    lib_ms = sum(e0.elapsed_time(e1) for _n, e0, e1, _w, _b in prof) / args.steps      # this library's kernels, per step
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    parity = multi_gpu_parity(rank, world, dev, True, None) if world > 1 else None
    if rank == 0:
        moe_tokens = sum(m.moe_tokens_per_image()) * args.images * world
        line = dict(metric="swin_moe_images_per_s", value=args.images * world / (ms * 1e-3), unit="images/s", n_gpus=world,
                    steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak",
                    vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload="c4-swin-moe-b-like", images_per_gpu=args.images, img=192, experts=32, top_k=1,
                                moe_layers=len(m.moe_idx), mode="data-centric",
                                note="window attention with relative position bias and shifted-window mask; stock PyTorch "
                                     "attention blocks around one shared MoE_Cascaded"),
                    moe_layer_tokens_per_s=moe_tokens / (ms * 1e-3), parity=parity,
                    library_kernel_ms_per_step=round(lib_ms, 3),
                    library_note="moe_layer_tokens_per_s divides the MoE-layer tokens of a step by the whole step; "
                                 "library_kernel_ms_per_step is the part of the step spent in this library's kernels (MoE "
                                 "layers and the dense FFNs of model dim >= 512), the rest is stock PyTorch attention",
                    e2e=dict(value=args.images * world / (ms_e2e * 1e-3), unit="images/s", ms_per_step=ms_e2e,
                             h2d_bytes_per_step=imgs_host.numel() * 2, d2h_bytes_per_step=4),
                    gpu_launches=launches, clocks=clocks)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        m.cascaded_moe.dispatch_params.cache.close()
        dist.barrier()
        dist.destroy_process_group()


def mean_square(h):
    """mean(h^2) in fp32 as one reduction pass forward and one scaling pass backward (the unfused
    h.float().pow(2).mean() makes seven passes over an activation-sized tensor; the loss of the benchmark step should
    cost what a fused loss costs)."""
    import torch

    class _MeanSquare(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t):
            ctx.save_for_backward(t)
            return torch.linalg.vector_norm(t, dtype=torch.float32).square() / t.numel()

        @staticmethod
        def backward(ctx, g):
            (t,) = ctx.saved_tensors
            # the scalar in the tensor's own dtype: one vectorised pass (a 16-bit tensor times an fp32 scalar tensor takes
            # PyTorch's generic, three times slower, mixed-type kernel)
            return t * (g * (2.0 / t.numel())).to(t.dtype)
    return _MeanSquare.apply(h)


# ------------------------------------------------------------------------------------------------
# multi-GPU correctness and timeline, outside every timed region
# ------------------------------------------------------------------------------------------------
def multi_gpu_parity(rank, world, dev, data_centric, proportion, dtype_name="bfloat16"):
    """One small fixed-seed forward + backward of a two-layer module on all ranks (6 experts, d=64, hidden 256,
    384 tokens per rank, top-2), compared with the CPU oracle's float64 layer: output, input gradient and the four
    parameter gradients of both layers on every rank.  The oracle is the checker only.  Returns a dict for the JSON
    line; `ok` is the AND over ranks, `max_rel` the largest error over ranks relative to the tolerance's scale."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from hexa_moe import moe as hmoe
    from oracle import hexa_oracle as O
    dtype = getattr(torch, dtype_name)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    E, d, H, k, L, T = 6, 64, 256, 2, 2, 384
    m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'fp32_gate': True}, model_dim_list=[d] * L, moe_idx_list=[0, 1],
                          mlp_ratio=H // d, mlp_proportion=proportion, num_global_experts=E, total_depth=L,
                          data_centric=data_centric, activation_fn=lambda t: F.gelu(t))
    g = torch.Generator().manual_seed(0)
    P = [dict(w1=torch.randn(E, H, d, generator=g) * 0.15, w2=torch.randn(E, H, d, generator=g) * 0.1,
              b1=torch.randn(E, H, generator=g) * 0.1, b2=torch.randn(E, d, generator=g) * 0.1,
              wg=torch.randn(E, d, generator=g) * 0.5) for _ in range(L)]
    split = [m.local_dim_list_all[r][0] for r in range(world)]
    lo, n = sum(split[:rank]), split[rank]
    with torch.no_grad():
        for i in range(L):
            for prm in (m.batched_fc1_w[i], m.batched_fc2_w[i], m.batched_fc1_bias[i]):
                prm.zero_()
            m.batched_fc1_w[i][:, :n] = P[i]["w1"][:, lo: lo + n]
            m.batched_fc2_w[i][:, :n] = P[i]["w2"][:, lo: lo + n]
            m.batched_fc1_bias[i][:, :n] = P[i]["b1"][:, lo: lo + n]
            m.batched_fc2_bias[i].copy_(P[i]["b2"]); m.gates[i].wg.weight.copy_(P[i]["wg"])
    m = m.to(dtype).to(dev).eval()
    Pd = [{k_: v.to(dtype).float() for k_, v in p.items()} for p in P]      # what the module really holds
    xs = [torch.randn(T, d, generator=torch.Generator().manual_seed(100 + r)).to(dtype) for r in range(world)]
    x = xs[rank].to(dev).requires_grad_(True)
    ids_used, h = [], x
    # the small module cuts its tokens into as many chunks as the timed step does (model-centric mode)
    least = os.environ.get("HEXA_MC_MIN_CHUNK_TOKENS")
    os.environ["HEXA_MC_MIN_CHUNK_TOKENS"] = "64"
    try:
        for i in range(L):
            h, _ = m(i, h)
            ids_used.append(torch.stack([t.cpu() for t in m.dispatch_params.indices_], dim=1))
        h.float().sum().backward()
        torch.cuda.synchronize()
    finally:
        if least is None:
            del os.environ["HEXA_MC_MIN_CHUNK_TOKENS"]
        else:
            os.environ["HEXA_MC_MIN_CHUNK_TOKENS"] = least
    all_ids = [[None] * world for _ in range(L)]
    for i in range(L):
        dist.all_gather_object(all_ids[i], ids_used[i])

    def run_rank(r):
        cur, saved = xs[r].double(), []
        for i in range(L):
            res = O.moe_layer(cur, all_ids[i][r], Pd[i]["w1"], Pd[i]["w2"], Pd[i]["b1"], Pd[i]["b2"], F.gelu)
            saved.append((cur, all_ids[i][r])); cur = res["y"].to(dtype).double()
        gy, grads = torch.ones_like(cur), [None] * L
        for i in reversed(range(L)):
            cin, ids = saved[i]
            grads[i] = O.moe_layer(cin, ids, Pd[i]["w1"], Pd[i]["w2"], Pd[i]["b1"], Pd[i]["b2"], F.gelu, gy)
            gy = grads[i]["dx"].to(dtype).double()
        return cur, gy, grads
    outs = [run_rank(r) for r in range(world)]

    def err(a, b):
        a, b = a.detach().double().cpu(), b.double()
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
    worst = max(err(h, outs[rank][0]), err(x.grad, outs[rank][1]))
    for i in range(L):
        comb = (lambda key: sum(outs[r][2][i][key] for r in range(world)) / world) if data_centric else \
               (lambda key: sum(outs[r][2][i][key] for r in range(world)))
        for prm, key, sliced in ((m.batched_fc1_w[i], "dw1", True), (m.batched_fc2_w[i], "dw2", True),
                                 (m.batched_fc1_bias[i], "db1", True), (m.batched_fc2_bias[i], "db2", False)):
            want = comb(key)[:, lo: lo + n] if sliced else comb(key)
            got = prm.grad[:, :n] if sliced else prm.grad
            worst = max(worst, err(got, want) / 1.5)          # reduced gradients: 1.5 x the tolerance, as in tests/
    if m.dispatch_params.cache is not None:
        dist.barrier(); m.dispatch_params.cache.close(); dist.barrier()
    t = torch.tensor([worst], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst = float(t)
    return dict(ok=bool(worst < tol), max_rel=worst, tolerance=tol, dtype=dtype_name, ranks=world,
                mode="data-centric" if data_centric else "model-centric", hidden_split=split,
                checked="y, dx, dW1, dW2, db1, db2 of both layers on every rank against the float64 CPU oracle; "
                        "6 experts, d=64, hidden 256, 384 tokens per rank, top-2")


def scale_timeline(cache, step_fn, steps, dev, world, my_kernel_ms, ms_step):
    """Where a multi-GPU step spends time outside this library's kernels: spans recorded by the pipeline-shared cache
    around every wait of the compute stream and every action of the side stream during `steps` extra steps, plus
    the spread over ranks of the kernel time per step (the slowest rank paces a synchronous step)."""
    import torch
    import torch.distributed as dist
    cache.timeline = []
    dist.barrier()
    torch.cuda.synchronize()
    for _ in range(steps):
        step_fn()
    torch.cuda.synchronize()
    spans, cache.timeline = cache.timeline, None
    agg = {}
    for site, stream_name, a, b in spans:
        key = stream_name + ":" + site
        agg[key] = agg.get(key, 0.0) + a.elapsed_time(b) / steps
    everyone = [None] * world
    dist.all_gather_object(everyone, dict(spans=agg, kernel_ms=my_kernel_ms))
    sites = sorted({k for e in everyone for k in e["spans"]})
    table = {}
    for k in sites:
        v = [e["spans"].get(k, 0.0) for e in everyone]
        table[k] = dict(min=round(min(v), 3), mean=round(sum(v) / len(v), 3), max=round(max(v), 3))
    km = [e["kernel_ms"] for e in everyone]
    exposed = [sum(v for k, v in e["spans"].items() if k.startswith("compute:")) for e in everyone]
    return dict(unit="ms per step", steps=steps, ms_per_step=round(ms_step, 3),
                kernel_ms_by_rank=[round(v, 2) for v in km], exposed_wait_ms_by_rank=[round(v, 3) for v in exposed],
                note="compute:* = time the compute stream was held at that wait; side:* = duration on the side stream "
                     "(overlapped with compute unless a compute wait shows it)", sites=table)


# ------------------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # the collectives overlap the persistent GEMM kernels: keep NCCL to a few CTAs (NVSwitch needs few to
        # saturate the links) so the SMs the GEMMs leave free (HEXA_COMM_SMS) are enough for it
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world

    from hexa_moe_b200 import build, ops
    from hexa_moe import moe as hmoe
    if rank == 0 and build.needs_build():
        build.build()
    if world > 1:
        dist.barrier()

    if args.ops:
        if world > 1:
            raise SystemExit("--ops is a single-GPU sweep")
        return run_ops(args, dev)
    if args.workload == "c3":
        raise SystemExit("workload c3 is an operator sweep: add --ops")
    if args.workload == "c4":
        return run_swin(args, dev, rank, world, timed_factory=None)
    d, H, E, T_default = WORKLOADS[args.workload]
    k, L = TOP_K, LAYERS
    T = args.tokens or T_default
    proportion, _ = hetero_proportion(args, world)
    if args.hetero:
        T = (args.tokens or T_default) // world            # the token count is global: every rank contributes its share
    torch.manual_seed(0)
    m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'fp32_gate': True}, model_dim_list=[d] * L,
                          moe_idx_list=list(range(L)), mlp_ratio=H // d, mlp_proportion=proportion, num_global_experts=E,
                          total_depth=L, data_centric=args.mode == "data", mlp_fc1_bias=True, mlp_fc2_bias=True,
                          activation_fn=lambda t: F.gelu(t))
    with torch.no_grad():   # random-init weights at a scale that keeps activations O(1)
        for name, p in m.named_parameters():
            if name.startswith("batched_fc1_w"):
                p.normal_(0, d ** -0.5)
            elif name.startswith("batched_fc2_w"):
                p.normal_(0, H ** -0.5)
            elif "bias" in name:
                p.normal_(0, 0.02)
    m = m.to(torch.bfloat16).to(dev).train()
    for g in m.gates:
        g.gate_noise = 0.0
    params = [p for p in m.parameters()]

    gen = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(T, d, generator=gen).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    x_stage = torch.empty_like(x_dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step(x):
        for p in params:
            p.grad = None
        h = x.detach().requires_grad_(True)
        aux = 0
        for i in range(L):
            h, l = m(i, h)
            aux = aux + l
        loss = mean_square(h) + 0.01 * aux
        loss.backward()
        return loss

    def step_resident():
        return step(x_dev)

    loader = InputPrefetcher(x_host, [x_stage, torch.empty_like(x_dev)])

    def step_e2e():
        # the way a training loop feeds the module: this step's input was uploaded (pinned host -> device, on a copy
        # stream) while the previous step computed; the upload of the next one starts now; the loss is read back
        x = loader.next()
        loss = step(x)
        loss_host.copy_(loss.detach(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(loss_host)

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
            dist.barrier()
        return ms / n

    for _ in range(max(args.warmup, 3)):
        step_resident()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = ops.LAUNCHES
    ops.PROFILE = []
    ms = timed(step_resident, args.steps)
    prof, ops.PROFILE = ops.PROFILE, None
    launches = ops.LAUNCHES - launches0
    clocks = sampler.stop() if sampler else None

    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)

    # ---- per-kernel summary from the events recorded during the timed steps ----
    per, per_type = {}, {}
    for name, e0, e1, work, nbytes in prof:
        t_ms = e0.elapsed_time(e1)
        s = per.setdefault(name.split(":")[0], [0, 0.0, 0.0, 0.0])
        s[0] += 1; s[1] += t_ms; s[2] += work; s[3] += nbytes
        if name.startswith(("esmm:", "estmm:")):
            s = per_type.setdefault(name, [0, 0.0, 0.0, 0.0])
            s[0] += 1; s[1] += t_ms; s[2] += work; s[3] += nbytes
    pk = peaks()
    z = [0, 0.0, 0.0, 0.0]
    gemm_n = per.get("esmm", z)[0] + per.get("estmm", z)[0]
    gemm_ms = per.get("esmm", z)[1] + per.get("estmm", z)[1]
    gemm_fl = per.get("esmm", z)[2] + per.get("estmm", z)[2]
    gemm_by = per.get("esmm", z)[3] + per.get("estmm", z)[3]
    achieved = gemm_fl / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    # DRAM bytes per launch: ncu captures of these kernels (dram read + write per launch against the algorithmic
    # operand + output bytes, one launch of each type) give the ratio; the headline workload itself is too large to
    # capture, so `traffic` is the algorithmic bytes of the timed launches times that measured ratio
    traffic_bytes = sum(v[3] * TRAFFIC_RATIO.get(n_, 1.5) for n_, v in per_type.items())
    ratio = traffic_bytes / gemm_by if gemm_by > 0 else 1.0
    by_type = {n_: dict(launches=v[0], avg_ms=round(v[1] / v[0], 4), tflops=round(v[2] / (v[1] * 1e-3) / 1e12, 1),
                        frac_of_sustained=round(v[2] / (v[1] * 1e-3) / 1e12 / pk["tflops"], 3),
                        frac_of_burst=round(v[2] / (v[1] * 1e-3) / 1e12 / pk["burst"], 3))
               for n_, v in sorted(per_type.items()) if v[1] > 0}
    roofline = dict(bound="tensor", kernel="gemm_tc_kernel (ESMM + ESTMM launches)", achieved=achieved, peak=pk["tflops"],
                    unit="TFLOP/s", frac=achieved / pk["tflops"], peak_source=pk["source"] + " (sustained cuBLAS bf16)",
                    frac_of_burst=achieved / pk["burst"], burst_peak=pk["burst"],
                    launches=gemm_n, avg_launch_ms=gemm_ms / max(gemm_n, 1), flops_per_launch=gemm_fl / max(gemm_n, 1),
                    traffic=traffic_bytes / max(gemm_n, 1), algorithmic_bytes=gemm_by / max(gemm_n, 1),
                    traffic_source="algorithmic bytes of the timed launches x the dram/algorithmic ratio of their launch "
                                   "type (%.2f on average) measured by ncu at the headline d / hidden with 8 experts" % ratio,
                    by_launch_type=by_type)
    kernels = {n_: dict(calls=v[0], ms_total=round(v[1], 3)) for n_, v in per.items()}
    my_kernel_ms = sum(v[1] for v in per.values()) / args.steps

    parity, timeline = None, None
    if world > 1:
        cache = m.dispatch_params.cache
        if cache is not None and cache.side is not None:
            timeline = scale_timeline(cache, step_resident, 3, dev, world, my_kernel_ms, ms)
        dist.barrier()
        parity = multi_gpu_parity(rank, world, dev, args.mode == "data", proportion)

    tokens_per_step = T * n_gpus * L
    value = tokens_per_step / (ms * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e * 1e-3)
    layer_flops = 12.0 * T * k * d * H * L
    cpu_baseline = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        data = cpu_sample(d, H, k)
        cpu_pass(data)                                               # warm-up (thread pool, page faults)
        secs = sorted(cpu_pass(data) for _ in range(3))[1]           # median of three
        cpu_baseline = dict(value=CPU_SAMPLE_TOKENS / secs, unit="tokens/s", cores=os.cpu_count() or 1, kind="port",
                            seconds=round(secs, 2), sample=cpu_sample_text(k, E) + ", median of 3 passes after 1 warm-up",
                            extrapolated=False)
    if rank == 0:
        line = dict(metric="moe_layer_fwd_bwd_tokens_per_s", value=value, unit="tokens/s", n_gpus=n_gpus, steps=args.steps,
                    warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True,
                    scaling="strong" if args.hetero else "weak", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=layer_config(args, d, H, E, k, L, T, proportion),
                    model_tflops_per_gpu=layer_flops / (ms * 1e-3) / 1e12,
                    model_frac_of_burst=layer_flops / (ms * 1e-3) / 1e12 / pk["burst"],
                    e2e=dict(value=e2e_value, unit="tokens/s", ms_per_step=ms_e2e, h2d_bytes_per_step=x_host.numel() * 2,
                             d2h_bytes_per_step=4, result="the loss scalar is read back every step; gradients stay on the "
                                                          "device, where an optimizer would consume them"),
                    parity=parity, scale_timeline=timeline,
                    gpu_launches=launches, kernels=kernels, roofline=roofline, cpu_baseline=cpu_baseline, clocks=clocks)
        if world > 1 and args.mode == "model":
            from hexa_moe_b200.impls.layers import token_chunks
            line["config"]["token_chunks"] = len(token_chunks([T] * world)[0]) - 1
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        if m.dispatch_params.cache is not None:
            m.dispatch_params.cache.close()      # unmap the other ranks' memory before anyone exits
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
