#!/usr/bin/env python
"""Benchmark of the DecDEC decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one generated token's pass through every quantized linear of the model (per layer:
wqkv, wo, w1w3, w2), each a fused call `dec_lutgemm` = 3-bit binary-coded GEMV + dynamic error
compensation (bucket top-k selection, zero-copy fetch of 4-bit residual rows from pinned host memory,
residual GEMV).  Weights, scales and residuals are seeded random tensors of the model's shapes (there
are no checkpoints here); every layer has its own storage, so a step streams far more than L2 holds.

The JSON line reports tokens/s with compensation on (`value`), the same with compensation off, the
HBM roofline of the GEMV kernel, the host-link rate of the residual fetch, an end-to-end number with
host buffers, and the reference's PyTorch CPU math timed on this box's cores.
With --gpus N > 1 (launched by torchrun) the model is tensor-parallel: column-parallel wqkv/w1w3,
row-parallel wo/w2 with an NCCL all-reduce; every rank fetches its own residual shard.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODELS = {
    # name: (layers, hidden, q_heads, kv_heads, head_dim, ffn)
    "llama3-8b": (32, 4096, 32, 8, 128, 14336),
    "phi3-medium": (40, 5120, 40, 10, 128, 17920),
    "llama3-70b": (80, 8192, 64, 8, 128, 28672),
}
BITS, GROUP = 3, 128
# (n_tb, k_chunk of wqkv, wo, w1w3, w2) chosen by `python -m decdec_b200.tuner` for a 5 % layer slowdown budget
# on one B200 (profiles/tuner_llama3-8b.md); timed as an extra operating point beside k_chunk = 32
TUNED_5PCT = {"llama3-8b": "16:0,0,5,3"}
NCU_TRAFFIC_RATIO = 51.73 / 51.50   # measured DRAM bytes / algorithmic bytes of k_bcq_pipe, profiles/k_bcq_pipe_*.md


def projections(model: str, tp: int = 1, rank: int = 0):
    """[(name, N_local, K_local, parallel)] of one layer; fused wqkv / w1w3 as in the reference model
    (end-to-end/model.py:266,331)."""
    from decdec_b200 import tp as tpl
    _, d, hq, hkv, hd, ffn = MODELS[model]
    qkv = (hq + 2 * hkv) * hd

    def col(n):
        a, b = tpl.split_even(n, tp, 128 if n % (128 * tp) == 0 else 32)[rank]
        return b - a

    def row(k):
        a, b = tpl.k_ranges(k, tp, GROUP)[rank]
        return b - a

    return [
        ("wqkv", col(qkv), d, "col"),
        ("wo", d, row(d), "row"),
        ("w1w3", col(2 * ffn), d, "col"),
        ("w2", d, row(ffn), "row"),
    ]


def gemv_bytes(n, k):
    """Algorithmic bytes of one binary-coded GEMV call (planes + alpha + q_bias + x + y read/write)."""
    return BITS * n * k / 8 + (k / GROUP) * BITS * n * 2 + (k / GROUP) * n * 2 + 2 * k + 4 * n


def fetch_bytes(n, k, k_chunk):
    """Bytes that cross the host link per call: k selected rows of N/2 bytes."""
    return (k_chunk * k // 1024) * n / 2


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler running beside the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                       "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [v.strip() for v in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        return out


# --------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's PyTorch math on host cores
# --------------------------------------------------------------------------------------------------

def cpu_sample(model: str, k_chunk: int, reps: int, warm: int):
    """Times the reference's CPU path (dequantise every call, exact per-chunk top-k, two mat-vecs;
    oracle/forward.py) on a bounded sample: the `wo` projection (hidden x hidden) of one layer.
    Returns (seconds per sample, sample description, scale = weights per token / weights in sample)."""
    import torch
    from oracle import forward as ofw
    layers, d, *_ = MODELS[model]
    n = k = d
    g = torch.Generator().manual_seed(0)
    qw = torch.randint(-2**31, 2**31 - 1, (k // 32, BITS, n), dtype=torch.int32, generator=g)
    alpha = (torch.rand(k // GROUP, BITS, n, generator=g) * 0.01).half()
    qb = ((torch.rand(k // GROUP, n, generator=g) - 0.5) * 0.01).half()
    cs = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=g)
    sc = (torch.rand(n, generator=g) * 1e-3).half()
    x = torch.randn(k, generator=g)

    def once():
        wt = ofw.torch_bcq_dequant(qw, alpha, qb, GROUP)
        rt = ofw.torch_unpack_residual(cs, sc) if k_chunk else None
        return ofw.cpu_reference_linear(x, wt, rt, k_chunk)

    for _ in range(warm):
        once()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter(); once(); ts.append(time.perf_counter() - t0)
    per_token = layers * sum(nn * kk for _, nn, kk, _ in projections(model))
    return ts, f"wo projection {n}x{k} of one layer: BCQ dequant + residual unpack + per-chunk top-k + 2 matvec, fp32", per_token / (n * k)


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun sets OMP_NUM_THREADS=1 for its ranks; the CPU arm uses every core this process may run on
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    cores = torch.get_num_threads()
    ts, desc, scale = cpu_sample(args.model, args.k_chunk, args.steps, max(1, args.warmup))
    total = sum(ts)
    tok_s = len(ts) / (total * scale)
    line = {
        "impl": "reference", "metric": "batch-1 decode tok/s (DecDEC on)", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(ts) * scale,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc + f"; scaled x{scale:.0f} to a token"},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(args):
    layers, d, hq, hkv, hd, ffn = MODELS[args.model]
    return {"workload": f"{args.model} decode hot path: {layers} layers x (wqkv, wo, w1w3, w2) fused GEMV+DEC, "
                        f"{BITS}-bit binary-coded group-{GROUP} weights, 4-bit residual rows in pinned host memory",
            "k_chunk": args.k_chunk, "n_tb": args.n_tb, "batch": 1,
            "parallelism": (f"tp{args.gpus}, row-parallel outputs summed by " + ("a one-shot push kernel over NVLink peer memory"
                            if args.allreduce == "push" else "ncclAllReduce")) if args.gpus > 1 else "single",
            "cache": "inputs larger than L2 (every layer has its own weights and residual; no L2 flush needed)"}


# --------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------

def build_model(args, torch, ext, dev, rank, tp):
    """Random packed tensors of the model's shapes; one storage per layer and projection."""
    layers = MODELS[args.model][0]
    if args.layers:
        layers = args.layers
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    gc = torch.Generator().manual_seed(99 + rank)
    rows = torch.zeros(32 * 1024, dtype=torch.int32, device=dev)
    acts = torch.zeros(32 * 1024, dtype=torch.float16, device=dev)
    ctx = ext.create_dec_context(args.n_tb, rows, acts)
    proj = projections(args.model, tp, rank)
    # one random residual per projection shape on the host; every config pins its own copy
    host_res = {}
    for name, n, k, _ in proj:
        host_res[name] = (torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=gc),
                          (torch.rand(n, generator=gc) * 1e-3 + 1e-4).half(),
                          torch.sort(torch.randn(k, generator=gc).abs() * 3, descending=True).values.half())
    model = []
    for _ in range(layers):
        layer = []
        for name, n, k, par in proj:
            qw = torch.randint(-2**31, 2**31 - 1, (k // 32, BITS, n), dtype=torch.int32, device=dev, generator=g)
            alpha = (torch.rand(k // GROUP, BITS, n, device=dev, generator=g) * 0.01).half()
            qb = ((torch.rand(k // GROUP, n, device=dev, generator=g) - 0.5) * 0.01).half()
            q, sc, thr = host_res[name]
            cfg_on = ext.create_dec_config(ctx, args.k_chunk, q, sc, thr)
            layer.append(dict(name=name, n=n, k=k, par=par, qw=qw, alpha=alpha, qb=qb, cfg=cfg_on, thr=thr))
        model.append(layer)
    # all layer outputs live in one buffer that is cleared once per token (the entry points accumulate
    # into their output; the reference's modules clear each output with its own kernel before every call)
    total = sum(p["n"] for layer in model for p in layer)
    ybuf = torch.zeros(total, dtype=torch.float16, device=dev)
    off = 0
    for layer in model:
        for p in layer:
            p["y"] = ybuf[off:off + p["n"]].view(1, 1, p["n"])
            off += p["n"]
    return model, ctx, (rows, acts, ybuf, host_res)


def make_inputs(torch, model, dev, n_sets=4):
    """Activation sets (N(0,1) with 1% x20 outliers) per input width, rotated between steps so that
    the selected rows change from token to token."""
    g = torch.Generator().manual_seed(7)
    widths = sorted({p["k"] for p in model[0]})
    sets = []
    for _ in range(n_sets):
        s = {}
        for k in widths:
            x = torch.randn(k, generator=g)
            idx = torch.randperm(k, generator=g)[: max(1, k // 100)]
            x[idx] *= 20
            s[k] = x.half().reshape(1, 1, k)
        sets.append(s)
    return widths, sets


def run_micro(args):
    """One entry point on one layer shape: `--micro KIND --n N --k K [--k-chunk C --n-tb T --iters I]`.
    Launches rotate over enough distinct weight tensors to exceed L2 (cache-cold), are captured in a CUDA
    graph and timed with CUDA events; prints one JSON line (us per launch, algorithmic GB/s).  Also the
    command used for the single-kernel ncu captures under profiles/."""
    import torch
    import decdec_ext as ext
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    N, K, kind = args.n, args.k, args.micro
    g = torch.Generator(device=dev).manual_seed(1)
    wbytes = BITS * N * K / 8
    ncopy = max(2, min(32, int(160e6 // wbytes) + 1))
    x = [torch.randn(1, 1, K, device=dev, generator=g).half() for _ in range(8)]
    y = torch.zeros(1, 1, N, dtype=torch.float16, device=dev)
    ri = lambda *shape: torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=g)
    cfg = None
    if "dec" in kind:
        gc = torch.Generator().manual_seed(2)
        rows = torch.zeros(32 * 1024, dtype=torch.int32, device=dev)
        acts = torch.zeros(32 * 1024, dtype=torch.float16, device=dev)
        ctx = ext.create_dec_context(args.n_tb, rows, acts)
        cfg = ext.create_dec_config(ctx, args.k_chunk, torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int32, generator=gc),
                                    (torch.rand(N, generator=gc) * 1e-3 + 1e-4).half(),
                                    torch.sort(torch.randn(K, generator=gc).abs() * 3, descending=True).values.half())
    if "lutgemm" in kind:
        w = [(ri(K // 32, BITS, N), (torch.rand(K // GROUP, BITS, N, device=dev, generator=g) * 0.01).half(),
              ((torch.rand(K // GROUP, N, device=dev, generator=g) - 0.5) * 0.01).half()) for _ in range(ncopy)]
        hbm = gemv_bytes(N, K)
        if kind == "lutgemm":
            call = lambda i: ext.lutgemm_gemv(x[i % 8], y, *w[i % ncopy], BITS, GROUP)
        else:
            call = lambda i: ext.dec_lutgemm(cfg, x[i % 8], y, *w[i % ncopy], BITS, GROUP)
    elif "anyprec" in kind:
        w = [(ri(BITS, N, K // 32), (torch.randn(N, 2 ** BITS, device=dev, generator=g) * 0.02).half()) for _ in range(ncopy)]
        hbm = BITS * N * K / 8 + N * 2 ** BITS * 2 + 2 * K + 4 * N
        if kind == "anyprec":
            call = lambda i: ext.anyprec_gemv(x[i % 8], y, *w[i % ncopy], BITS)
        else:
            call = lambda i: ext.dec_anyprec(cfg, x[i % 8], y, *w[i % ncopy], BITS)
    elif kind == "sqllm":
        w = [(ri(K * BITS // 32, N), (torch.randn(N, 2 ** BITS, device=dev, generator=g) * 0.02).half()) for _ in range(ncopy)]
        hbm = BITS * N * K / 8 + N * 2 ** BITS * 2 + 2 * K + 4 * N
        call = lambda i: ext.sqllm_gemv(x[i % 8], y, *w[i % ncopy], BITS)
    elif kind == "dec":
        hbm = 0
        call = lambda i: ext.dec(cfg, x[i % 8], y)
    else:
        raise SystemExit(f"unknown --micro {kind}")
    iters = args.iters
    for i in range(min(3, iters)):
        call(i)
    torch.cuda.synchronize()
    us = None
    if iters > 3:
        n = min(iters, 32)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            call(0)
            s.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=s):
                for i in range(n):
                    call(i)
            gr.replay()
            s.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(1, iters // n)
            a.record(s)
            for _ in range(reps):
                gr.replay()
            b.record(s)
            s.synchronize()
        us = a.elapsed_time(b) * 1e3 / (reps * n)
    link = fetch_bytes(N, K, args.k_chunk) if "dec" in kind else 0
    print(json.dumps({"micro": kind, "N": N, "K": K, "k_chunk": args.k_chunk if "dec" in kind else None,
                      "n_tb": args.n_tb if "dec" in kind else None, "us_per_launch": us, "distinct_weight_sets": ncopy,
                      "hbm_algorithmic_bytes": hbm, "hbm_gbs": (hbm / us / 1e3) if us and hbm else None,
                      "host_link_bytes": link, "host_link_gbs": (link / us / 1e3) if us and link else None}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--k-chunk", type=int, default=32)
    ap.add_argument("--n-tb", type=int, default=int(os.environ.get("DECDEC_BENCH_NTB", "96")))
    ap.add_argument("--layers", type=int, default=0, help="use fewer layers (profiling captures only)")
    ap.add_argument("--tuned", default=None, help="extra operating point 'n_tb:k_wqkv,k_wo,k_w1w3,k_w2' ('' = skip; default: the tuner's 5 %% result for the model, single GPU only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--resident-n-tb", type=int, default=32, help="thread-block budget of the residual-in-HBM operating point")
    ap.add_argument("--no-resident", action="store_true",
                    help="skip the extra operating point with the residual held in HBM instead of pinned host memory")
    ap.add_argument("--allreduce", default="nccl", choices=["push", "nccl"],
                    help="multi-GPU: exchange of the row-parallel outputs (push = one-shot kernel over NVLink peer memory)")
    ap.add_argument("--micro", default="", help="single entry point: lutgemm | dec_lutgemm | anyprec | dec_anyprec | sqllm | dec")
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    if args.micro:
        return run_micro(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    import torch
    import decdec_ext as ext   # the drop-in module: torch shim -> C ABI -> CUDA kernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    tp = world
    allreduce = None
    if dist is not None:
        if args.allreduce == "push":
            from decdec_b200.tp import PushAllReduce
            allreduce = PushAllReduce(max(MODELS[args.model][1], 1024))
        else:
            allreduce = dist.all_reduce

    model, ctx, _keep = build_model(args, torch, ext, dev, rank, tp)
    widths, in_sets = make_inputs(torch, model, dev)
    if dist is not None:
        # ranks finish their set-up seconds apart; the push exchange waits for a peer for about a second only
        dist.barrier()
        torch.cuda.synchronize()
    xbuf = {k: torch.zeros(1, 1, k, dtype=torch.float16, device=dev) for k in widths}
    pinned_in = [{k: v.pin_memory() for k, v in s.items()} for s in in_sets]
    out_host = torch.zeros(1, 1, model[0][-1]["n"], dtype=torch.float16).pin_memory()

    def token(on: bool):
        """All quantized linears of one token.  Inputs come from fixed activation buffers (attention,
        norms and the element-wise glue between the linears are not part of the measured path)."""
        _keep[2].zero_()
        for layer in model:
            for p in layer:
                if on:
                    ext.dec_lutgemm(p["cfg"], xbuf[p["k"]], p["y"], p["qw"], p["alpha"], p["qb"], BITS, GROUP)
                else:
                    ext.lutgemm_gemv(xbuf[p["k"]], p["y"], p["qw"], p["alpha"], p["qb"], BITS, GROUP)
                if p["par"] == "row" and allreduce is not None:
                    allreduce(p["y"])

    def load_inputs(i):
        for k in widths:
            xbuf[k].copy_(pinned_in[i % len(pinned_in)][k], non_blocking=True)

    # warm-up outside capture (allocates the library workspace), then capture one token per mode
    stream = torch.cuda.Stream()
    graphs = {}
    with torch.cuda.stream(stream):
        load_inputs(0)
        for on in (True, False):
            token(on)
        stream.synchronize()
        for on in (True, False):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                token(on)
            graphs[on] = g
        # extra operating point: per-projection k_chunk and a smaller thread-block budget.  The configs are
        # re-pointed in place (launch arguments are baked into the graphs captured above).
        tuned = args.tuned if args.tuned is not None else (TUNED_5PCT.get(args.model, "") if world == 1 else "")
        tuned_cfg = None
        if tuned:
            n_tb_t, ks = tuned.split(":")
            ks = [int(v) for v in ks.split(",")]
            tuned_cfg = {"n_tb": int(n_tb_t), "k_chunk": dict(zip([p["name"] for p in model[0]], ks))}
            ctx_t = ext.create_dec_context(int(n_tb_t), _keep[0], _keep[1])
            for layer in model:
                for p, kc in zip(layer, ks):
                    ext.update_dec_config(p["cfg"], ctx_t, kc)
            token(True)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                token(True)
            graphs["tuned"] = g
        # extra operating point: the same compensation with the residual resident in HBM (3.5 GB for this model, which a
        # 180 GB part can afford) - what is left of the cost once the host link is out of the picture
        if world == 1 and not args.no_resident:
            dev_cfgs = []
            ctx_r = ext.create_dec_context(args.resident_n_tb, _keep[0], _keep[1])
            for layer in model:
                for p in layer:
                    q, sc, thr = _keep[3][p["name"]]
                    dev_cfgs.append(ext.create_dec_config(ctx_r, args.k_chunk, q.to(dev), sc, thr))

            def token_resident():
                _keep[2].zero_()
                i = 0
                for layer in model:
                    for p in layer:
                        ext.dec_lutgemm(dev_cfgs[i], xbuf[p["k"]], p["y"], p["qw"], p["alpha"], p["qb"], BITS, GROUP)
                        i += 1

            token_resident()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                token_resident()
            graphs["resident"] = g
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(on: bool, steps: int, warm: int, e2e: bool):
        """K graph replays timed with CUDA events on the launching stream; max over ranks."""
        with torch.cuda.stream(stream):
            for i in range(warm):
                load_inputs(i)
                graphs[on].replay()
            stream.synchronize()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if not e2e:
                # inputs already resident: rotate device-side activation sets without host traffic
                dev_sets = [{k: v.to(dev) for k, v in s.items()} for s in in_sets]
                stream.synchronize()
                a.record(stream)
                for i in range(steps):
                    for k in widths:
                        xbuf[k].copy_(dev_sets[i % len(dev_sets)][k], non_blocking=True)
                    graphs[on].replay()
                b.record(stream)
            else:
                a.record(stream)
                for i in range(steps):
                    load_inputs(i)                                     # H2D from pinned host memory
                    graphs[on].replay()
                    out_host.copy_(model[-1][-1]["y"], non_blocking=True)   # D2H of the step's result
                    stream.synchronize()
                b.record(stream)
            stream.synchronize()
        barrier()
        ms = a.elapsed_time(b)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local) if rank == 0 else None
    ms_on = timed(True, args.steps, args.warmup, e2e=False)
    ms_off = timed(False, args.steps, args.warmup, e2e=False)
    ms_e2e = timed(True, args.steps, args.warmup, e2e=True)
    ms_tuned = timed("tuned", args.steps, args.warmup, e2e=False) if "tuned" in graphs else None
    ms_res = timed("resident", args.steps, args.warmup, e2e=False) if "resident" in graphs else None
    clocks = sampler.stop() if sampler else {}      # sampled across all timed regions of the run

    n_layers = len(model)
    calls = n_layers * len(model[0])
    hbm_bytes = n_layers * sum(gemv_bytes(p["n"], p["k"]) for p in model[0])
    link_bytes = n_layers * sum(fetch_bytes(p["n"], p["k"], args.k_chunk) for p in model[0])
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
    gemv_gbs = hbm_bytes / (ms_off * 1e-3) / 1e9
    link_gbs = link_bytes / (ms_on * 1e-3) / 1e9
    h2d = sum(2 * k for k in widths)
    d2h = out_host.numel() * 2

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline:
            try:
                torch.set_num_threads(len(os.sched_getaffinity(0)))      # torchrun pins ranks to one OpenMP thread
            except (AttributeError, RuntimeError):
                pass
            ts, desc, scale = cpu_sample(args.model, args.k_chunk, 5, 1)
            cpu = {"value": len(ts) / (sum(ts) * scale), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": desc + f"; 5 repetitions, scaled x{scale:.0f} to a token"}
        line = {
            "metric": "batch-1 decode tok/s (DecDEC on)", "value": 1e3 / ms_on, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_on, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 in/out, f32 accumulate", "data": "synthetic",
            "config": workload_config(args),
            "decdec_off": {"value": 1e3 / ms_off, "unit": "tokens/s", "ms_per_step": ms_off,
                           "slowdown_on_vs_off": ms_on / ms_off},
            "roofline": {"bound": "hbm", "achieved": gemv_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gemv_gbs / hbm_peak,
                         # ncu capture of the w1w3 launch (profiles/): dram read+write 51.73 MB for 51.50 MB algorithmic
                         "traffic": NCU_TRAFFIC_RATIO * hbm_bytes / calls, "kernel": "k_bcq_pipe<fp16,3> (GEMV role, compensation off)", "launches_per_step": calls,
                         "algorithmic_bytes_per_step": hbm_bytes, "peak_source": peak_src, "frac_of_spec_8000": gemv_gbs / 8000.0,
                         "note": "bytes of all GEMV launches of a step / event-timed duration of the step with compensation off"},
            "host_link": {"achieved": link_gbs, "unit": "GB/s", "peak_spec": 64.0, "frac_of_spec": link_gbs / 64.0,
                          "measured_h2d_memcpy_peak": 55.4, "fetched_bytes_per_step": link_bytes,
                          "note": "residual bytes of a step / event-timed duration of the step with compensation on (lower bound of the link rate)"},
            "e2e": {"value": 1e3 / ms_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e},
            "gpu_launches": calls * args.steps,
            "clocks": clocks,
        }
        if ms_tuned is not None:
            tb = n_layers * sum(fetch_bytes(p["n"], p["k"], tuned_cfg["k_chunk"][p["name"]]) for p in model[0])
            line["tuned"] = {"value": 1e3 / ms_tuned, "unit": "tokens/s", "ms_per_step": ms_tuned,
                             "slowdown_vs_off": ms_tuned / ms_off, "n_tb": tuned_cfg["n_tb"], "k_chunk": tuned_cfg["k_chunk"],
                             "fetched_bytes_per_step": tb,
                             "note": "operating point of the (n_tb, k_chunk) tuner for a 5 % layer slowdown budget"}
        if ms_res is not None:
            line["residual_in_hbm"] = {"value": 1e3 / ms_res, "unit": "tokens/s", "ms_per_step": ms_res, "slowdown_vs_off": ms_res / ms_off,
                                       "k_chunk": args.k_chunk, "n_tb": args.resident_n_tb, "hbm_bytes_for_residual": int(link_bytes / args.k_chunk * 1024) if args.k_chunk else 0,
                                       "note": "same launches with q_residual in device memory (create_dec_config accepts a CUDA tensor); not the reference's operating mode"}
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if dist is not None and args.allreduce == "push":
        allreduce.check()          # raises if any wait for a peer ever ran out
    if dist is not None:
        # graphs that captured NCCL work must go before the communicator; leave without running
        # interpreter-exit destructors, which can block on a communicator with captured collectives
        graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
