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
row-parallel wo/w2 whose partial outputs are summed by one exchange per layer (a one-shot push kernel over
NVLink peer memory by default, ncclAllReduce with --allreduce nccl); every rank fetches its own residual shard
over its own host link.  The line also carries `config4`: the same measurement on Llama-3-70B shapes, the
configuration that needs tensor parallelism.
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
# (n_tb, k_chunk of wqkv, wo, w1w3, w2) and the layer-slowdown budget in percent it was searched for: operating point
# chosen by `python -m decdec_b200.tuner --target-slowdown 15` on one B200, timed as an extra operating point beside
# k_chunk = 32.  (For a 5 % budget the same search returns no compensation at all: a fused launch costs at least
# 1 us more than the GEMV alone on the widest projection, and a layer of GEMVs takes 35.6 us.)
TUNED_POINT = {"llama3-8b": ("32:0,0,5,3", 15)}
# DRAM bytes read + written by one launch of the GEMV kernel on the 28672x4096 layer under ncu, divided by the
# algorithmic bytes of that launch (51.73 MB / 51.50 MB): every weight byte is read once, so the traffic of other
# launches is scaled from their algorithmic bytes with this ratio
NCU_TRAFFIC_RATIO = 51.73 / 51.50


def projections(model: str, tp: int = 1, rank: int = 0):
    """One layer's projections as dicts {name, n, k, par, n_full, n0}: n x k is this rank's GEMV, n_full the width
    of the layer's output vector and n0 where this rank's outputs start in it.  Fused wqkv / w1w3 as in the
    reference model (end-to-end/model.py:266,331); column-parallel wqkv / w1w3, row-parallel wo / w2 cut at
    selection-chunk boundaries (decdec_b200.tp.row_plan)."""
    from decdec_b200 import tp as tpl
    _, d, hq, hkv, hd, ffn = MODELS[model]
    qkv = (hq + 2 * hkv) * hd

    def col(name, n, k):
        a, b = tpl.split_even(n, tp, 128 if n % (128 * tp) == 0 else 32)[rank]
        return dict(name=name, n=b - a, k=k, par="col", n_full=b - a, n0=0)

    def row(name, n, k):
        k0, k1, n0, n1 = tpl.row_plan(k, n, tp)[rank]
        return dict(name=name, n=n1 - n0, k=k1 - k0, par="row", n_full=n, n0=n0)

    return [col("wqkv", qkv, d), row("wo", d, d), col("w1w3", 2 * ffn, d), row("w2", d, ffn)]


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

CPU_ROWS = 2048      # outputs per projection in the timed CPU sample (cost is linear in the outputs)


def cpu_layer_sample(model: str, k_chunk: int):
    """Tensors of ONE layer for the CPU path: the four projection shapes with at most CPU_ROWS outputs each.
    Returns [(name, n_full, n_sample, k, tensors)]."""
    import torch
    out = []
    g = torch.Generator().manual_seed(0)
    for p in projections(model):
        n, k = p["n"], p["k"]
        ns = min(n, CPU_ROWS)
        qw = torch.randint(-2**31, 2**31 - 1, (k // 32, BITS, ns), dtype=torch.int32, generator=g)
        alpha = (torch.rand(k // GROUP, BITS, ns, generator=g) * 0.01).half()
        qb = ((torch.rand(k // GROUP, ns, generator=g) - 0.5) * 0.01).half()
        cs = torch.randint(-2**31, 2**31 - 1, (k, ns // 8), dtype=torch.int32, generator=g)
        sc = (torch.rand(ns, generator=g) * 1e-3).half()
        x = torch.randn(k, generator=g)
        out.append((p["name"], n, ns, k, (qw, alpha, qb, cs, sc, x)))
    return out


def cpu_time_layer(sample, k_chunk: int, predequant):
    """Seconds for one decode step of one layer on the CPU, every projection scaled from its sampled outputs to its
    full width.  predequant = list of (W^T, R^T) prepared beforehand, or None for the reference modules' behaviour
    (dequantise at every call, end-to-end/LUTGEMMLinear.py:41-82)."""
    from oracle import forward as ofw
    total, raw = 0.0, 0.0
    for i, (_, n, ns, k, (qw, alpha, qb, cs, sc, x)) in enumerate(sample):
        t0 = time.perf_counter()
        if predequant is None:
            wt = ofw.torch_bcq_dequant(qw, alpha, qb, GROUP)
            rt = ofw.torch_unpack_residual(cs, sc) if k_chunk else None
        else:
            wt, rt = predequant[i]
        ofw.cpu_reference_linear(x, wt, rt, k_chunk)
        dt = time.perf_counter() - t0
        raw += dt
        total += dt * (n / ns)
    return total, raw


def cpu_baseline(model: str, k_chunk: int, reps: int, warm: int):
    """Median per-token time of the reference's CPU math: BCQ dequant + residual unpack + exact per-chunk top-k +
    two mat-vecs (oracle/forward.py), both dequantising at every call and with the dense matrices prepared once."""
    import torch
    from oracle import forward as ofw
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))      # torchrun pins its ranks to one OpenMP thread
    except (AttributeError, RuntimeError):
        pass
    layers = MODELS[model][0]
    sample = cpu_layer_sample(model, k_chunk)
    pre = [(ofw.torch_bcq_dequant(t[0], t[1], t[2], GROUP), ofw.torch_unpack_residual(t[3], t[4]) if k_chunk else None)
           for *_, t in sample]
    for _ in range(warm):
        cpu_time_layer(sample, k_chunk, None)
        cpu_time_layer(sample, k_chunk, pre)
    every_raw = [cpu_time_layer(sample, k_chunk, None) for _ in range(reps)]
    once_raw = [cpu_time_layer(sample, k_chunk, pre) for _ in range(reps)]
    every, once = [t for t, _ in every_raw], [t for t, _ in once_raw]
    desc = (f"one layer of {model} (wqkv, wo, w1w3, w2), {CPU_ROWS} of each projection's outputs timed and scaled to its width, "
            f"then x{layers} layers: BCQ dequant + residual unpack + per-chunk top-k + 2 matvec in fp32; median of {reps} repetitions; "
            "the token time is extrapolated from this sample, not run in full")
    return {"s_per_token_dequant_every_call": statistics.median(every) * layers,
            "s_per_token_predequantised": statistics.median(once) * layers,
            "measured_wall_s": sum(r for _, r in every_raw), "cores": torch.get_num_threads(), "sample": desc}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_baseline(args.model, args.k_chunk, max(args.steps, 10), max(1, args.warmup))
    tok_s = 1.0 / r["s_per_token_dequant_every_call"]
    line = {
        "impl": "reference", "metric": "batch-1 decode tok/s (DecDEC on)", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * r["s_per_token_dequant_every_call"],
        "measured_wall_s": r["measured_wall_s"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"],
                         "predequantised_tokens_per_s": 1.0 / r["s_per_token_predequantised"]},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(args, model=None):
    model = model or args.model
    layers, d, hq, hkv, hd, ffn = MODELS[model]
    return {"workload": f"{model} decode hot path: {layers} layers x (wqkv, wo, w1w3, w2) fused GEMV+DEC, "
                        f"{BITS}-bit binary-coded group-{GROUP} weights, 4-bit residual rows in pinned host memory; "
                        "linears only (attention, norms and lm_head are not part of the measured path)",
            "k_chunk": args.k_chunk, "n_tb": args.n_tb, "batch": 1,
            "parallelism": (f"tp{args.gpus}, row-parallel outputs summed by " + ("a one-shot push kernel over NVLink peer memory"
                            if args.allreduce == "push" else "ncclAllReduce")) if args.gpus > 1 else "single",
            "cache": "inputs larger than L2 (every layer has its own weights and residual; no L2 flush needed)"}


# --------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------

class Workload:
    """The quantized linears of one model on this rank: random packed tensors of the model's shapes (one storage per
    layer and projection), their compensation configs, CUDA graphs of one token per mode, and event timing."""

    def __init__(self, env, model_name, k_chunk, n_tb, layers=0, resident=False):
        torch, ext = env["torch"], env["ext"]
        self.env, self.name, self.k_chunk = env, model_name, k_chunk
        dev, rank, tp = env["dev"], env["rank"], env["world"]
        n_layers = layers or MODELS[model_name][0]
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        gc = torch.Generator().manual_seed(99 + rank)
        self.rows = torch.zeros(32 * 1024, dtype=torch.int32, device=dev)
        self.acts = torch.zeros(32 * 1024, dtype=torch.float16, device=dev)
        self.ctx = ext.create_dec_context(n_tb, self.rows, self.acts)
        proj = projections(model_name, tp, rank)
        # one random residual per projection shape on the host; every config pins its own copy
        self.host_res = {}
        for p in proj:
            n, k = p["n"], p["k"]
            self.host_res[p["name"]] = (torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=gc),
                                        (torch.rand(n, generator=gc) * 1e-3 + 1e-4).half(),
                                        torch.sort(torch.randn(k, generator=gc).abs() * 3, descending=True).values.half())
        self.model = []
        for _ in range(n_layers):
            layer = []
            for p in proj:
                n, k = p["n"], p["k"]
                q, sc, thr = self.host_res[p["name"]]
                e = dict(p)
                e["qw"] = torch.randint(-2**31, 2**31 - 1, (k // 32, BITS, n), dtype=torch.int32, device=dev, generator=g)
                e["alpha"] = (torch.rand(k // GROUP, BITS, n, device=dev, generator=g) * 0.01).half()
                e["qb"] = ((torch.rand(k // GROUP, n, device=dev, generator=g) - 0.5) * 0.01).half()
                e["cfg"] = ext.create_dec_config(self.ctx, k_chunk, q.to(dev) if resident else q, sc, thr)
                e["thr"] = thr
                layer.append(e)
            self.model.append(layer)
        # all layer outputs live in one buffer that is cleared once per token (the entry points accumulate into their
        # output; the reference's modules clear each output with its own kernel before every call).  A row-parallel
        # rank writes its partial sums into its range of the layer's full-width vector, which is then summed over ranks.
        total = sum(p["n_full"] for layer in self.model for p in layer)
        self.ybuf = torch.zeros(total, dtype=torch.float16, device=dev)
        off = 0
        for layer in self.model:
            for p in layer:
                p["y_full"] = self.ybuf[off:off + p["n_full"]]
                p["y"] = p["y_full"][p["n0"]:p["n0"] + p["n"]].view(1, 1, p["n"])
                off += p["n_full"]
        # activation sets (N(0,1) with 1% x20 outliers) per input width, rotated between steps so that the selected
        # rows change from token to token
        gi = torch.Generator().manual_seed(7)
        self.widths = sorted({p["k"] for p in self.model[0]})
        self.in_sets = []
        for _ in range(4):
            st = {}
            for k in self.widths:
                x = torch.randn(k, generator=gi)
                idx = torch.randperm(k, generator=gi)[: max(1, k // 100)]
                x[idx] *= 20
                st[k] = x.half().reshape(1, 1, k)
            self.in_sets.append(st)
        self.xbuf = {k: torch.zeros(1, 1, k, dtype=torch.float16, device=dev) for k in self.widths}
        self.pinned_in = [{k: v.pin_memory() for k, v in st.items()} for st in self.in_sets]
        self.dev_sets = [{k: v.to(dev) for k, v in st.items()} for st in self.in_sets]
        self.out_host = torch.zeros(1, 1, self.model[-1][-1]["n"], dtype=torch.float16).pin_memory()
        self.stream = torch.cuda.Stream()
        self.graphs = {}

    # ---- one token ------------------------------------------------------------------------------------------
    def token(self, mode):
        """All quantized linears of one token.  mode: "on" (fused GEMV + compensation), "off" (GEMV only),
        "gemv" (GEMV only and no exchange between ranks), "xchg" (the exchanges alone).  Inputs come from fixed
        activation buffers (the glue between the linears is not part of the measured path)."""
        ext, allreduce = self.env["ext"], self.env["allreduce"]
        self.ybuf.zero_()
        for layer in self.model:
            for p in layer:
                if mode == "on":
                    ext.dec_lutgemm(p["cfg"], self.xbuf[p["k"]], p["y"], p["qw"], p["alpha"], p["qb"], BITS, GROUP)
                elif mode in ("off", "gemv"):
                    ext.lutgemm_gemv(self.xbuf[p["k"]], p["y"], p["qw"], p["alpha"], p["qb"], BITS, GROUP)
                if p["par"] == "row" and allreduce is not None and mode != "gemv":
                    allreduce(p["y_full"])

    def load_inputs(self, i):
        for k in self.widths:
            self.xbuf[k].copy_(self.pinned_in[i % len(self.pinned_in)][k], non_blocking=True)

    def capture(self, key, mode):
        torch = self.env["torch"]
        self.barrier()                       # ranks build their tensors at different speeds; the exchange's wait for a
                                             # peer is bounded (about a second), so they enter the first token together
        with torch.cuda.stream(self.stream):
            self.load_inputs(0)
            self.token(mode)                 # outside capture: allocates the library workspace of this stream
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                self.token(mode)
            self.graphs[key] = g
        torch.cuda.synchronize()

    def barrier(self):
        if self.env["dist"] is not None:
            self.env["dist"].barrier()
        self.env["torch"].cuda.synchronize()

    def retune(self, n_tb, k_chunks):
        """Re-point every config at a context with another thread-block budget and per-projection k_chunk (launch
        arguments are baked into graphs already captured, so this only affects later captures)."""
        ext = self.env["ext"]
        ctx = ext.create_dec_context(n_tb, self.rows, self.acts)
        for layer in self.model:
            for p, kc in zip(layer, k_chunks):
                ext.update_dec_config(p["cfg"], ctx, kc)
        return ctx

    def timed(self, key, steps, warm, e2e=False):
        """`steps` graph replays timed with CUDA events on the launching stream; max over ranks."""
        torch, dist, dev = self.env["torch"], self.env["dist"], self.env["dev"]
        g = self.graphs[key]
        barrier = self.barrier
        barrier()
        with torch.cuda.stream(self.stream):
            for i in range(warm):
                self.load_inputs(i)
                g.replay()
            self.stream.synchronize()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if not e2e:
                # inputs already resident: rotate device-side activation sets without host traffic
                a.record(self.stream)
                for i in range(steps):
                    for k in self.widths:
                        self.xbuf[k].copy_(self.dev_sets[i % len(self.dev_sets)][k], non_blocking=True)
                    g.replay()
                b.record(self.stream)
            else:
                a.record(self.stream)
                for i in range(steps):
                    self.load_inputs(i)                                          # H2D from pinned host memory
                    g.replay()
                    self.out_host.copy_(self.model[-1][-1]["y"], non_blocking=True)   # D2H of the step's result
                    self.stream.synchronize()
                b.record(self.stream)
            self.stream.synchronize()
        barrier()
        ms = a.elapsed_time(b)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # ---- bytes ----------------------------------------------------------------------------------------------
    def hbm_bytes(self):
        return len(self.model) * sum(gemv_bytes(p["n"], p["k"]) for p in self.model[0])

    def link_bytes(self, k_chunks=None):
        ks = k_chunks or [self.k_chunk] * len(self.model[0])
        return len(self.model) * sum(fetch_bytes(p["n"], p["k"], kc) for p, kc in zip(self.model[0], ks))

    def calls(self):
        return len(self.model) * len(self.model[0])

    def exchanges(self):
        return len(self.model) * sum(1 for p in self.model[0] if p["par"] == "row")

    def close(self):
        ext = self.env["ext"]
        self.graphs.clear()
        self.env["torch"].cuda.synchronize()
        for layer in self.model:
            for p in layer:
                ext.destroy_dec_config(p["cfg"])
        self.model = []


def all_ranks_sum(env, v):
    if env["dist"] is None:
        return v
    t = env["torch"].tensor([float(v)], device=env["dev"], dtype=env["torch"].float64)
    env["dist"].all_reduce(t)
    return float(t.item())


def measure(env, args, model_name, layers, steps, warm, extras):
    """on / off / GEMV-only / exchange timings of one model; `extras` adds e2e, the tuned and the resident operating points."""
    world = env["world"]
    n_tb = args.n_tb if world == 1 else max(16, args.n_tb // world)     # the compensation budget shrinks with the shard
    w = Workload(env, model_name, args.k_chunk, n_tb, layers)
    out = {"n_tb": n_tb, "layers": len(w.model)}
    w.capture("on", "on")
    w.capture("off", "off")
    out["ms_on"] = w.timed("on", steps, warm)
    out["ms_off"] = w.timed("off", steps, warm)
    if world > 1:
        w.capture("gemv", "gemv")
        w.capture("xchg", "xchg")
        out["ms_gemv"] = w.timed("gemv", steps, warm)
        out["ms_xchg"] = w.timed("xchg", steps, warm)
    else:
        out["ms_gemv"] = out["ms_off"]
    if extras:
        out["ms_e2e"] = w.timed("on", steps, warm, e2e=True)
        out["h2d"] = sum(2 * k for k in w.widths)
        out["d2h"] = w.out_host.numel() * 2
    out["hbm_bytes"] = all_ranks_sum(env, w.hbm_bytes())                  # all ranks' GEMV bytes of a step
    out["link_bytes"] = all_ranks_sum(env, w.link_bytes())
    out["link_bytes_rank"] = w.link_bytes()
    out["calls"] = w.calls()
    out["exchanges"] = w.exchanges() if world > 1 else 0
    tuned = args.tuned if args.tuned is not None else (TUNED_POINT.get(model_name, ("", 0))[0] if world == 1 else "")
    if extras and tuned:
        n_tb_t, ks = tuned.split(":")
        ks = [int(v) for v in ks.split(",")]
        w.retune(int(n_tb_t), ks)
        w.capture("tuned", "on")
        out["tuned"] = {"ms": w.timed("tuned", steps, warm), "n_tb": int(n_tb_t),
                        "k_chunk": dict(zip([p["name"] for p in w.model[0]], ks)), "bytes": w.link_bytes(ks)}
    w.close()
    del w
    env["torch"].cuda.empty_cache()
    if extras and world == 1 and not args.no_resident:
        # the same compensation with the residual resident in HBM (3.5 GB for Llama-3-8B, which a 180 GB part can
        # afford): what is left of the cost once the host link is out of the picture
        wr = Workload(env, model_name, args.k_chunk, args.resident_n_tb, layers, resident=True)
        wr.capture("on", "on")
        out["resident"] = {"ms": wr.timed("on", steps, warm), "n_tb": args.resident_n_tb}
        wr.close()
        del wr
        env["torch"].cuda.empty_cache()
    return out


def run_micro(args):
    """One entry point on one layer shape: `--micro KIND --n N --k K [--k-chunk C --n-tb T --iters I]`.
    Launches rotate over enough distinct weight tensors to exceed L2 (cache-cold), are captured in a CUDA
    graph and timed with CUDA events; prints one JSON line (us per launch, algorithmic GB/s).  Also the
    command used for single-kernel ncu captures."""
    import torch
    import decdec_ext as ext
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    N, K, kind = args.n, args.k, args.micro
    bits = args.bits
    g = torch.Generator(device=dev).manual_seed(1)
    wbytes = bits * N * K / 8
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
        w = [(ri(K // 32, bits, N), (torch.rand(K // GROUP, bits, N, device=dev, generator=g) * 0.01).half(),
              ((torch.rand(K // GROUP, N, device=dev, generator=g) - 0.5) * 0.01).half()) for _ in range(ncopy)]
        hbm = gemv_bytes(N, K)
        if kind == "lutgemm":
            call = lambda i: ext.lutgemm_gemv(x[i % 8], y, *w[i % ncopy], bits, GROUP)
        else:
            call = lambda i: ext.dec_lutgemm(cfg, x[i % 8], y, *w[i % ncopy], bits, GROUP)
    elif "anyprec" in kind:
        w = [(ri(bits, N, K // 32), (torch.randn(N, 2 ** bits, device=dev, generator=g) * 0.02).half()) for _ in range(ncopy)]
        hbm = bits * N * K / 8 + N * 2 ** bits * 2 + 2 * K + 4 * N
        if kind == "anyprec":
            call = lambda i: ext.anyprec_gemv(x[i % 8], y, *w[i % ncopy], bits)
        else:
            call = lambda i: ext.dec_anyprec(cfg, x[i % 8], y, *w[i % ncopy], bits)
    elif kind == "sqllm":
        w = [(ri(K * bits // 32, N), (torch.randn(N, 2 ** bits, device=dev, generator=g) * 0.02).half()) for _ in range(ncopy)]
        hbm = bits * N * K / 8 + N * 2 ** bits * 2 + 2 * K + 4 * N
        call = lambda i: ext.sqllm_gemv(x[i % 8], y, *w[i % ncopy], bits)
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
    ap.add_argument("--tuned", default=None, help="extra operating point 'n_tb:k_wqkv,k_wo,k_w1w3,k_w2' ('' = skip; default: the tuner's result for the model, single GPU only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--resident-n-tb", type=int, default=32, help="thread-block budget of the residual-in-HBM operating point")
    ap.add_argument("--no-resident", action="store_true",
                    help="skip the extra operating point with the residual held in HBM instead of pinned host memory")
    ap.add_argument("--allreduce", default="push", choices=["push", "nccl"],
                    help="multi-GPU: exchange of the row-parallel outputs (push = one-shot kernel over NVLink peer memory)")
    ap.add_argument("--no-config4", action="store_true", help="skip the Llama-3-70B-shaped measurement")
    ap.add_argument("--config4-layers", type=int, default=0, help="layers of the Llama-3-70B-shaped model (0 = all 80)")
    ap.add_argument("--bits", type=int, default=BITS, help="bit width of the --micro entry point")
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
    allreduce = None
    if dist is not None:
        if args.allreduce == "push":
            from decdec_b200.tp import PushAllReduce
            allreduce = PushAllReduce(max(max(m[1] for m in MODELS.values()), 1024))
        else:
            allreduce = dist.all_reduce
    env = dict(torch=torch, ext=ext, dev=dev, rank=rank, world=world, dist=dist, allreduce=allreduce)
    if dist is not None:
        # ranks finish their set-up seconds apart; the push exchange waits for a peer for about a second only
        dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    r = measure(env, args, args.model, args.layers, args.steps, args.warmup, extras=True)
    c4 = None
    if not args.no_config4 and args.model != "llama3-70b":
        try:
            c4 = measure(env, args, "llama3-70b", args.config4_layers, max(3, args.steps // 2), 3, extras=False)
        except RuntimeError as e:      # e.g. the pinned host memory for 80 layers of residuals could not be had
            c4 = {"unavailable": str(e).splitlines()[0][:200]}
    clocks = sampler.stop() if sampler else {}      # sampled across all timed regions of the run

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"

    def roofline(m):
        gbs = m["hbm_bytes"] / (m["ms_gemv"] * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": hbm_peak * world, "unit": "GB/s", "frac": gbs / (hbm_peak * world),
                "traffic": NCU_TRAFFIC_RATIO * m["hbm_bytes"] / (m["calls"] * world),
                "traffic_note": "scaled from the algorithmic bytes with the DRAM/algorithmic ratio of one profiled launch (28672x4096), not measured in this run",
                "kernel": "k_bcq_pipe<fp16,3> (GEMV role, compensation off, no exchange between ranks)",
                "launches_per_step": m["calls"], "algorithmic_bytes_per_step": m["hbm_bytes"], "peak_source": peak_src + (f" x {world} GPUs" if world > 1 else ""),
                "frac_of_spec_8000": gbs / (8000.0 * world),
                "note": "bytes of all GEMV launches of a step (all ranks) / event-timed duration of the GEMV-only step"}

    def summary(m):
        d = {"on": {"value": 1e3 / m["ms_on"], "unit": "tokens/s", "ms_per_step": m["ms_on"]},
             "off": {"value": 1e3 / m["ms_off"], "unit": "tokens/s", "ms_per_step": m["ms_off"]},
             "slowdown_on_vs_off": m["ms_on"] / m["ms_off"], "layers": m["layers"], "n_tb": m["n_tb"],
             "roofline": roofline(m),
             "host_link": {"achieved_all_ranks": m["link_bytes"] / (m["ms_on"] * 1e-3) / 1e9,
                           "achieved_per_rank": m["link_bytes_rank"] / (m["ms_on"] * 1e-3) / 1e9, "unit": "GB/s", "peak_spec_per_rank": 64.0,
                           "fetched_bytes_per_step": m["link_bytes"]}}
        if world > 1:
            d["exchange"] = {"kind": args.allreduce, "calls_per_step": m["exchanges"], "us_per_call": 1e3 * m["ms_xchg"] / max(1, m["exchanges"]),
                             "ms_per_step_alone": m["ms_xchg"], "gemv_only_ms_per_step": m["ms_gemv"]}
        return d

    if rank == 0:
        ms_on, ms_off = r["ms_on"], r["ms_off"]
        link_gbs = r["link_bytes"] / (ms_on * 1e-3) / 1e9
        line = {
            "metric": "batch-1 decode tok/s (DecDEC on)", "value": 1e3 / ms_on, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_on, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 in/out, f32 accumulate", "data": "synthetic",
            "config": workload_config(args),
            "decdec_off": {"value": 1e3 / ms_off, "unit": "tokens/s", "ms_per_step": ms_off, "slowdown_on_vs_off": ms_on / ms_off},
            "roofline": roofline(r),
            "host_link": {"achieved": link_gbs, "unit": "GB/s", "peak_spec": 64.0 * world, "frac_of_spec": link_gbs / (64.0 * world),
                          "per_rank": r["link_bytes_rank"] / (ms_on * 1e-3) / 1e9,
                          "measured_h2d_memcpy_peak": 55.4, "fetched_bytes_per_step": r["link_bytes"],
                          "note": "residual bytes of a step (all ranks) / event-timed duration of the step with compensation on (lower bound of the link rate)"},
            "e2e": {"value": 1e3 / r["ms_e2e"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                    "ms_per_step": r["ms_e2e"]},
            "gpu_launches": (r["calls"] + r["exchanges"] * (1 if args.allreduce == "push" else 0)) * args.steps,
            "clocks": clocks,
        }
        if world > 1:
            line["exchange"] = summary(r)["exchange"]
        if "tuned" in r:
            t = r["tuned"]
            line["tuned"] = {"value": 1e3 / t["ms"], "unit": "tokens/s", "ms_per_step": t["ms"], "slowdown_vs_off": t["ms"] / ms_off,
                             "n_tb": t["n_tb"], "k_chunk": t["k_chunk"], "fetched_bytes_per_step": t["bytes"],
                             "note": ("operating point of the (n_tb, k_chunk) tuner for a %d %% layer slowdown budget (its 5 %% search returns no compensation)"
                                      % TUNED_POINT.get(args.model, ("", 0))[1]) if args.tuned is None else "operating point given with --tuned"}
        if "resident" in r:
            t = r["resident"]
            line["residual_in_hbm"] = {"value": 1e3 / t["ms"], "unit": "tokens/s", "ms_per_step": t["ms"], "slowdown_vs_off": t["ms"] / ms_off,
                                       "k_chunk": args.k_chunk, "n_tb": t["n_tb"],
                                       "hbm_bytes_for_residual": int(r["link_bytes"] / args.k_chunk * 1024) if args.k_chunk else 0,
                                       "note": "same launches with q_residual in device memory (create_dec_config accepts a CUDA tensor); not the reference's operating mode"}
        if c4 is not None:
            line["config4"] = c4 if "unavailable" in c4 else dict(summary(c4), workload=workload_config(args, "llama3-70b")["workload"])
        if not args.no_cpu_baseline:
            cb = cpu_baseline(args.model, args.k_chunk, 10, 1)
            line["cpu_baseline"] = {"value": 1.0 / cb["s_per_token_dequant_every_call"], "unit": "tokens/s", "cores": cb["cores"], "kind": "port",
                                    "sample": cb["sample"], "predequantised_tokens_per_s": 1.0 / cb["s_per_token_predequantised"]}
        print(json.dumps(line), flush=True)
    if dist is not None and args.allreduce == "push":
        allreduce.check()          # raises if any wait for a peer ever ran out
    if dist is not None:
        # graphs that captured NCCL work must go before the communicator; leave without running
        # interpreter-exit destructors, which can block on a communicator with captured collectives
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
