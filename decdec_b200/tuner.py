"""(n_tb, k_chunk) tuner for the fused GEMV + compensation launches.

Same question as the reference's autotuner (autotuner/tuner.py:128-351): given, per projection of a decoder
layer, the standalone GEMV time and the fused time for a grid of (n_tb, k_chunk), find the thread-block budget
n_tb and the per-projection k_chunk that fetch the most residual rows while the layer (the four projections)
stays within `target_slowdown` x its compensation-off time.  The reference fills the table from an Nsight
Systems trace of a whole model run (autotuner/run_profile.py, nsys_parser.py); here the table comes from CUDA
event timings of graph-replayed launches through the same `decdec_ext` entry points a model would call, so no
profiler is needed.

    python -m decdec_b200.tuner --model llama3-8b --target-slowdown 5            # measure + search + verify
    python -m decdec_b200.tuner --qkv 4096 6144 --o 4096 4096 --gu 4096 28672 --d 14336 4096 --target-slowdown 10

`search()` is pure Python and runs without a GPU; `measure()` / `verify()` need the CUDA extension.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

MODULES = ("qkv", "o", "gu", "d")

# (in_features, out_features) per projection; same table as the reference's autotuner/README.md
MODEL_DIMS = {
    "llama3-8b": {"qkv": (4096, 6144), "o": (4096, 4096), "gu": (4096, 28672), "d": (14336, 4096)},
    "phi3-medium": {"qkv": (5120, 7680), "o": (5120, 5120), "gu": (5120, 35840), "d": (17920, 5120)},
    "llama3-70b": {"qkv": (8192, 10240), "o": (8192, 8192), "gu": (8192, 57344), "d": (28672, 8192)},
}


class TunerRangeError(ValueError):
    """The largest measured k_chunk still fits the target for some n_tb: measure a wider k_chunk range.
    (The reference raises ValueError at the same point, autotuner/tuner.py:219-220.)"""


def estimate_k_chunk(bitwidth: int, hbm_gbs: float, link_gbs: float, residual_bits: int = 4, chunk: int = 1024) -> int:
    """Rows per chunk whose fetch takes as long as streaming the chunk's base weights
    (autotuner/run_profile.py:26-30): bitwidth / (HBM/link) / residual_bits * chunk."""
    return int(bitwidth / (hbm_gbs / link_gbs) / residual_bits * chunk)


def pcie_gbs(gen: int, lanes: int) -> float:
    """Nominal one-direction link bandwidth, autotuner/run_profile.py:26."""
    return (1 / 8) * (2 ** gen) * lanes


# ---------------------------------------------------------------------------------------------------------
# search
# ---------------------------------------------------------------------------------------------------------

def _n_tb_at(times: Mapping[int, Mapping[int, float]], n_max: int) -> Optional[int]:
    ok = [n for n in times if n <= n_max]
    return max(ok) if ok else None


def search(table: Mapping[str, Mapping], target_slowdown: float, log=None) -> dict:
    """Two-phase search of autotuner/tuner.py:128-351.

    table[module] = {"dims": (K, N), "baseline_us": t0, "times_us": {n_tb: {k_chunk: t}}}; module order is the
    order of the mapping.  `target_slowdown` is a ratio (1.05 = 5 % slower than compensation off).

    Phase 1 (global): one k_chunk for all modules and one thread-block budget.  For every integer budget between
    the smallest and largest measured n_tb, each module runs at its largest measured n_tb within the budget; the
    common k_chunk grows from 1 until the layer time exceeds the target.  The budget with the largest k_chunk
    wins, ties go to the lower layer time.  If not even k_chunk = 1 fits, the smallest module (by K*N) is taken
    out of compensation (it then costs its baseline) and the phase repeats.
    Phase 2 (fine-grained): per module, k_chunk is raised one step at a time, cheapest time increase first, while
    the layer stays within the target.
    """
    say = log if log is not None else (lambda *_: None)
    mods = list(table)
    base = {m: float(table[m]["baseline_us"]) for m in mods}
    times = {m: {int(n): {int(k): float(t) for k, t in row.items()} for n, row in table[m]["times_us"].items()} for m in mods}
    layer_base = sum(base.values())
    layer_target = layer_base * target_slowdown
    say(f"Layer baseline: {layer_base:.2f} us; target {layer_target:.2f} us (slowdown {target_slowdown:.2f})")

    k_max = max(k for m in mods for row in times[m].values() for k in row)
    n_lo = min(min(times[m]) for m in mods)
    n_hi = max(max(times[m]) for m in mods)
    by_size = sorted(mods, key=lambda m: table[m]["dims"][0] * table[m]["dims"][1])
    included = list(mods)
    excluded: List[str] = []

    best_budget: Optional[int] = None
    best_k = 0
    best_time = math.inf
    while True:
        best_budget, best_k, best_time = None, 0, math.inf
        for budget in range(n_lo, n_hi + 1):
            k_fit, t_fit = 0, layer_base
            for k in range(1, k_max + 1):
                total = sum(base[m] for m in excluded)
                for m in included:
                    n = _n_tb_at(times[m], budget)
                    total += times[m][n].get(k, math.inf) if n is not None else math.inf
                if total > layer_target:
                    break
                k_fit, t_fit = k, total
            else:
                raise TunerRangeError("global search did not converge - increase the range of k_chunk")
            if k_fit > best_k or (k_fit == best_k and t_fit < best_time):
                best_budget, best_k, best_time = budget, k_fit, t_fit
        if best_k > 0:
            break
        smallest = by_size.pop(0)
        included.remove(smallest)
        excluded.append(smallest)
        if not included:
            say("Unable to fetch any rows for any module within the target.")
            break
        say(f"Excluding smallest module {smallest} {tuple(table[smallest]['dims'])} and retrying the global search")

    n_tb_of: Dict[str, Optional[int]] = {}
    t_of: Dict[str, float] = {}
    k_of: Dict[str, int] = {}
    for m in mods:
        if m in included:
            n_tb_of[m] = _n_tb_at(times[m], best_budget)
            t_of[m] = times[m][n_tb_of[m]][best_k]
            k_of[m] = best_k
        else:
            n_tb_of[m], t_of[m], k_of[m] = None, base[m], 0
    say(f"Global: n_tb budget {best_budget}, k_chunk {best_k}, layer {sum(t_of.values()):.2f} us")

    while included:
        delta = {}
        for m in mods:
            row = times[m][n_tb_of[m]] if m in included else {}
            nxt = k_of[m] + 1
            delta[m] = (row[nxt] - row[k_of[m]]) if nxt in row else math.inf
        moved = False
        for m in sorted(mods, key=lambda q: delta[q]):     # stable: ties keep module order
            if sum(t_of.values()) + delta[m] <= layer_target:
                k_of[m] += 1
                t_of[m] += delta[m]
                moved = True
        if not moved:
            break

    return {
        "matrix_dims": {m: tuple(table[m]["dims"]) for m in mods},
        "target_slowdown": target_slowdown,
        "layer_baseline_us": layer_base,
        "best_max_n_tb": best_budget,
        "threadblocks_per_module": [n_tb_of[m] for m in mods],
        "k_chunk_per_module": [k_of[m] for m in mods],
        "time_by_module": [t_of[m] for m in mods],
        "layer_time": sum(t_of.values()),
        "excluded": list(excluded),
    }


def format_report(res: Mapping, title: str = "") -> str:
    mods = list(res["matrix_dims"])
    lines = []
    bar = "~" * 70
    lines += [bar, f"Tuning results {title} @ {100 * (res['target_slowdown'] - 1):.1f}% slowdown", bar]
    lines.append(f"Layer baseline           : {res['layer_baseline_us']:.2f} us")
    lines.append(f"Best n_tb                : {res['best_max_n_tb']}")
    lines.append("k_chunk per module       : " + ", ".join(str(k) for k in res["k_chunk_per_module"]))
    lines.append(f"Layer time               : {res['layer_time']:.2f} us (slowdown {res['layer_time'] / res['layer_baseline_us']:.3f})")
    for i, m in enumerate(mods):
        K, N = res["matrix_dims"][m]
        n_tb = res["threadblocks_per_module"][i]
        tag = "(excluded)" if m in res["excluded"] else f"(n_tb={n_tb})"
        lines.append(f"    {m} ({K} x {N}): k_chunk {res['k_chunk_per_module'][i]} / 1024 {tag}  {res['time_by_module'][i]:.2f} us")
    lines.append(bar)
    return "\n".join(lines)


# ---------------------------------------------------------------------------------------------------------
# measurement (GPU)
# ---------------------------------------------------------------------------------------------------------

class _Module:
    """One projection: distinct weight copies that together exceed L2, one residual config, rotating inputs."""

    def __init__(self, torch, ext, dev, K, N, algo, bits, group, seed, max_k_chunk):
        self.torch, self.ext, self.K, self.N, self.algo, self.bits, self.group = torch, ext, K, N, algo, bits, group
        g = torch.Generator(device=dev).manual_seed(seed)
        gc = torch.Generator().manual_seed(seed + 1)
        wbytes = bits * N * K / 8
        self.ncopy = max(2, min(32, int(160e6 // wbytes) + 1))
        ri = lambda *shape: torch.randint(-2 ** 31, 2 ** 31 - 1, shape, dtype=torch.int32, device=dev, generator=g)
        if algo == "lutgemm":
            self.w = [(ri(K // 32, bits, N), (torch.rand(K // group, bits, N, device=dev, generator=g) * 0.01).half(),
                       ((torch.rand(K // group, N, device=dev, generator=g) - 0.5) * 0.01).half()) for _ in range(self.ncopy)]
        elif algo == "anyprec":
            self.w = [(ri(bits, N, K // 32), (torch.randn(N, 2 ** bits, device=dev, generator=g) * 0.02).half())
                      for _ in range(self.ncopy)]
        else:
            raise ValueError(f"unknown algo {algo!r} (lutgemm | anyprec)")
        # activations with a fixed 1 % outlier subset, thresholds from the same distribution
        xs = torch.randn(8, K, device=dev, generator=g)
        out_idx = torch.randperm(K, device=dev, generator=g)[: max(1, K // 100)]
        xs[:, out_idx] *= 20.0
        self.x = [xs[i].half().reshape(1, 1, K) for i in range(8)]
        self.y = torch.zeros(1, 1, N, dtype=torch.float16, device=dev)
        self.residual = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, generator=gc)
        self.scales = (torch.rand(N, generator=gc) * 1e-3 + 1e-4).half()
        self.thresholds = torch.sort(xs.abs().flatten()[torch.randperm(xs.numel(), device=dev, generator=g)[:K]],
                                     descending=True).values.half().cpu()
        self.cfg = None
        self.max_k_chunk = max_k_chunk

    def bind(self, ctx, k_chunk):
        if self.cfg is None:
            self.cfg = self.ext.create_dec_config(ctx, k_chunk, self.residual, self.scales, self.thresholds)
        else:
            self.ext.update_dec_config(self.cfg, ctx, k_chunk)

    def call(self, i, on):
        x, w = self.x[i % 8], self.w[i % self.ncopy]
        if self.algo == "lutgemm":
            if on:
                self.ext.dec_lutgemm(self.cfg, x, self.y, *w, self.bits, self.group)
            else:
                self.ext.lutgemm_gemv(x, self.y, *w, self.bits, self.group)
        else:
            if on:
                self.ext.dec_anyprec(self.cfg, x, self.y, *w, self.bits)
            else:
                self.ext.anyprec_gemv(x, self.y, *w, self.bits)

    def close(self):
        if self.cfg is not None:
            self.ext.destroy_dec_config(self.cfg)
            self.cfg = None


def _time_graph(torch, stream, body, launches, reps):
    """us per launch of `body` (which issues `launches` launches), graph-captured and replayed `reps` times."""
    with torch.cuda.stream(stream):
        body()
        stream.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=stream):
            body()
        gr.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            gr.replay()
        b.record(stream)
        stream.synchronize()
    us = a.elapsed_time(b) * 1e3 / (reps * launches)
    del gr
    return us


def _load_ext():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("the tuner measures on a GPU: no CUDA device is visible")
    import decdec_ext as ext          # raises if the CUDA library is missing; there is no fallback
    return torch, ext


def measure(dims: Mapping[str, Tuple[int, int]], algo: str = "lutgemm", bits: int = 3, group: int = 128,
            n_tb_grid: Sequence[int] = (4, 8, 12, 16, 24, 32, 48, 64, 96), max_k_chunk: int = 16,
            launches: int = 32, reps: int = 6, log=None) -> dict:
    """Fill the table `search()` consumes: per module the standalone GEMV time and the fused time for every
    (n_tb, k_chunk) with k_chunk = 1..max_k_chunk.  Launches rotate over weight copies larger than L2."""
    torch, ext = _load_ext()
    say = log if log is not None else (lambda *_: None)
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.Stream()
    rows = torch.zeros(64 * 1024, dtype=torch.int32, device=dev)
    acts = torch.zeros(64 * 1024, dtype=torch.float16, device=dev)
    ctxs = {n: ext.create_dec_context(n, rows, acts) for n in n_tb_grid}
    table = {}
    for idx, (name, (K, N)) in enumerate(dims.items()):
        mod = _Module(torch, ext, dev, K, N, algo, bits, group, 100 + 10 * idx, max_k_chunk)
        body_off = lambda: [mod.call(i, False) for i in range(launches)]
        t0 = min(_time_graph(torch, stream, body_off, launches, reps) for _ in range(2))
        grid = {}
        for n in n_tb_grid:
            row = {}
            for k in range(1, max_k_chunk + 1):
                mod.bind(ctxs[n], k)
                body_on = lambda: [mod.call(i, True) for i in range(launches)]
                row[k] = _time_graph(torch, stream, body_on, launches, reps)
            grid[n] = row
            say(f"  {name} ({K} x {N}) n_tb={n}: off {t0:.2f} us; k_chunk 1..{max_k_chunk}: " + " ".join(f"{row[k]:.1f}" for k in row))
        table[name] = {"dims": (K, N), "baseline_us": t0, "times_us": grid}
        mod.close()
    return table          # contexts are small host records; the binding surface has no destroy call for them


def verify(dims: Mapping[str, Tuple[int, int]], res: Mapping, algo: str = "lutgemm", bits: int = 3, group: int = 128,
           layers: int = 8, reps: int = 10) -> dict:
    """Time `layers` consecutive layers (qkv, o, gu, d in order, distinct weights per launch) with compensation
    off and with the tuned (n_tb, k_chunk); returns the measured per-layer times and slowdown."""
    torch, ext = _load_ext()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.Stream()
    rows = torch.zeros(64 * 1024, dtype=torch.int32, device=dev)
    acts = torch.zeros(64 * 1024, dtype=torch.float16, device=dev)
    names = list(dims)
    mods = {}
    ctxs = {}
    for idx, name in enumerate(names):
        K, N = dims[name]
        k = res["k_chunk_per_module"][idx]
        n_tb = res["threadblocks_per_module"][idx]
        mods[name] = _Module(torch, ext, dev, K, N, algo, bits, group, 100 + 10 * idx, max(k, 1))
        if k > 0 and n_tb:
            if n_tb not in ctxs:
                ctxs[n_tb] = ext.create_dec_context(int(n_tb), rows, acts)
            mods[name].bind(ctxs[n_tb], int(k))

    def body(on):
        for layer in range(layers):
            for idx, name in enumerate(names):
                mods[name].call(layer, on and res["k_chunk_per_module"][idx] > 0 and mods[name].cfg is not None)

    n = layers * len(names)
    off = min(_time_graph(torch, stream, lambda: body(False), n, reps) for _ in range(2)) * len(names)
    on = min(_time_graph(torch, stream, lambda: body(True), n, reps) for _ in range(2)) * len(names)
    for m in mods.values():
        m.close()
    return {"layer_off_us": off, "layer_on_us": on, "slowdown": on / off}


# ---------------------------------------------------------------------------------------------------------
# CLI
# ---------------------------------------------------------------------------------------------------------

def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="DecDEC (n_tb, k_chunk) tuner driven by CUDA-event timings")
    ap.add_argument("--model", choices=sorted(MODEL_DIMS), help="use the projection sizes of a known model")
    for m in MODULES:
        ap.add_argument(f"--{m}", nargs=2, type=int, metavar=("K", "N"), help=f"in/out features of the {m} projection")
    ap.add_argument("--algo", default="lutgemm", choices=["lutgemm", "anyprec"])
    ap.add_argument("--bitwidth", type=int, default=3)
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--target-slowdown", type=float, default=5.0, help="percent over the compensation-off layer time")
    ap.add_argument("--n-tb", type=int, nargs="+", default=[4, 8, 12, 16, 24, 32, 48, 64, 96])
    ap.add_argument("--max-k-chunk", type=int, default=0, help="0: twice the bandwidth-ratio estimate, at least 16")
    ap.add_argument("--hbm-gbs", type=float, default=8000.0)
    ap.add_argument("--pcie", nargs=2, type=int, default=[5, 16], metavar=("GEN", "LANES"))
    ap.add_argument("--table", help="read the timing table from this JSON file instead of measuring")
    ap.add_argument("--save-table", help="write the measured table to this JSON file")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--open-loop", action="store_true", help="verify once, do not tighten the budget when the sequence misses the target")
    ap.add_argument("--verify-layers", type=int, default=32)
    ap.add_argument("--json", action="store_true", help="print the result as one JSON line at the end")
    args = ap.parse_args(argv)

    dims = dict(MODEL_DIMS[args.model]) if args.model else {}
    for m in MODULES:
        v = getattr(args, m)
        if v:
            dims[m] = (v[0], v[1])
    if not args.table and set(dims) != set(MODULES):
        ap.error("give --model or all of --qkv --o --gu --d")
    dims = {m: dims[m] for m in MODULES if m in dims}

    say = lambda *a: print(*a, file=sys.stderr, flush=True)
    if args.table:
        raw = json.load(open(args.table))
        table = {m: {"dims": tuple(v["dims"]), "baseline_us": v["baseline_us"],
                     "times_us": {int(n): {int(k): t for k, t in row.items()} for n, row in v["times_us"].items()}}
                 for m, v in raw.items()}
        dims = {m: table[m]["dims"] for m in table}
    else:
        est = estimate_k_chunk(args.bitwidth, args.hbm_gbs, pcie_gbs(*args.pcie))
        kmax = args.max_k_chunk or max(2 * est, 16)
        say(f"bandwidth-ratio estimate k_chunk = {est}; measuring k_chunk 1..{kmax}, n_tb {args.n_tb}")
        table = measure(dims, args.algo, args.bitwidth, args.group, args.n_tb, kmax, log=say)
        if args.save_table:
            json.dump(table, open(args.save_table, "w"))
    target = 1.0 + args.target_slowdown / 100.0
    res = search(table, target, log=say)
    print(format_report(res, f"{args.model or 'custom'} {args.algo} {args.bitwidth}-bit"))
    if not args.no_verify and not args.table:
        # The table times every projection on its own; in a layer sequence the launches follow one another
        # and the sum is a little optimistic.  Closed loop: measure the chosen point on a layer sequence and,
        # if it misses the target, search again with the budget tightened by the observed excess.
        eff = target
        for attempt in range(4):
            v = verify(dims, res, args.algo, args.bitwidth, args.group, layers=args.verify_layers)
            print(f"Measured on a {args.verify_layers}-layer sequence: off {v['layer_off_us']:.2f} us, tuned {v['layer_on_us']:.2f} us, "
                  f"slowdown {v['slowdown']:.3f} (target {target:.3f})")
            res["verify"] = v
            if v["slowdown"] <= target or not any(res["k_chunk_per_module"]) or args.open_loop:
                break
            eff = 1.0 + (eff - 1.0) * (target - 1.0) / (v["slowdown"] - 1.0) * 0.9
            say(f"tightening the search budget to {100 * (eff - 1):.2f} %")
            res = search(table, eff, log=say)
            res["target_slowdown"] = target
            print(format_report(res, f"{args.model or 'custom'} {args.algo} {args.bitwidth}-bit (budget {100 * (eff - 1):.2f} %)"))
    if args.json:
        print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
