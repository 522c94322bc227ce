"""Generates tests/golden/tuner_cases.json by running the REFERENCE's search function
(autotuner/tuner.py:tuner of SNU-ARC/DecDEC checked out at REF, the first argument) on seeded synthetic
timing tables.

    python tests/golden/make_tuner_golden.py REF

`tuner.py` imports matplotlib and its Nsight parser at module level; neither is used by the search, so both
are replaced by empty stand-in modules for the import.  The tables are synthetic cost models (a launch floor,
a per-row link cost that shrinks with n_tb, a GEMV slowdown that grows with n_tb, plus seeded noise); they are
not measurements.
"""
import contextlib
import importlib.util
import io
import json
import os
import sys
import types

import numpy as np

if len(sys.argv) < 2:
    raise SystemExit("usage: python " + sys.argv[0] + " <path of the SNU-ARC/DecDEC checkout>")
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))

DIMS = {"qkv": (4096, 6144), "o": (4096, 4096), "gu": (4096, 28672), "d": (14336, 4096)}


def load_reference():
    for name in ("matplotlib", "matplotlib.pyplot", "nsys_parser"):
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    spec = importlib.util.spec_from_file_location("ref_tuner", os.path.join(REF, "autotuner", "tuner.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def synth_table(rng, n_tb_grid, k_max, floor_scale, link_scale, noise):
    """module -> (baseline, {n_tb: {k: time}})"""
    table = {}
    for m, (K, N) in DIMS.items():
        base = 4.0 + K * N / 2.0e6 * (0.8 + 0.4 * rng.random())
        grid = {}
        for n in n_tb_grid:
            gemv = base * (1.0 + 0.6 * n / 148.0)                     # GEMV loses SMs to the compensation blocks
            row = {}
            for k in range(1, k_max + 1):
                fetch = floor_scale * (5.0 + 20.0 / n) + link_scale * k * (K / 1024) * N / 2 / 50e3 * (1.0 + 8.0 / n)
                t = max(gemv, fetch) + 0.15 * min(gemv, fetch)
                row[k] = round(float(t * (1.0 + noise * (rng.random() - 0.5))), 3)
            grid[n] = row
        table[m] = (round(float(base), 3), grid)
    return table


def main():
    ref = load_reference()
    rng = np.random.default_rng(7)
    cases = []
    specs = [
        # n_tb grid, k_max, floor scale, link scale, noise, target
        ((4, 8, 12, 16, 24, 32), 24, 0.5, 1.0, 0.02, 1.10),
        ((4, 8, 12, 16, 24, 32), 24, 0.5, 1.0, 0.02, 1.025),
        ((4, 6, 8, 10, 12, 14, 16), 32, 0.3, 1.6, 0.05, 1.20),
        ((8, 16, 32, 64), 32, 0.2, 2.5, 0.0, 1.50),
        ((4, 8, 16, 32, 64, 74), 16, 1.2, 1.5, 0.03, 1.05),      # small modules cannot fit: exclusion path
        ((4, 8, 16), 12, 3.0, 2.0, 0.01, 1.01),                   # nothing fits at all
        ((5, 9, 13), 40, 0.4, 0.9, 0.10, 1.15),
        ((4, 8, 12, 16, 24, 32, 48), 20, 0.1, 0.3, 0.02, 1.30),      # every k fits: range error
    ]
    for grid, k_max, fs, ls, noise, target in specs:
        table = synth_table(rng, grid, k_max, fs, ls, noise)
        results_by_module = {m: (b, t, {}, {}, {}) for m, (b, t) in table.items()}
        entry = {"target_slowdown": target,
                 "table": {m: {"dims": list(DIMS[m]), "baseline_us": b, "times_us": {str(n): {str(k): v for k, v in row.items()} for n, row in t.items()}}
                           for m, (b, t) in table.items()}}
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                res = ref.tuner(results_by_module, target, dict(DIMS))
            entry["expect"] = {"best_max_n_tb": res["best_max_n_tb"],
                               "threadblocks_per_module": res["threadblocks_per_module"],
                               "k_chunk_per_module": [int(k) for k in res["k_chunk_per_module"]],
                               "time_by_module": [float(t) for t in res["time_by_module"]],
                               "layer_time": float(res["layer_time"])}
        except ValueError as e:
            entry["expect_error"] = str(e)
        cases.append(entry)
    with open(os.path.join(OUT, "tuner_cases.json"), "w") as f:
        json.dump(cases, f)
    for c in cases:
        print(c.get("expect", c.get("expect_error")))


if __name__ == "__main__":
    main()
