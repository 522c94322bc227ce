"""(n_tb, k_chunk) search against the reference's own search (autotuner/tuner.py:128-351).

tests/golden/tuner_cases.json holds seeded synthetic timing tables and what the reference's `tuner()` returned
for them (generator: tests/golden/make_tuner_golden.py).  No GPU involved.
"""
import json
import math
import os

import pytest

from decdec_b200 import tuner

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "golden", "tuner_cases.json")))


def _table(case):
    return {m: {"dims": tuple(v["dims"]), "baseline_us": v["baseline_us"],
                "times_us": {int(n): {int(k): t for k, t in row.items()} for n, row in v["times_us"].items()}}
            for m, v in case["table"].items()}


@pytest.mark.parametrize("i", range(len(CASES)))
def test_search_matches_reference(i):
    case = CASES[i]
    table = _table(case)
    if "expect_error" in case:
        with pytest.raises(tuner.TunerRangeError):
            tuner.search(table, case["target_slowdown"])
        return
    res = tuner.search(table, case["target_slowdown"])
    exp = case["expect"]
    assert res["best_max_n_tb"] == exp["best_max_n_tb"]
    assert res["threadblocks_per_module"] == exp["threadblocks_per_module"]
    assert res["k_chunk_per_module"] == exp["k_chunk_per_module"]
    assert res["time_by_module"] == pytest.approx(exp["time_by_module"], rel=1e-9)
    assert res["layer_time"] == pytest.approx(exp["layer_time"], rel=1e-9)


def test_golden_covers_all_paths():
    kinds = set()
    for c in CASES:
        if "expect_error" in c:
            kinds.add("range")
        elif all(k == 0 for k in c["expect"]["k_chunk_per_module"]):
            kinds.add("nothing")
        elif any(n is None for n in c["expect"]["threadblocks_per_module"]):
            kinds.add("excluded")
        else:
            kinds.add("all")
    assert kinds == {"range", "nothing", "excluded", "all"}


@pytest.mark.parametrize("i", [j for j, c in enumerate(CASES) if "expect" in c])
def test_result_is_feasible_and_maximal(i):
    """Independent of the reference: the answer fits the target and no module can take one more row."""
    case = CASES[i]
    table = _table(case)
    res = tuner.search(table, case["target_slowdown"])
    target = res["layer_baseline_us"] * case["target_slowdown"]
    assert res["layer_time"] <= target * (1 + 1e-12)
    for idx, m in enumerate(table):
        n_tb, k = res["threadblocks_per_module"][idx], res["k_chunk_per_module"][idx]
        if n_tb is None:
            assert k == 0 and res["time_by_module"][idx] == table[m]["baseline_us"]
            continue
        row = table[m]["times_us"][n_tb]
        assert res["time_by_module"][idx] == pytest.approx(row[k])
        if k + 1 in row:
            assert res["layer_time"] - row[k] + row[k + 1] > target


def test_estimate_matches_reference_formula():
    # autotuner/run_profile.py:26-30 with 8000 GB/s HBM and PCIe 5.0 x16
    assert tuner.pcie_gbs(5, 16) == 64.0
    assert tuner.estimate_k_chunk(3, 8000.0, 64.0) == 6
    assert tuner.estimate_k_chunk(4, 8000.0, 64.0) == 8
    assert tuner.pcie_gbs(4, 16) == 32.0


def test_report_and_cli_from_table(tmp_path, capsys):
    case = next(c for c in CASES if "expect" in c)
    p = tmp_path / "table.json"
    p.write_text(json.dumps(case["table"]))
    rc = tuner.main(["--table", str(p), "--target-slowdown", str(100 * (case["target_slowdown"] - 1)), "--json"])
    assert rc == 0
    out = capsys.readouterr().out
    assert "Best n_tb" in out and "k_chunk per module" in out
    res = json.loads(out.strip().splitlines()[-1])
    assert res["k_chunk_per_module"] == case["expect"]["k_chunk_per_module"]


def test_measure_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(RuntimeError):
        tuner.measure(tuner.MODEL_DIMS["llama3-8b"])
