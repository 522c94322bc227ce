"""Tuner measurement path on the GPU: a tiny grid through the real entry points, then the search."""
import pytest

pytestmark = pytest.mark.gpu


def test_measure_search_verify_small():
    from decdec_b200 import tuner
    dims = {"qkv": (1024, 1536), "o": (1024, 1024), "gu": (1024, 4096), "d": (2048, 1024)}
    table = tuner.measure(dims, algo="lutgemm", bits=3, group=128, n_tb_grid=(4, 8), max_k_chunk=3, launches=8, reps=2)
    assert list(table) == list(dims)
    for m, (K, N) in dims.items():
        assert table[m]["dims"] == (K, N)
        assert table[m]["baseline_us"] > 0
        assert set(table[m]["times_us"]) == {4, 8}
        for row in table[m]["times_us"].values():
            assert set(row) == {1, 2, 3} and all(t > 0 for t in row.values())
    try:
        res = tuner.search(table, 1.5)
    except tuner.TunerRangeError:
        res = tuner.search(table, 1.0001)       # nothing fits: every module excluded
    assert len(res["k_chunk_per_module"]) == 4
    v = tuner.verify(dims, res, layers=2, reps=2)
    assert v["layer_off_us"] > 0 and v["layer_on_us"] > 0


def test_measure_anyprec_small():
    from decdec_b200 import tuner
    dims = {"qkv": (1024, 1536), "o": (1024, 1024), "gu": (1024, 2048), "d": (2048, 1024)}
    table = tuner.measure(dims, algo="anyprec", bits=3, n_tb_grid=(8,), max_k_chunk=2, launches=4, reps=1)
    assert all(table[m]["times_us"][8][2] > 0 for m in dims)
