"""CPU tests of the host side: the C-ABI library loads, exports every symbol the header declares,
and rejects bad arguments with the documented status codes before touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    from decdec_b200 import capi as m
    return m


def test_header_symbols_are_exported(capi):
    hdr = open(os.path.join(ROOT, "include", "decdec_b200.h")).read()
    declared = set(re.findall(r"\b(decdec_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(capi.lib, name), f"{name} declared in the header but not exported"
    assert set(capi.SIGNATURES) <= declared | {"decdec_last_error"}
    assert capi.lib.decdec_compiled_arch() == 100


def test_status_codes_without_gpu(capi):
    h = C.c_size_t(0)
    assert capi.lib.decdec_create_context(4, None, None, 16, capi.FP16, C.byref(h)) == -1
    assert b"must be on GPU" in capi.lib.decdec_last_error()
    assert capi.lib.decdec_create_context(4, 16, 16, 16, 7, C.byref(h)) == -1           # bad dtype
    assert capi.lib.decdec_create_config(0, 8, 16, 0, 1024, 64, 16, 0, 16, capi.FP16, C.byref(h)) == -1   # null context
    info = capi.ConfigInfo()
    assert capi.lib.decdec_read_config(0, C.byref(info)) == -1
    assert capi.lib.decdec_dec(0, 16, 16, 1024, 64, capi.FP16, None) == -1
    assert capi.lib.decdec_lutgemm_gemv(16, 16, 16, 16, 16, 64, 1024, 9, 128, capi.FP16, None) == -1
    assert b"Bitwidth must be between 1 and 8" in capi.lib.decdec_last_error()
    assert capi.lib.decdec_lutgemm_gemv(16, 16, 16, 16, 16, 64, 1000, 3, 128, capi.FP16, None) == -1     # K % 32
    assert capi.lib.decdec_anyprec_gemv(16, 16, 16, 3, 16, 64, 1024, 3, capi.FP32, None) == -1
    assert b"does not support float" in capi.lib.decdec_last_error()
    assert capi.lib.decdec_anyprec_gemv(16, 16, 16, 2, 16, 64, 1024, 3, capi.FP16, None) == -1            # planes < bits
    assert capi.lib.decdec_sqllm_gemv(16, 16, 16, 16, 64, 1024, 5, capi.FP16, None) == -1
    assert capi.lib.decdec_anyprec_dequant(16, 16, 16, 64, 1024, 3, capi.FP32, None) == -1
    with pytest.raises(capi.DecdecError) as e:
        capi.call("decdec_sqllm_gemv", 16, 16, 16, 16, 64, 1024, 5, capi.FP16, None)
    assert e.value.code == -1 and "3 or 4" in str(e.value)


def test_added_entry_points_without_gpu(capi):
    """Host-side checks of the entry points that have no reference counterpart (no device work)."""
    f, s, st, b = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert capi.lib.decdec_tp_layout(2, 4096, C.byref(f), C.byref(s), C.byref(st), C.byref(b)) == 0
    assert f.value == 256 and s.value % 256 == 0 and s.value >= f.value + 2 * 64 * 4
    assert st.value >= 4096 * 4 and st.value % 256 == 0
    assert b.value == s.value + 2 * 2 * st.value                       # two halves x world slots
    assert capi.lib.decdec_tp_layout(8, 8192, None, None, None, C.byref(b)) == 0 and b.value > 2 * 8 * 8192 * 4
    assert capi.lib.decdec_tp_layout(9, 4096, None, None, None, None) == -1      # world out of range
    assert capi.lib.decdec_tp_layout(0, 4096, None, None, None, None) == -1
    h = C.c_size_t(0)
    assert capi.lib.decdec_tp_create(2, 2, 4096, C.byref(h), None) == -1          # rank >= world
    assert capi.lib.decdec_tp_create(2, 0, 0, C.byref(h), None) != 0              # empty vector
    assert capi.lib.decdec_tp_allreduce(0, 16, 1024, capi.FP16, None) == -1       # null communicator
    assert capi.lib.decdec_tp_destroy(0) == 0
    assert capi.lib.decdec_lutgemm_dequant(16, 16, 16, 16, 64, 1024, 9, 128, capi.FP16, None) == -1
    assert b"Bitwidth must be between 1 and 8" in capi.lib.decdec_last_error()
    assert capi.lib.decdec_lutgemm_dequant(16, 16, 16, 16, 63, 1024, 3, 128, capi.FP16, None) != 0      # odd out_features
    assert capi.lib.decdec_lutgemm_dequant(16, 16, 16, 16, 64, 1024, 3, 100, capi.FP16, None) == -1     # bad group


def test_drop_in_module_surface():
    """`import decdec_ext` gives the 17 functions of the reference binding (bindings.cpp:19-40) and the
    tensor checks run before any device work."""
    import torch
    import decdec_ext
    names = {"create_dec_context", "create_dec_config", "read_dec_config", "update_dec_config", "destroy_dec_config",
             "dec", "unfused_dec", "anyprec_dequant", "anyprec_gemv", "lutgemm_gemv", "sqllm_gemv", "dec_anyprec",
             "dec_lutgemm", "dec_sqllm", "dummy_anyprec", "dummy_lutgemm", "dummy_sqllm"}
    assert names == set(decdec_ext.__all__)
    from decdec_b200 import ops
    assert names == set(ops.__all__)
    x, y = torch.zeros(1, 1, 64, dtype=torch.half), torch.zeros(1, 1, 8)
    for mod in (decdec_ext, ops):
        with pytest.raises(RuntimeError, match="Mismatched data types"):
            mod.lutgemm_gemv(x, y, torch.zeros(2, 3, 8, dtype=torch.int32), torch.zeros(1, 3, 8).half(), torch.zeros(1, 8).half(), 3, 64)
        with pytest.raises(RuntimeError, match="must be on GPU"):
            mod.create_dec_context(4, torch.zeros(4, dtype=torch.int32), torch.zeros(4).half())
        with pytest.raises(RuntimeError, match="Bitwidth must be 3 or 4"):
            mod.sqllm_gemv(x, y.half(), torch.zeros(10, 8, dtype=torch.int32), torch.zeros(8, 32).half(), 5)


def test_bench_accounting():
    import bench
    assert bench.gemv_bytes(4096, 4096) == pytest.approx(7.36e6, rel=0.01)        # table of algorithmic bytes: 7.36 MB
    assert bench.fetch_bytes(4096, 4096, 32) == 128 * 2048
    p = bench.projections("llama3-8b")
    assert [(e["n"], e["k"]) for e in p] == [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
    p8 = bench.projections("llama3-70b", tp=8)
    assert [(e["n"], e["k"]) for e in p8] == [(1280, 8192), (8192, 1024), (7168, 8192), (8192, 4096)]   # 28 chunks -> 4,4,4,4,3,3,3,3
    # Llama-3-8B over 8 ranks: wo has 4 selection chunks, so two ranks share a chunk and split its outputs
    q8 = bench.projections("llama3-8b", tp=8, rank=3)
    assert (q8[1]["n"], q8[1]["k"], q8[1]["n0"], q8[1]["n_full"]) == (2048, 1024, 2048, 4096)
    assert (q8[3]["n"], q8[3]["k"]) == (4096, 2048)          # 14 chunks -> 2,2,2,2,2,2,1,1
