"""GPU cross-check against the reference's own CUDA kernels.

`oracle/build_ref.py` compiles the reference's decdec_extension sources, unmodified, into
`oracle/_ref/decdec_ref*.so` (the same pybind module under another name).  These tests feed identical
tensors to that module and to this library (through the C ABI) and compare

  * the channel selection of `fused_dec_kernel` (decdec_extension/dec.cu:78-182) by the rule that is
    reproducible for it: per chunk the same number of picks from every bucket, the same set from
    the buckets taken completely, the same count from the bucket that overflows the quota with all
    picks being members of it, and recorded activations bitwise equal to x[row];
  * `anyprec_dequant` exactly;
  * every GEMV and fused entry point through three errors against the float64 oracle:
    err(new, oracle), err(ref, oracle), err(new, ref).  The assertion is
    err(new, oracle) <= max(1e-2, err(ref, oracle)) (max abs) and rel L2 <= max(1e-3, ref's).

The reference trips a device assert on activations that are not finite (dec.cu:178), so only finite
inputs are given to it.  The measured table is written to reference_crosscheck.json in the directory that the
environment variable DECDEC_REPORT_DIR names (if set).
"""
import importlib.util
import json
import os
import sys

import numpy as np
import pytest
import torch

from oracle import forward as ofw
from oracle import selection
from tests import problems as P

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
REPORT = {}


def _load_ref():
    import sysconfig
    path = os.path.join(REF_DIR, "decdec_ref" + sysconfig.get_config_var("EXT_SUFFIX"))
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("decdec_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    mod = _load_ref()
    if mod is None:
        pytest.skip("reference build absent: run `python oracle/build_ref.py <DecDEC checkout>` first")
    yield mod
    out = os.environ.get("DECDEC_REPORT_DIR", "")
    if REPORT and out and os.path.isdir(out):
        with open(os.path.join(out, "reference_crosscheck.json"), "w") as f:
            json.dump(REPORT, f, indent=1, sort_keys=True)


@pytest.fixture(scope="module")
def ops():
    from decdec_b200 import ops as _ops
    return _ops


def _bufs(size, dtype):
    return (torch.full((size,), -1, dtype=torch.int32, device="cuda"),
            torch.zeros(size, dtype=P.TORCH_DT[dtype], device="cuda"))


def _three_errors(name, y_new, y_ref, oracle, tol_abs=1e-2, tol_rel=1e-3):
    new_o = P.errors(y_new, oracle)
    ref_o = P.errors(y_ref, oracle)
    new_r = P.errors(y_new, P.to_np(y_ref).reshape(-1))
    REPORT[name] = {"new_vs_oracle": new_o, "ref_vs_oracle": ref_o, "new_vs_ref": new_r}
    assert new_o[0] <= max(tol_abs, ref_o[0]), f"{name}: max abs new/oracle {new_o[0]:.3e}, ref/oracle {ref_o[0]:.3e}"
    assert new_o[1] <= max(tol_rel, ref_o[1]), f"{name}: rel L2 new/oracle {new_o[1]:.3e}, ref/oracle {ref_o[1]:.3e}"
    return new_o, ref_o, new_r


# ------------------------------------------------------------------------------------------------
# selection
# ------------------------------------------------------------------------------------------------

def _bucket_of(x64, floors):
    ax = np.abs(x64)
    ge = ax[:, None] >= floors[None, :]
    return np.where(ge.any(1), ge.argmax(1), selection.NUM_BUCKETS)


def _check_selection_rule(x, thr, k_chunk, dtype, rows_ref, acts_ref, rows_new):
    x64 = P.to_np(x).reshape(-1)
    K = x64.shape[0]
    k = k_chunk * K // 1024
    t = P.to_np(thr)
    floors = selection.bucket_floors(t[0], t[k - 1], dtype)
    bucket = _bucket_of(x64, floors)
    exp_rows, _, hist = selection.select(x64, t[0], t[k - 1], k_chunk, dtype)
    assert np.array_equal(rows_new, exp_rows)
    for c in range((K + 1023) // 1024):
        s, e = c * 1024, min((c + 1) * 1024, K)
        kq = k_chunk * (e - s) // 1024
        pr = rows_ref[c * k_chunk: c * k_chunk + kq].astype(np.int64)
        pn = rows_new[c * k_chunk: c * k_chunk + kq].astype(np.int64)
        assert ((pr >= s) & (pr < e)).all(), f"chunk {c}: reference picked outside the chunk"
        assert len(set(pr.tolist())) == kq, f"chunk {c}: reference picked a channel twice"
        cum = np.cumsum(hist[c])
        lb = int(np.nonzero(cum >= kq)[0][0])
        # (1) the same number of picks from every bucket = the same histogram up to the boundary bucket
        cr = np.bincount(bucket[pr], minlength=33)[:32]
        cn = np.bincount(bucket[pn], minlength=33)[:32]
        want = np.minimum(hist[c], np.maximum(kq - (cum - hist[c]), 0))
        assert np.array_equal(cr, want), f"chunk {c}: reference bucket counts {cr} != {want}"
        assert np.array_equal(cn, want)
        # (2) identical set from the buckets taken completely
        assert set(pr[bucket[pr] < lb].tolist()) == set(pn[bucket[pn] < lb].tolist()), f"chunk {c}: sets differ below bucket {lb}"
        # (3) the same count from the boundary bucket, all of them members (covered by the counts above)
        assert (bucket[pr] <= lb).all() and (bucket[pn] <= lb).all()
    # (4) recorded activations are the signed activations of the recorded rows, bitwise
    got = acts_ref[:k].view(torch.int16 if dtype != "fp32" else torch.int32).cpu().numpy()
    src = x.reshape(-1).cuda()[torch.from_numpy(rows_ref[:k].astype(np.int64)).cuda()]
    assert np.array_equal(got, src.view(torch.int16 if dtype != "fp32" else torch.int32).cpu().numpy())


@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("K,N,k_chunk,n_tb", [
    (4096, 4096, 32, 16),      # single 4096x4096 layer, k_chunk 32
    (4096, 1024, 8, 8),        # k/v projection
    (4096, 14336, 64, 32),     # gate/up
    (14336, 4096, 16, 24),     # down projection
    (17920, 512, 16, 32),      # 17.5 chunks: partial last chunk (dec.cu:84-86)
])
def test_selection_matches_reference_kernel(ref, ops, dtype, K, N, k_chunk, n_tb):
    cs, rs = P.random_residual(N, K, seed=K + N, dtype=dtype)
    thr = P.make_thresholds(K, dtype)
    x = P.make_activation(K, seed=K + k_chunk + 1, dtype=dtype)
    k = k_chunk * K // 1024
    rows_r, acts_r = _bufs(K, dtype)
    rows_n, acts_n = _bufs(K, dtype)
    cfg_r = ref.create_dec_config(ref.create_dec_context(n_tb, rows_r, acts_r), k_chunk, cs, rs, thr)
    cfg_n = ops.create_dec_config(ops.create_dec_context(n_tb, rows_n, acts_n), k_chunk, cs, rs, thr)
    y_r = torch.zeros(1, 1, N, dtype=P.TORCH_DT[dtype], device="cuda")
    y_n = torch.zeros_like(y_r)
    xd = x.cuda()
    ref.dec(cfg_r, xd, y_r)
    ops.dec(cfg_n, xd, y_n)
    torch.cuda.synchronize()
    _check_selection_rule(x, thr, k_chunk, dtype, rows_r[:k].cpu().numpy(), acts_r, rows_n[:k].cpu().numpy())
    # compensation term: both against the float64 value for the rows each one selected
    d_new = ofw.dec_delta(P.to_np(x), rows_n[:k].cpu().numpy(), cs.numpy(), P.to_np(rs))
    d_ref = ofw.dec_delta(P.to_np(x), rows_r[:k].cpu().numpy(), cs.numpy(), P.to_np(rs))
    e_new, e_ref = P.errors(y_n, d_new), P.errors(y_r, d_ref)
    REPORT[f"dec {N}x{K} kc{k_chunk} {dtype}"] = {"new_vs_oracle": e_new, "ref_vs_oracle": e_ref}
    ta, tr = {"fp16": (1e-2, 1e-3), "bf16": (8e-2, 6e-3), "fp32": (1e-3, 1e-5)}[dtype]
    assert e_new[0] <= max(ta, e_ref[0]) and e_new[1] <= max(tr, e_ref[1]), (e_new, e_ref)
    ref.destroy_dec_config(cfg_r)
    ops.destroy_dec_config(cfg_n)


def test_reference_script_shape(ref, ops):
    """Inputs of the reference's decdec_extension/tests/test_dec.py (K=14336, N=4096, n_tb=24,
    k_chunk=20, x ~ U(-1,1), thresholds = sorted |x|, random residual words)."""
    K, N, n_tb, k_chunk = 14336, 4096, 24, 20
    g = torch.Generator().manual_seed(0)
    q = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int32, generator=g)
    scales = torch.rand(N, generator=g)
    x32 = torch.rand(1, 1, K, generator=g) * 2 - 1
    thr32 = torch.sort(x32.abs().view(-1), descending=True).values
    k = k_chunk * K // 1024
    for dtype in ["fp32", "fp16", "bf16"]:
        td = P.TORCH_DT[dtype]
        x, thr, sc = x32.to(td), thr32.to(td), scales.to(td)
        rows_r, acts_r = _bufs(K, dtype)
        rows_n, acts_n = _bufs(K, dtype)
        cfg_r = ref.create_dec_config(ref.create_dec_context(n_tb, rows_r, acts_r), k_chunk, q, sc, thr)
        cfg_n = ops.create_dec_config(ops.create_dec_context(n_tb, rows_n, acts_n), k_chunk, q, sc, thr)
        y_r = torch.zeros(1, 1, N, dtype=td, device="cuda")
        y_n = torch.zeros_like(y_r)
        ref.dec(cfg_r, x.cuda(), y_r)
        ops.dec(cfg_n, x.cuda(), y_n)
        torch.cuda.synchronize()
        _check_selection_rule(x, thr, k_chunk, dtype, rows_r[:k].cpu().numpy(), acts_r, rows_n[:k].cpu().numpy())
        d_new = ofw.dec_delta(P.to_np(x), rows_n[:k].cpu().numpy(), q.numpy(), P.to_np(sc))
        d_ref = ofw.dec_delta(P.to_np(x), rows_r[:k].cpu().numpy(), q.numpy(), P.to_np(sc))
        rel_new = np.linalg.norm(P.to_np(y_n).reshape(-1) - d_new) / np.linalg.norm(d_new)
        rel_ref = np.linalg.norm(P.to_np(y_r).reshape(-1) - d_ref) / np.linalg.norm(d_ref)
        REPORT[f"test_dec.py shape {dtype}"] = {"rel_new_vs_oracle": rel_new, "rel_ref_vs_oracle": rel_ref}
        assert rel_new <= max({"fp32": 1e-5, "fp16": 1e-3, "bf16": 6e-3}[dtype], rel_ref)
        ref.destroy_dec_config(cfg_r)
        ops.destroy_dec_config(cfg_n)


def test_unfused_dec_matches_reference(ref, ops):
    K, N, k_chunk = 4096, 4096, 32
    cs, rs = P.random_residual(N, K, seed=21)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=22)
    k = k_chunk * K // 1024
    top = torch.from_numpy(selection.exact_topk(P.to_np(x).reshape(-1), k)).cuda()
    rows_r, acts_r = _bufs(K, "fp16")
    rows_n, acts_n = _bufs(K, "fp16")
    cfg_r = ref.create_dec_config(ref.create_dec_context(16, rows_r, acts_r), k_chunk, cs, rs, thr)
    cfg_n = ops.create_dec_config(ops.create_dec_context(16, rows_n, acts_n), k_chunk, cs, rs, thr)
    rows_r[:k] = top
    rows_n[:k] = top
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.unfused_dec(cfg_r, x.cuda(), y_r)
    ops.unfused_dec(cfg_n, x.cuda(), y_n)
    torch.cuda.synchronize()
    delta = ofw.dec_delta(P.to_np(x), top.cpu().numpy(), cs.numpy(), P.to_np(rs))
    _three_errors("unfused_dec 4096x4096 kc32 fp16", y_n, y_r, delta)


# ------------------------------------------------------------------------------------------------
# any-precision
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("bits,N,K", [(3, 256, 4096), (3, 64, 1536), (4, 128, 2048), (5, 64, 1024), (6, 64, 2048), (7, 32, 1024), (8, 64, 1024)])
def test_anyprec_dequant_equals_reference(ref, ops, dtype, bits, N, K):
    """The reference's `dequant_kbit_store` (anyprec.cu:261-331) defines the bit layout: both modules must
    turn the same planes into the same dense matrix, which also pins the packer of the oracle."""
    L = P.lut_layer(N, K, bits, seed=bits * 7 + 1, dtype=dtype, real=False)
    qw, lut = L["qweight"].cuda(), L["lut"].cuda()
    w_ref = ref.anyprec_dequant(qw, lut, bits)
    w_new = ops.anyprec_dequant(qw, lut, bits)
    torch.cuda.synchronize()
    assert w_ref.shape == w_new.shape == (N, K)
    assert torch.equal(w_ref, w_new), "dense weights differ from the reference's dequantization"
    assert np.array_equal(P.to_np(w_ref), L["w_hat"]), "oracle's any-precision packing differs from the reference layout"


@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_anyprec_gemv_three_errors(ref, ops, N, K):
    """Llama-3-8B projection shapes, 3-bit LUT weights, activations with x20 outliers."""
    L = P.lut_layer(N, K, 3, seed=N + 3, real=False)
    x = P.make_activation(K, seed=43)
    qw, lut, xd = L["qweight"].cuda(), L["lut"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.anyprec_gemv(xd, y_r, qw, lut, 3)
    ops.anyprec_gemv(xd, y_n, qw, lut, 3)
    torch.cuda.synchronize()
    _three_errors(f"anyprec_gemv {N}x{K} b3 fp16", y_n, y_r, ofw.layer_output(L["w_hat"], P.to_np(x)))


@pytest.mark.parametrize("bits", [4, 5, 8])
def test_anyprec_gemv_other_widths(ref, ops, bits):
    N, K = 1024, 4096
    L = P.lut_layer(N, K, bits, seed=bits, real=False)
    x = P.make_activation(K, seed=44)
    qw, lut, xd = L["qweight"].cuda(), L["lut"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.anyprec_gemv(xd, y_r, qw, lut, bits)
    ops.anyprec_gemv(xd, y_n, qw, lut, bits)
    torch.cuda.synchronize()
    _three_errors(f"anyprec_gemv {N}x{K} b{bits} fp16", y_n, y_r, ofw.layer_output(L["w_hat"], P.to_np(x)))


@pytest.mark.parametrize("N,K,k_chunk,n_tb", [(14336, 4096, 64, 96), (14336, 4096, 8, 16), (4096, 14336, 16, 32), (4096, 4096, 32, 64)])
def test_dec_anyprec_three_errors(ref, ops, N, K, k_chunk, n_tb):
    L = P.lut_layer(N, K, 3, seed=N + k_chunk, real=False)
    cs, rs = P.random_residual(N, K, seed=45)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=43)
    k = k_chunk * K // 1024
    rows_r, acts_r = _bufs(K, "fp16")
    rows_n, acts_n = _bufs(K, "fp16")
    cfg_r = ref.create_dec_config(ref.create_dec_context(n_tb, rows_r, acts_r), k_chunk, cs, rs, thr)
    cfg_n = ops.create_dec_config(ops.create_dec_context(n_tb, rows_n, acts_n), k_chunk, cs, rs, thr)
    qw, lut, xd = L["qweight"].cuda(), L["lut"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.dec_anyprec(cfg_r, xd, y_r, qw, lut, 3)
    ops.dec_anyprec(cfg_n, xd, y_n, qw, lut, 3)
    torch.cuda.synchronize()
    base = ofw.layer_output(L["w_hat"], P.to_np(x))
    o_new = base + ofw.dec_delta(P.to_np(x), rows_n[:k].cpu().numpy(), cs.numpy(), P.to_np(rs))
    o_ref = base + ofw.dec_delta(P.to_np(x), rows_r[:k].cpu().numpy(), cs.numpy(), P.to_np(rs))
    e_new, e_ref = P.errors(y_n, o_new), P.errors(y_r, o_ref)
    REPORT[f"dec_anyprec {N}x{K} kc{k_chunk} fp16"] = {"new_vs_oracle": e_new, "ref_vs_oracle": e_ref}
    assert e_new[0] <= max(1e-2, e_ref[0]) and e_new[1] <= max(1e-3, e_ref[1]), (e_new, e_ref)
    ref.destroy_dec_config(cfg_r)
    ops.destroy_dec_config(cfg_n)


# ------------------------------------------------------------------------------------------------
# binary-coded and SqueezeLLM
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("N,K,bits", [(4096, 4096, 3), (6144, 4096, 3), (4096, 14336, 3), (2048, 4096, 4)])
def test_lutgemm_gemv_three_errors(ref, ops, dtype, N, K, bits):
    L = P.bcq_layer(N, K, bits, 128, seed=1, dtype=dtype) if (N == K == 4096 and dtype == "fp16") else P.random_bcq_layer(N, K, bits, 128, seed=N + bits, dtype=dtype)
    x = P.make_activation(K, seed=2, dtype=dtype)
    qw, al, qb, xd = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=P.TORCH_DT[dtype], device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.lutgemm_gemv(xd, y_r, qw, al, qb, bits, 128)
    ops.lutgemm_gemv(xd, y_n, qw, al, qb, bits, 128)
    torch.cuda.synchronize()
    ta, tr = {"fp16": (1e-2, 1e-3), "bf16": (8e-2, 6e-3), "fp32": (1e-3, 1e-5)}[dtype]
    _three_errors(f"lutgemm_gemv {N}x{K} b{bits} {dtype}", y_n, y_r, ofw.layer_output(L["w_hat"], P.to_np(x)), ta, tr)


def test_dec_lutgemm_single_layer_three_errors(ref, ops):
    """The single-layer configuration end to end: real 3-bit group-128 quantization, real 4-bit residual, k_chunk 32."""
    N = K = 4096
    L = P.bcq_layer(N, K, 3, 128, seed=1)
    cs, rs = P.quantized_residual(L["w"], L["w_fake"])
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=2)
    rows_r, acts_r = _bufs(K, "fp16")
    rows_n, acts_n = _bufs(K, "fp16")
    cfg_r = ref.create_dec_config(ref.create_dec_context(16, rows_r, acts_r), 32, cs, rs, thr)
    cfg_n = ops.create_dec_config(ops.create_dec_context(16, rows_n, acts_n), 32, cs, rs, thr)
    qw, al, qb, xd = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.dec_lutgemm(cfg_r, xd, y_r, qw, al, qb, 3, 128)
    ops.dec_lutgemm(cfg_n, xd, y_n, qw, al, qb, 3, 128)
    torch.cuda.synchronize()
    base = ofw.layer_output(L["w_hat"], P.to_np(x))
    o_new = base + ofw.dec_delta(P.to_np(x), rows_n[:128].cpu().numpy(), cs.numpy(), P.to_np(rs))
    o_ref = base + ofw.dec_delta(P.to_np(x), rows_r[:128].cpu().numpy(), cs.numpy(), P.to_np(rs))
    e_new, e_ref = P.errors(y_n, o_new), P.errors(y_r, o_ref)
    REPORT["dec_lutgemm 4096x4096 kc32 fp16"] = {"new_vs_oracle": e_new, "ref_vs_oracle": e_ref}
    assert e_new[0] <= max(1e-2, e_ref[0]) and e_new[1] <= max(1e-3, e_ref[1]), (e_new, e_ref)
    ref.destroy_dec_config(cfg_r)
    ops.destroy_dec_config(cfg_n)


@pytest.mark.parametrize("bits", [3, 4])
def test_sqllm_three_errors(ref, ops, bits):
    N, K = 4096, 4096
    L = P.lut_layer(N, K, bits, seed=bits + 10, fmt="sqllm", real=False)
    x = P.make_activation(K, seed=81)
    qw, lut, xd = L["qweight"].cuda(), L["lut"].cuda(), x.cuda()
    y_r = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    y_n = torch.zeros_like(y_r)
    ref.sqllm_gemv(xd, y_r, qw, lut, bits)
    ops.sqllm_gemv(xd, y_n, qw, lut, bits)
    torch.cuda.synchronize()
    _three_errors(f"sqllm_gemv {N}x{K} b{bits} fp16", y_n, y_r, ofw.layer_output(L["w_hat"], P.to_np(x)))
    # fused
    cs, rs = P.random_residual(N, K, seed=52)
    thr = P.make_thresholds(K)
    rows_r, acts_r = _bufs(K, "fp16")
    rows_n, acts_n = _bufs(K, "fp16")
    cfg_r = ref.create_dec_config(ref.create_dec_context(16, rows_r, acts_r), 16, cs, rs, thr)
    cfg_n = ops.create_dec_config(ops.create_dec_context(16, rows_n, acts_n), 16, cs, rs, thr)
    y_r.zero_(); y_n.zero_()
    ref.dec_sqllm(cfg_r, xd, y_r, qw, lut, bits)
    ops.dec_sqllm(cfg_n, xd, y_n, qw, lut, bits)
    torch.cuda.synchronize()
    base = ofw.layer_output(L["w_hat"], P.to_np(x))
    o_new = base + ofw.dec_delta(P.to_np(x), rows_n[:64].cpu().numpy(), cs.numpy(), P.to_np(rs))
    o_ref = base + ofw.dec_delta(P.to_np(x), rows_r[:64].cpu().numpy(), cs.numpy(), P.to_np(rs))
    e_new, e_ref = P.errors(y_n, o_new), P.errors(y_r, o_ref)
    REPORT[f"dec_sqllm {N}x{K} b{bits} kc16 fp16"] = {"new_vs_oracle": e_new, "ref_vs_oracle": e_ref}
    assert e_new[0] <= max(1e-2, e_ref[0]) and e_new[1] <= max(1e-3, e_ref[1]), (e_new, e_ref)
    ref.destroy_dec_config(cfg_r)
    ops.destroy_dec_config(cfg_n)


# ------------------------------------------------------------------------------------------------
# timings of the reference kernels beside this library's (not asserted; written to the report)
# ------------------------------------------------------------------------------------------------

def _time_us(call, n_sets, iters=64):
    """Event-timed average of `call(i)` over a captured graph of 32 launches that rotate over weight
    sets larger than L2; falls back to eager launches when the calls cannot be captured."""
    for i in range(3):
        call(i)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(s):
        call(0)
        s.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for i in range(32):
                    call(i)
            g.replay()
            s.synchronize()
            a.record(s)
            for _ in range(max(1, iters // 32)):
                g.replay()
            b.record(s)
            s.synchronize()
            return a.elapsed_time(b) * 1e3 / (32 * max(1, iters // 32)), "graph"
        except Exception:
            torch.cuda.synchronize()
    a.record()
    for i in range(iters):
        call(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters, "eager"


def test_reference_kernel_timings(ref, ops):
    import decdec_ext as ext
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    ri = lambda *shape: torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=g)
    out = {}
    for N, K in [(4096, 4096), (6144, 4096), (28672, 4096), (4096, 14336)]:
        ncopy = max(2, min(24, int(160e6 // (3 * N * K / 8)) + 1))
        x = torch.randn(1, 1, K, device=dev, generator=g).half()
        y = torch.zeros(1, 1, N, dtype=torch.float16, device=dev)
        wb = [(ri(K // 32, 3, N), (torch.rand(K // 128, 3, N, device=dev, generator=g) * 0.01).half(),
               ((torch.rand(K // 128, N, device=dev, generator=g) - 0.5) * 0.01).half()) for _ in range(ncopy)]
        wa = [(ri(3, N, K // 32), (torch.randn(N, 8, device=dev, generator=g) * 0.02).half()) for _ in range(ncopy)]
        gc = torch.Generator().manual_seed(2)
        q = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int32, generator=gc)
        sc = (torch.rand(N, generator=gc) * 1e-3 + 1e-4).half()
        thr = torch.sort(torch.randn(K, generator=gc).abs() * 3, descending=True).values.half()
        rows_r, acts_r = _bufs(32 * 1024, "fp16")
        rows_n, acts_n = _bufs(32 * 1024, "fp16")
        cfg_r = ref.create_dec_config(ref.create_dec_context(24, rows_r, acts_r), 8, q, sc, thr)
        cfg_n = ext.create_dec_config(ext.create_dec_context(24, rows_n, acts_n), 8, q, sc, thr)
        row = {}
        row["lutgemm_gemv ref"] = _time_us(lambda i: ref.lutgemm_gemv(x, y, *wb[i % ncopy], 3, 128), ncopy)
        row["lutgemm_gemv new"] = _time_us(lambda i: ext.lutgemm_gemv(x, y, *wb[i % ncopy], 3, 128), ncopy)
        row["anyprec_gemv ref"] = _time_us(lambda i: ref.anyprec_gemv(x, y, *wa[i % ncopy], 3), ncopy)
        row["anyprec_gemv new"] = _time_us(lambda i: ext.anyprec_gemv(x, y, *wa[i % ncopy], 3), ncopy)
        if N * K <= 6144 * 4096 or K == 4096:
            n4 = max(2, min(ncopy, 4))
            w4 = [(ri(4, N, K // 32), (torch.randn(N, 16, device=dev, generator=g) * 0.02).half()) for _ in range(n4)]
            row["anyprec_gemv 4-bit ref"] = _time_us(lambda i: ref.anyprec_gemv(x, y, *w4[i % n4], 4), n4)
            row["anyprec_gemv 4-bit new"] = _time_us(lambda i: ext.anyprec_gemv(x, y, *w4[i % n4], 4), n4)
            del w4
        row["dec kc8 ref"] = _time_us(lambda i: ref.dec(cfg_r, x, y), 1)
        row["dec kc8 new"] = _time_us(lambda i: ext.dec(cfg_n, x, y), 1)
        row["dec_lutgemm kc8 ref"] = _time_us(lambda i: ref.dec_lutgemm(cfg_r, x, y, *wb[i % ncopy], 3, 128), ncopy)
        row["dec_lutgemm kc8 new"] = _time_us(lambda i: ext.dec_lutgemm(cfg_n, x, y, *wb[i % ncopy], 3, 128), ncopy)
        out[f"{N}x{K}"] = row
        ref.destroy_dec_config(cfg_r)
        ext.destroy_dec_config(cfg_n)
        del wb, wa
        torch.cuda.empty_cache()
    REPORT["timings_us"] = out
