"""CPU tests: the oracle against the golden vectors produced by the reference's own Python code
(tests/golden/make_golden.py), plus self-consistency identities of the packers and the selection rule."""
import os

import numpy as np
import pytest
import torch

from oracle import formats, residual, selection, forward as ofw

G = os.path.join(os.path.dirname(__file__), "golden")


def test_residual_quantizer_matches_reference_bit_exact():
    d = np.load(os.path.join(G, "cheatsheet.npz"))
    err = torch.from_numpy(d["w"]) - torch.from_numpy(d["wq"])         # fp16 - fp16, as in cheatsheet.py:40
    q, scales = residual.quantize_residual(err)
    cs, rs = residual.pack_cheatsheet(q.numpy(), scales.numpy())
    assert cs.dtype == np.int32 and cs.shape == d["cheatsheet"].shape
    assert np.array_equal(cs, d["cheatsheet"])
    assert np.array_equal(rs.view(np.uint16), d["reordered_scales"].view(np.uint16))
    q2, s2 = residual.unpack_cheatsheet(d["cheatsheet"], d["reordered_scales"])
    assert np.array_equal(q2, q.numpy()) and np.array_equal(s2, scales.numpy())
    assert q2.min() >= -7 and q2.max() <= 7


@pytest.mark.parametrize("bits", [3, 4])
def test_uniform_quantizer_matches_reference(bits):
    d = np.load(os.path.join(G, f"uniform_b{bits}.npz"))
    w_fake, s, z, codes = formats.pseudo_quantize_uniform(d["w"], bits, 128)
    assert np.array_equal(s, d["scales"]) and np.array_equal(z, d["zeros"])
    assert np.array_equal(w_fake, d["w_fake"])
    assert codes.min() >= 0 and codes.max() <= 2 ** bits - 1
    # binary-coded form reproduces the fake-quantized weights (qmodule.py:61-92)
    qw, alpha, qb = formats.uniform_to_bcq(s, z, codes, bits)
    assert qw.shape == (d["w"].shape[1] // 32, bits, d["w"].shape[0])
    dense = formats.bcq_dequant(qw, alpha, qb, 128)
    assert np.abs(dense - w_fake).max() < 1e-7


def test_bcq_dequant_matches_reference():
    d = np.load(os.path.join(G, "lutgemm_dequant.npz"))
    dense = formats.bcq_dequant(d["binary"], d["alpha"], d["q_bias"], int(d["group"]))
    # the reference sums in fp16 (evaltools.py:561-580): a few half ulps at |w| ~ 0.03
    assert np.abs(dense - d["dense"]).max() <= 4 * 2.0 ** -16
    # same function through the torch CPU path used as timed baseline
    t = ofw.torch_bcq_dequant(torch.from_numpy(d["binary"]), torch.from_numpy(d["alpha"]), torch.from_numpy(d["q_bias"]), int(d["group"]))
    assert np.abs(t.numpy().T - dense).max() < 1e-6


@pytest.mark.parametrize("bits", [3, 4])
def test_sqllm_unpack_matches_reference(bits):
    d = np.load(os.path.join(G, f"sqllm_dequant_b{bits}.npz"))
    codes = formats.sqllm_unpack(d["qweight"], bits)
    dense = formats.lut_dequant(d["lut"], codes, np.float32)
    assert np.array_equal(dense, d["dense"])
    assert np.array_equal(formats.sqllm_pack(codes, bits), d["qweight"])


@pytest.mark.parametrize("K", [32, 96, 1024, 1536, 1024 + 32, 4096, 17920 // 4])
def test_anyprec_layout_matches_reference_bit_tricks(K):
    """pack -> literal emulation of the reference's 3-bit dequant kernel gives back lut[code]."""
    rng = np.random.default_rng(K)
    codes = rng.integers(0, 8, (4, K)).astype(np.int32)
    q = formats.anyprec_pack(codes, 3)
    assert q.shape == (3, 4, K // 32) and np.array_equal(formats.anyprec_unpack(q, 3), codes)
    lut = rng.standard_normal((4, 8)).astype(np.float16)
    assert np.array_equal(formats.anyprec_reference_emulation_3bit(q, lut), formats.lut_dequant(lut, codes, np.float16))
    kmap = formats.anyprec_k_of(K)
    assert sorted(kmap.reshape(-1).tolist()) == list(range(K))


@pytest.mark.parametrize("bits", [3, 4, 5, 8])
def test_anyprec_pack_roundtrip_all_widths(bits):
    rng = np.random.default_rng(bits)
    codes = rng.integers(0, 2 ** bits, (3, 1024 + 256)).astype(np.int32)
    assert np.array_equal(formats.anyprec_unpack(formats.anyprec_pack(codes, bits), bits), codes)
    # extra planes are ignored
    q = np.concatenate([formats.anyprec_pack(codes, bits), rng.integers(-2**31, 2**31, (1, 3, 40), dtype=np.int64).astype(np.int32)])
    assert np.array_equal(formats.anyprec_unpack(q, bits), codes)


def test_bucket_floors_recipe():
    for dtype, a, b in [("fp16", 77.3, 2.41), ("bf16", 77.3, 2.41), ("fp32", 77.3, 2.41), ("fp16", 0.5, 0.5)]:
        f = selection.bucket_floors(a, b, dtype)
        assert f[0] == selection._rn(a, dtype) and f[31] == 0.0
        assert np.all(np.diff(f[:16]) <= 0) and np.all(np.diff(f[16:]) <= 0)
    # fp16 recipe: floor[15] = a + half(b - a), not b itself
    f = selection.bucket_floors(80.0, 2.4, "fp16")
    assert f[15] == float(np.float16(np.float16(80.0) + np.float16(np.float16(2.4) - np.float16(80.0))))
    assert selection._round_bf16(1.00390625) == 1.0 and selection._round_bf16(1.01171875) == 1.015625


def test_selection_properties_and_edges():
    rng = np.random.default_rng(3)
    K, k_chunk = 4096 + 512, 32                      # ragged: last chunk has 512 channels -> kq = 16
    x = rng.standard_normal(K).astype(np.float16)
    x[rng.choice(K, 40, replace=False)] *= 20
    thr = -np.sort(-np.abs(x.astype(np.float32)))
    k = k_chunk * K // 1024
    rows, acts, hist = selection.select(x, thr[0], thr[k - 1], k_chunk, "fp16")
    assert rows.shape == (k,) and k == 4 * 32 + 16
    floors = selection.bucket_floors(thr[0], thr[k - 1], "fp16")
    for c in range(5):
        s, e = c * 1024, min((c + 1) * 1024, K)
        kq = k_chunk * (e - s) // 1024
        sel = rows[c * k_chunk: c * k_chunk + kq]
        assert len(set(sel.tolist())) == kq and sel.min() >= s and sel.max() < e
        assert np.array_equal(acts[c * k_chunk: c * k_chunk + kq], x[sel].astype(np.float64))
        assert hist[c].sum() == e - s
        # every unselected channel lies in the boundary bucket or a later one
        ax = np.abs(x[s:e].astype(np.float64))
        bucket = (ax[:, None] >= floors[None, :]).argmax(1)
        unsel = np.setdiff1d(np.arange(s, e), sel)
        assert bucket[sel - s].max() <= bucket[unsel - s].min()
    # k_chunk = 0 and empty input
    r0, a0, _ = selection.select(x, thr[0], thr[0], 0, "fp16")
    assert r0.size == 0 and a0.size == 0
    # NaN / inf never selected; fewer finite values than the quota -> padded with (chunk start, 0)
    y = np.full(1024, np.nan, np.float32); y[:3] = [1.0, np.inf, 2.0]
    r, a, _ = selection.select(y, 4.0, 0.5, 8, "fp32")
    assert r.tolist() == [0, 2, 0, 0, 0, 0, 0, 0] and a.tolist() == [1.0, 2.0, 0, 0, 0, 0, 0, 0]
    # exact top-k agrees with the bucket rule on the set when thresholds separate the values cleanly
    z = np.zeros(1024, np.float32); z[[5, 900, 17]] = [3.0, -4.0, 2.5]
    r, _, _ = selection.select(z, 4.0, 2.0, 3, "fp32")
    assert sorted(r.tolist()) == sorted(selection.exact_topk(z, 3).tolist())


def test_dec_delta_linear_and_cpu_baseline_consistency():
    rng = np.random.default_rng(9)
    N, K = 64, 2048
    q = rng.integers(-7, 8, (N, K))
    sc = (rng.random(N) * 1e-3).astype(np.float16)
    cs, rs = residual.pack_cheatsheet(q, sc)
    x = rng.standard_normal(K).astype(np.float16)
    rows = np.array([3, 1500, 77, 2047], np.int32)
    d = ofw.dec_delta(x, rows, cs, rs)
    ref = (q[:, rows].astype(np.float64) * sc.astype(np.float64)[:, None]) @ x[rows].astype(np.float64)
    assert np.allclose(d, ref, rtol=1e-12, atol=1e-15)
    # linearity in the activations
    assert np.allclose(ofw.dec_delta(2 * x.astype(np.float64), rows, cs, rs), 2 * d)
    # torch CPU baseline: per-chunk exact top-k + residual matvec equals the dense formula
    rt = ofw.torch_unpack_residual(torch.from_numpy(cs), torch.from_numpy(rs))
    wt = torch.zeros(K, N)
    y = ofw.cpu_reference_linear(torch.from_numpy(x).float(), wt, rt, 4)
    sel = np.concatenate([np.argsort(-np.abs(x[s:s + 1024].astype(np.float32)), kind="stable")[:4] + s for s in (0, 1024)])
    ref2 = (q[:, sel].astype(np.float64) * sc.astype(np.float64)[:, None]) @ x[sel].astype(np.float64)
    assert np.allclose(y.numpy(), ref2, rtol=1e-4, atol=1e-6)
