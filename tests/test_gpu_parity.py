"""GPU parity tests: the CUDA library, called through its C ABI (decdec_b200.ops -> capi -> .so),
against the CPU oracle on the same seeded inputs.

Tolerances (north star): fp16 outputs max abs err <= 1e-2 and rel L2 <= 1e-3 against the float64
oracle; bf16 outputs carry 8 mantissa bits, so 8e-2 / 6e-3; fp32 1e-3 / 1e-5.  Channel selection is
compared bit-exactly (rows and recorded activations).
"""
import os

import numpy as np
import pytest
import torch

from oracle import forward as ofw
from oracle import formats, selection
from tests import problems as P

pytestmark = pytest.mark.gpu

TOL = {"fp16": (1e-2, 1e-3), "bf16": (8e-2, 6e-3), "fp32": (1e-3, 1e-5)}


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from decdec_b200 import ops as _ops
    return _ops


def _y0(N, dtype, seed=5):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(1, 1, N, generator=g) * 0.5).to(P.TORCH_DT[dtype])


def _assert_close(y, ref, dtype, what=""):
    ma, rl = P.errors(y, ref)
    ta, tr = TOL[dtype]
    assert ma <= ta and rl <= tr, f"{what}: max abs {ma:.3e} (tol {ta}), rel L2 {rl:.3e} (tol {tr})"


def _ctx(ops, n_tb, size, dtype):
    rows = torch.full((size,), -1, dtype=torch.int32, device="cuda")
    acts = torch.zeros(size, dtype=P.TORCH_DT[dtype], device="cuda")
    return ops.create_dec_context(n_tb, rows, acts), rows, acts


# ------------------------------------------------------------------------------------------------
# binary-coded (LUT-GEMM) GEMV
# ------------------------------------------------------------------------------------------------

def test_lutgemm_config0_fp16(ops):
    """The single-layer configuration: 4096x4096, 3-bit asymmetric group-128, fp16; output accumulated into y0."""
    N = K = 4096
    L = P.bcq_layer(N, K, 3, 128, seed=1)
    x = P.make_activation(K, seed=2)
    y0 = _y0(N, "fp16")
    y = y0.clone().cuda()
    ops.lutgemm_gemv(x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
    ref = ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0))
    _assert_close(y, ref, "fp16", "lutgemm config0")
    # deterministic up to fp32 reduction order: two runs agree to the output rounding
    y2 = y0.clone().cuda()
    ops.lutgemm_gemv(x.cuda(), y2, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
    assert (y.float() - y2.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("N,K,bits,group", [
    (1024, 4096, 3, 128),    # k/v projection
    (512, 1024, 4, 128),
    (72, 1088, 3, 32),       # ragged: N not a multiple of 32, K not a multiple of 512, group 32
    (256, 2048, 1, 64),
    (128, 1536, 2, 128),
    (96, 512, 5, 128),
    (64, 1024, 8, 256),
])
def test_lutgemm_shapes(ops, dtype, N, K, bits, group):
    L = P.random_bcq_layer(N, K, bits, group, seed=N + K + bits, dtype=dtype)
    x = P.make_activation(K, seed=3, dtype=dtype)
    y0 = _y0(N, dtype)
    y = y0.clone().cuda()
    ops.lutgemm_gemv(x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), bits, group)
    ref = ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0))
    _assert_close(y, ref, dtype, f"lutgemm {N}x{K} b{bits} g{group} {dtype}")


def test_lutgemm_down_proj_fp16(ops):
    """Llama-3-8B down projection 14336 -> 4096 (28 K slices)."""
    N, K = 4096, 14336
    L = P.random_bcq_layer(N, K, 3, 128, seed=11)
    x = P.make_activation(K, seed=4)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.lutgemm_gemv(x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
    _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x)), "fp16", "lutgemm down")


@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("N,K,bits,group", [(4096, 1024, 3, 128), (48, 256, 3, 128), (130, 96, 4, 32), (256, 512, 1, 64), (64, 2048, 8, 256)])
def test_lutgemm_dequant_prefill_operand(ops, dtype, N, K, bits, group):
    """Dense [K, N] operand of the prefill GEMM: bit-exact against the reference's arithmetic
    (LUTGEMMLinear.py:41-82: plane sum rounded to the layer dtype, then + q_bias in that dtype)."""
    L = P.random_bcq_layer(N, K, bits, group, seed=N + K + bits, dtype=dtype)
    out = ops.lutgemm_dequant(L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), bits, group)
    assert out.shape == (K, N) and out.dtype == P.TORCH_DT[dtype]
    # emulation with the same roundings on the CPU (fp32 plane sum in plane order)
    words = L["qweight"].numpy().view(np.uint32)                                        # [K/32, bits, N]
    bit = ((words[:, None, :, :] >> np.arange(32, dtype=np.uint32)[None, :, None, None]) & 1).reshape(K, bits, N)
    sign = torch.from_numpy(bit.astype(np.float32) * 2 - 1)
    gidx = torch.arange(K) // group
    a = L["alpha"].float()[gidx]                                                         # [K, bits, N]
    s32 = torch.zeros(K, N)
    for p in range(bits):
        s32 = s32 + sign[:, p, :] * a[:, p, :]
    exp = s32.to(P.TORCH_DT[dtype]) + L["q_bias"][gidx]
    assert torch.equal(out.cpu(), exp), "dequantized operand differs from the two-rounding arithmetic"
    # and it is the matrix the GEMV kernels use
    rel = {"fp16": 2.0 ** -9, "bf16": 2.0 ** -6, "fp32": 1e-6}[dtype]          # two roundings to the layer dtype
    assert np.abs(P.to_np(out).T - L["w_hat"]).max() <= rel * np.abs(L["w_hat"]).max() + 1e-7


def test_lutgemm_dequant_matches_reference_output(ops):
    """Against the reference's own `lutgemm_dequant` output on the committed fixture (tests/golden)."""
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lutgemm_dequant.npz"))
    out = ops.lutgemm_dequant(torch.from_numpy(d["binary"]).cuda(), torch.from_numpy(d["alpha"]).cuda(),
                              torch.from_numpy(d["q_bias"]).cuda(), 3, int(d["group"]))
    ref = d["dense"]
    got = out.float().cpu().numpy()
    if ref.shape != got.shape:
        ref = ref.T
    assert np.abs(got - ref).max() <= 2 * 2.0 ** -16          # the reference sums the planes in fp16: <= 2 half ulps at |w| ~ 0.03


# ------------------------------------------------------------------------------------------------
# selection
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("K,k_chunk,n_tb", [
    (4096, 32, 16), (4096, 8, 4), (4096, 64, 148), (14336, 20, 24), (17920, 16, 32),   # 17920 = 17.5 chunks
    (1024, 1, 1), (2048, 1000, 8), (1536, 33, 3),
])
def test_selection_bit_exact(ops, dtype, K, k_chunk, n_tb):
    N = 256
    cs, rs = P.random_residual(N, K, seed=K, dtype=dtype)
    thr = P.make_thresholds(K, dtype)
    x = P.make_activation(K, seed=K + k_chunk, dtype=dtype)
    k = k_chunk * K // 1024
    ctx, rows, acts = _ctx(ops, n_tb, max(k, 1), dtype)
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=P.TORCH_DT[dtype], device="cuda")
    ops.dec(cfg, x.cuda(), y)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, dtype)
    assert np.array_equal(rows[:k].cpu().numpy(), exp_rows), "selected rows differ from the oracle"
    assert np.array_equal(P.to_np(acts[:k]), exp_acts), "recorded activations differ"
    # recorded activation is the signed activation of the recorded row
    assert np.array_equal(P.to_np(acts[:k]), P.to_np(x).reshape(-1)[exp_rows])
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    _assert_close(y, delta, dtype, "dec output")
    ops.destroy_dec_config(cfg)


def test_selection_degenerate_inputs(ops):
    """all-equal activations, a == b, zeros, and NaN/inf (which belong to no bucket): no trap, oracle-equal."""
    K, N, k_chunk = 2048, 64, 16
    cs, rs = P.random_residual(N, K, seed=7)
    cases = []
    cases.append((torch.full((K,), 0.5), torch.full((K,), 0.5)))                       # all equal, a == b
    cases.append((torch.zeros(K), torch.linspace(3, 0.001, K)))                         # all zero input
    xs = torch.randn(K, generator=torch.Generator().manual_seed(1))
    xs[5] = float("nan"); xs[1030] = float("inf"); xs[77] = -float("inf")
    cases.append((xs, torch.sort(torch.randn(K).abs(), descending=True).values))
    few = torch.full((K,), float("nan")); few[:10] = 1.0                                 # fewer finite values than k
    cases.append((few, torch.linspace(2, 0.01, K)))
    for xv, tv in cases:
        x = xv.half().reshape(1, 1, K)
        thr = tv.half()
        ctx, rows, acts = _ctx(ops, 8, 64, "fp16")
        cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        ops.dec(cfg, x.cuda(), y)
        torch.cuda.synchronize()
        k = k_chunk * K // 1024
        exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
        assert np.array_equal(rows[:k].cpu().numpy(), exp_rows)
        got = P.to_np(acts[:k])
        assert np.array_equal(np.nan_to_num(got, nan=123.0), np.nan_to_num(exp_acts, nan=123.0))
        ops.destroy_dec_config(cfg)


def test_dec_reference_smoke_shape(ops):
    """Shapes and inputs of the reference's own script decdec_extension/tests/test_dec.py
    (K=14336, N=4096, n_tb=24, k_chunk=20, x~U(-1,1), thresholds = sorted |x|, random int32 residual
    words including nibble 0), all three dtypes."""
    K, N, n_tb, k_chunk = 14336, 4096, 24, 20
    g = torch.Generator().manual_seed(0)
    q = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int32, generator=g)
    scales = torch.rand(N, generator=g)
    x32 = torch.rand(1, 1, K, generator=g) * 2 - 1
    thr32 = torch.sort(x32.abs().view(-1), descending=True).values
    for dtype in ["fp32", "fp16", "bf16"]:
        td = P.TORCH_DT[dtype]
        x, thr, sc = x32.to(td), thr32.to(td), scales.to(td)
        ctx, rows, acts = _ctx(ops, n_tb, K, dtype)
        cfg = ops.create_dec_config(ctx, k_chunk, q, sc, thr)
        y = torch.zeros(1, 1, N, dtype=td, device="cuda")
        ops.dec(cfg, x.cuda(), y)
        torch.cuda.synchronize()
        k = k_chunk * K // 1024
        exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, dtype)
        assert np.array_equal(rows[:k].cpu().numpy(), exp_rows)
        delta = ofw.dec_delta(P.to_np(x), exp_rows, q.numpy(), P.to_np(sc), exp_acts)
        d = P.to_np(y).reshape(-1) - delta
        rel = np.linalg.norm(d) / np.linalg.norm(delta)
        assert rel <= {"fp32": 1e-5, "fp16": 1e-3, "bf16": 6e-3}[dtype], f"{dtype}: rel L2 {rel}"
        ops.destroy_dec_config(cfg)


def test_unfused_dec_exact_topk(ops):
    """`unfused_dec` with rows written by the caller (exact global top-k, evaltools.py:327-343)."""
    K, N, k_chunk = 4096, 512, 32
    cs, rs = P.random_residual(N, K, seed=21)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=22)
    k = k_chunk * K // 1024
    ctx, rows, acts = _ctx(ops, 16, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    top = selection.exact_topk(P.to_np(x).reshape(-1), k)
    rows[:k] = torch.from_numpy(top).cuda()
    y0 = _y0(N, "fp16")
    y = y0.clone().cuda()
    ops.unfused_dec(cfg, x.cuda(), y)
    ref = P.to_np(y0).reshape(-1) + ofw.dec_delta(P.to_np(x), top, cs.numpy(), P.to_np(rs))
    _assert_close(y, ref, "fp16", "unfused_dec")


def test_k_chunk_zero_is_noop_and_update(ops):
    K, N = 2048, 128
    cs, rs = P.random_residual(N, K, seed=31)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=32)
    ctx, rows, acts = _ctx(ops, 8, 1024, "fp16")
    cfg = ops.create_dec_config(ctx, 0, cs, rs, thr)
    y0 = _y0(N, "fp16")
    y = y0.clone().cuda()
    ops.dec(cfg, x.cuda(), y)
    assert torch.equal(y.cpu(), y0)
    # re-tune without re-uploading the residual (dec_config.cu:295-326)
    ctx2, rows2, acts2 = _ctx(ops, 3, 1024, "fp16")
    ops.update_dec_config(cfg, ctx2, 24)
    info = ops.read_dec_config(cfg)
    assert info["k_chunk"] == 24 and info["num_chunks"] == 2 and info["chunk_size"] == 1024
    assert set(info) == {"num_chunks", "chunk_size", "k_chunk", "channels_per_tb", "n_tb", "block_dim_x",
                         "block_dim_y", "shared_memory_size", "reduced_shared_memory"}
    ops.dec(cfg, x.cuda(), y)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, 24, "fp16")
    assert np.array_equal(rows2[:48].cpu().numpy(), exp_rows)
    ref = P.to_np(y0).reshape(-1) + ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    _assert_close(y, ref, "fp16", "dec after update")
    with pytest.raises(RuntimeError, match="buffer size is too small"):
        ops.update_dec_config(cfg, ctx2, 1000)


# ------------------------------------------------------------------------------------------------
# fused base GEMV + compensation
# ------------------------------------------------------------------------------------------------

def test_dec_lutgemm_config0(ops):
    """The single-layer configuration end to end: real 3-bit quantization, real 4-bit residual, k_chunk = 32."""
    N = K = 4096
    L = P.bcq_layer(N, K, 3, 128, seed=1)
    cs, rs = P.quantized_residual(L["w"], L["w_fake"])
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=2)
    ctx, rows, acts = _ctx(ops, 16, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, 32, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec_lutgemm(cfg, x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, 32, "fp16")
    assert np.array_equal(rows[:128].cpu().numpy(), exp_rows)
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    ref = ofw.layer_output(L["w_hat"], P.to_np(x), None, delta)
    _assert_close(y, ref, "fp16", "dec_lutgemm config0")
    # the compensation moves the output toward the unquantized layer
    full = L["w"].astype(np.float64) @ P.to_np(x).reshape(-1)
    base = ofw.layer_output(L["w_hat"], P.to_np(x))
    assert np.linalg.norm(P.to_np(y).reshape(-1) - full) < np.linalg.norm(base - full)


@pytest.mark.parametrize("entry", ["dec", "dec_lutgemm", "dec_anyprec"])
@pytest.mark.parametrize("n_tb,k_chunk", [
    (1, 1), (1, 9), (2, 5), (4, 3), (4, 17), (8, 4), (8, 32), (12, 7), (16, 2), (24, 12), (48, 1), (96, 32), (148, 6),
])
def test_compensation_geometry_sweep(ops, entry, n_tb, k_chunk):
    """Few wide compensation thread blocks (direct fetch: vector reductions, row groups, several load batches)
    through many narrow ones (grouped fetch), alone and fused into both pipelined GEMVs: same result."""
    N, K = 4096, 3072
    cs, rs = P.random_residual(N, K, seed=61)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=62)
    ctx, rows, acts = _ctx(ops, n_tb, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    if entry == "dec":
        ops.dec(cfg, x.cuda(), y)
        ref = delta
    elif entry == "dec_lutgemm":
        L = P.bcq_layer(N, K, 3, 128, seed=63)
        ops.dec_lutgemm(cfg, x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
        ref = ofw.layer_output(L["w_hat"], P.to_np(x), None, delta)
    else:
        L = P.lut_layer(N, K, 3, seed=64)
        ops.dec_anyprec(cfg, x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), 3)
        ref = ofw.layer_output(L["w_hat"], P.to_np(x), None, delta)
    torch.cuda.synchronize()
    k = k_chunk * K // 1024
    assert np.array_equal(rows[:k].cpu().numpy(), exp_rows)
    _assert_close(y, ref, "fp16", f"{entry} n_tb={n_tb} k_chunk={k_chunk}")
    # a second call accumulates onto y again: the workspace was left clean by the first
    y2 = torch.zeros_like(y)
    if entry == "dec":
        ops.dec(cfg, x.cuda(), y2)
        torch.cuda.synchronize()
        _assert_close(y2, ref, "fp16", f"{entry} second call")
    ops.destroy_dec_config(cfg)


@pytest.mark.parametrize("dtype", ["bf16", "fp32"])
@pytest.mark.parametrize("n_tb,k_chunk", [(2, 9), (4, 3), (16, 2), (96, 32)])
def test_compensation_geometry_other_dtypes(ops, dtype, n_tb, k_chunk):
    """Direct and grouped fetch with bf16 / fp32 activations, scales and outputs (compensation alone)."""
    N, K = 4096, 2048
    cs, rs = P.random_residual(N, K, seed=81, dtype=dtype)
    thr = P.make_thresholds(K, dtype)
    x = P.make_activation(K, seed=82, dtype=dtype)
    ctx, rows, acts = _ctx(ops, n_tb, 32 * 1024, dtype)
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y0 = _y0(N, dtype)
    y = y0.clone().cuda()
    ops.dec(cfg, x.cuda(), y)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, dtype)
    k = k_chunk * K // 1024
    assert np.array_equal(rows[:k].cpu().numpy(), exp_rows)
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    _assert_close(y, P.to_np(y0).reshape(-1) + delta, dtype, f"dec {dtype} n_tb={n_tb} k_chunk={k_chunk}")
    ops.destroy_dec_config(cfg)


def test_fused_projection_artifacts_feed_the_kernel(ops):
    """q/k/v residuals fused by decdec_b200.artifacts (scales re-derived for the fused width) give the same
    compensation as the three projections one after the other."""
    from decdec_b200 import artifacts as A
    K, widths = 2048, (1024, 256, 256)
    parts, dense = [], []
    for i, n in enumerate(widths):
        cs, rs = P.random_residual(n, K, seed=90 + i)
        parts.append({"cheatsheet": cs, "reordered_scales": rs})
        dense.append(A.residual_matrix(cs, rs))
    fused = A.fuse_projections(parts)
    N = sum(widths)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=93)
    ctx, rows, acts = _ctx(ops, 12, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, 16, fused["cheatsheet"], fused["reordered_scales"], thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec(cfg, x.cuda(), y)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, 16, "fp16")
    R = torch.cat(dense, dim=0).double().numpy()                          # [N, K]
    ref = R[:, exp_rows] @ exp_acts.astype(np.float64)
    _assert_close(y, ref, "fp16", "dec with fused q/k/v artifacts")
    ops.destroy_dec_config(cfg)


@pytest.mark.parametrize("k_chunk", [0, 8, 16, 32, 64])
def test_dec_anyprec_config1_sweep(ops, k_chunk):
    """Llama-3-8B k/v projection shape (4096 -> 1024), 3-bit non-uniform LUT weights, k_chunk sweep."""
    N, K = 1024, 4096
    L = P.lut_layer(N, K, 3, seed=41)
    cs, rs = P.random_residual(N, K, seed=42)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=43)
    ctx, rows, acts = _ctx(ops, 16, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec_anyprec(cfg, x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), 3)
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts) if k_chunk else None
    _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x), None, delta), "fp16", f"dec_anyprec kc={k_chunk}")


@pytest.mark.parametrize("N,K,k_chunk,n_tb", [(14336, 4096, 64, 96), (14336, 4096, 8, 16), (4096, 14336, 16, 32), (4096, 4096, 32, 64)])
def test_dec_anyprec_config1_full_shapes(ops, N, K, k_chunk, n_tb):
    """3-bit LUT weights at the full Llama-3-8B projection sizes (gate/up, down, q/o), random codes and LUTs."""
    L = P.lut_layer(N, K, 3, seed=N + k_chunk, real=False)
    cs, rs = P.random_residual(N, K, seed=45)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=43)
    ctx, rows, acts = _ctx(ops, n_tb, 32 * 1024, "fp16")
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec_anyprec(cfg, x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), 3)
    torch.cuda.synchronize()
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
    k = k_chunk * K // 1024
    assert np.array_equal(rows[:k].cpu().numpy(), exp_rows)
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    ma, rl = P.errors(y, ofw.layer_output(L["w_hat"], P.to_np(x), None, delta))
    # rel L2 as everywhere.  Max abs: the kernel adds 4 products per half lane in fp16 before it goes to fp32 (the reference
    # adds whole rows in fp16); with x20 outliers over up to 14336 channels single outputs of magnitude 10-30 land one fp16
    # ulp (0.008-0.016) from the float64 value.  Measured on the same inputs (test_gpu_reference_crosscheck.py): this kernel
    # 0.6e-2 .. 1.3e-2, the reference's own kernel 1.5e-2 .. 2.8e-2 - so the bound here is 2e-2, not the 1e-2 of the
    # fp32-accumulating kernels, and the cross-check asserts that this kernel is never worse than the reference.
    assert rl <= TOL["fp16"][1] and ma <= 2e-2, f"dec_anyprec {N}x{K} kc={k_chunk}: max abs {ma:.3e}, rel L2 {rl:.3e}"
    ops.destroy_dec_config(cfg)


@pytest.mark.parametrize("bits", [3, 4])
def test_dec_sqllm(ops, bits):
    N, K = 512, 2048
    L = P.lut_layer(N, K, bits, seed=51, fmt="sqllm")
    cs, rs = P.random_residual(N, K, seed=52)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=53)
    ctx, rows, acts = _ctx(ops, 6, 1024, "fp16")
    cfg = ops.create_dec_config(ctx, 16, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec_sqllm(cfg, x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), bits)
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, 16, "fp16")
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x), None, delta), "fp16", f"dec_sqllm b{bits}")


# ------------------------------------------------------------------------------------------------
# any-precision and SqueezeLLM GEMVs
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("N,K,bits", [
    (4096, 4096, 3),        # q/o projection
    (1024, 4096, 3),
    (512, 14336, 3),        # down-projection K
    (256, 1536, 3),         # tail block (K = 1.5 blocks)
    (200, 1024 + 128, 3),   # ragged N, small tail
    (128, 96, 3),           # K below one block and not a multiple of 128 -> generic path
    (128, 2048, 4),
    (64, 1056, 5),          # K not a multiple of 128 -> generic path
    (64, 1024, 8),
    (4096, 4096, 4),        # pipelined lookup decoder at every width
    (1000, 14336, 4),       # ragged N, four K segments per row
    (512, 4096 + 640, 5),   # tail block
    (512, 4096, 6),
    (256, 2048, 7),
    (512, 14336, 8),        # widest rows: fewer rows per stage
    (64, 28672, 8),
])
def test_anyprec_gemv(ops, dtype, N, K, bits):
    L = P.lut_layer(N, K, bits, seed=N + K + bits, dtype=dtype, real=(bits == 3 and N <= 1024))
    x = P.make_activation(K, seed=61, dtype=dtype)
    y0 = _y0(N, dtype)
    y = y0.clone().cuda()
    ops.anyprec_gemv(x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), bits)
    ref = ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0))
    _assert_close(y, ref, dtype, f"anyprec {N}x{K} b{bits} {dtype}")


@pytest.mark.parametrize("entry", ["anyprec", "sqllm", "lutgemm", "dec_lutgemm"])
def test_output_views_and_odd_widths(ops, entry):
    """Outputs that are not 8-byte aligned (a view one element into a buffer) and widths that are not a multiple
    of four take the scalar path of the finalizer; the elements around the view must stay untouched."""
    K = 2048
    N = {"anyprec": 131, "sqllm": 70, "lutgemm": 264, "dec_lutgemm": 264}[entry]
    x = P.make_activation(K, seed=71)
    big = torch.full((1, 1, N + 3), 7.0, dtype=torch.float16, device="cuda")
    y = big[:, :, 1:1 + N]
    assert y.data_ptr() % 8 != 0
    y.zero_()
    if entry == "anyprec":
        L = P.lut_layer(N, K, 3, seed=72)
        ops.anyprec_gemv(x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), 3)
        ref = ofw.layer_output(L["w_hat"], P.to_np(x))
    elif entry == "sqllm":
        L = P.lut_layer(N, K, 3, seed=73, fmt="sqllm")
        ops.sqllm_gemv(x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), 3)
        ref = ofw.layer_output(L["w_hat"], P.to_np(x))
    else:
        L = P.bcq_layer(N, K, 3, 128, seed=74)
        if entry == "lutgemm":
            ops.lutgemm_gemv(x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
            ref = ofw.layer_output(L["w_hat"], P.to_np(x))
        else:
            cs, rs = P.random_residual(N, K, seed=75)
            thr = P.make_thresholds(K)
            ctx, rows, acts = _ctx(ops, 8, 1024, "fp16")
            cfg = ops.create_dec_config(ctx, 8, cs, rs, thr)
            ops.dec_lutgemm(cfg, x.cuda(), y, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), 3, 128)
            exp_rows, exp_acts, _ = P.expected_selection(x, thr, 8, "fp16")
            delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
            ref = ofw.layer_output(L["w_hat"], P.to_np(x), None, delta)
    torch.cuda.synchronize()
    _assert_close(y, ref, "fp16", f"{entry} into an unaligned view")
    assert float(big[0, 0, 0]) == 7.0 and float(big[0, 0, N + 1]) == 7.0 and float(big[0, 0, N + 2]) == 7.0


@pytest.mark.parametrize("bits,K", [(3, 4096), (3, 1536), (4, 2048), (8, 1024), (3, 96)])
def test_anyprec_dequant_exact_and_extra_planes(ops, bits, K):
    """Dequantized weights equal lut[code] exactly; a tensor with more planes than `bitwidth` is
    accepted and only the leading planes are used (decdec.cu:295)."""
    N = 64
    L = P.lut_layer(N, K, bits, seed=71, real=False)
    w = ops.anyprec_dequant(L["qweight"].cuda(), L["lut"].cuda(), bits)
    assert np.array_equal(P.to_np(w), L["w_hat"])
    if bits < 8:
        extra = torch.cat([L["qweight"], torch.randint(-2**31, 2**31 - 1, (1, N, K // 32), dtype=torch.int32)], 0)
        # seed prefix of a wider tensor: the first `bits` planes define the code
        x = P.make_activation(K, seed=72)
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        ops.anyprec_gemv(x.cuda(), y, extra.cuda(), L["lut"].cuda(), bits)
        _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x)), "fp16", "anyprec extra planes")


@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("N,K,bits", [(1024, 4096, 3), (512, 4096, 4), (72, 1024, 3), (40, 96, 4)])
def test_sqllm_gemv(ops, dtype, N, K, bits):
    L = P.lut_layer(N, K, bits, seed=N + bits, dtype=dtype, fmt="sqllm", real=False)
    x = P.make_activation(K, seed=81, dtype=dtype)
    y0 = _y0(N, dtype)
    y = y0.clone().cuda()
    ops.sqllm_gemv(x.cuda(), y, L["qweight"].cuda(), L["lut"].cuda(), bits)
    _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0)), dtype, f"sqllm {N}x{K} b{bits}")


def test_dummy_entry_points(ops):
    """GEMV next to the busy kernel gives the same result as the plain GEMV."""
    N, K = 256, 1024
    x = P.make_activation(K, seed=91)
    Lb = P.random_bcq_layer(N, K, 3, 128, seed=92)
    La = P.lut_layer(N, K, 3, seed=93, real=False)
    Ls = P.lut_layer(N, K, 4, seed=94, fmt="sqllm", real=False)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dummy_lutgemm(x.cuda(), y, Lb["qweight"].cuda(), Lb["alpha"].cuda(), Lb["q_bias"].cuda(), 3, 128, 8, 1000)
    _assert_close(y, ofw.layer_output(Lb["w_hat"], P.to_np(x)), "fp16", "dummy_lutgemm")
    y.zero_()
    ops.dummy_anyprec(x.cuda(), y, La["qweight"].cuda(), La["lut"].cuda(), 3, 8, 1000)
    _assert_close(y, ofw.layer_output(La["w_hat"], P.to_np(x)), "fp16", "dummy_anyprec")
    y.zero_()
    ops.dummy_sqllm(x.cuda(), y, Ls["qweight"].cuda(), Ls["lut"].cuda(), 4, 8, 1000)
    _assert_close(y, ofw.layer_output(Ls["w_hat"], P.to_np(x)), "fp16", "dummy_sqllm")


# ------------------------------------------------------------------------------------------------
# API behaviour
# ------------------------------------------------------------------------------------------------

def test_error_behaviour(ops):
    N, K = 128, 1024
    L = P.random_bcq_layer(N, K, 3, 128, seed=1)
    x = P.make_activation(K, seed=1).cuda()
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    qw, al, qb = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda()
    with pytest.raises(RuntimeError, match="Bitwidth must be between 1 and 8"):
        ops.lutgemm_gemv(x, y, qw, al, qb, 9, 128)
    with pytest.raises(RuntimeError, match="Mismatched data types"):
        ops.lutgemm_gemv(x, y.float(), qw, al, qb, 3, 128)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        ops.lutgemm_gemv(x, y, qw.transpose(0, 2), al, qb, 3, 128)
    with pytest.raises(RuntimeError, match="Batch size must be 1"):
        ops.lutgemm_gemv(x.expand(2, 1, K).contiguous(), y, qw, al, qb, 3, 128)
    with pytest.raises(RuntimeError, match="q_weight tensor must be of shape"):
        ops.lutgemm_gemv(x, y, qw[:, :2].contiguous(), al, qb, 3, 128)
    La = P.lut_layer(N, K, 3, seed=2, real=False)
    with pytest.raises(RuntimeError, match="does not support float"):
        ops.anyprec_gemv(x.float(), y.float(), La["qweight"].cuda(), La["lut"].cuda().float(), 3)
    with pytest.raises(RuntimeError, match="Bitwidth must be 3 or 4"):
        ops.sqllm_gemv(x, y, torch.zeros(K * 5 // 32, N, dtype=torch.int32, device="cuda"), torch.zeros(N, 32, dtype=torch.float16, device="cuda"), 5)
    # context / config coupling
    rows = torch.zeros(64, dtype=torch.int32, device="cuda")
    acts = torch.zeros(64, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="must be on GPU"):
        ops.create_dec_context(4, rows.cpu(), acts)
    with pytest.raises(RuntimeError, match="same size"):
        ops.create_dec_context(4, rows[:32], acts)
    ctx = ops.create_dec_context(4, rows, acts)
    cs, rs = P.random_residual(N, K, seed=3)
    thr = P.make_thresholds(K)
    with pytest.raises(RuntimeError, match="thresholds must be on CPU"):
        ops.create_dec_config(ctx, 8, cs, rs, thr.cuda())
    with pytest.raises(RuntimeError, match="same data type"):
        ops.create_dec_config(ctx, 8, cs, rs.float(), thr)
    with pytest.raises(RuntimeError, match="Data type mismatch between DECConfig and DECContext"):
        ops.create_dec_config(ctx, 8, cs, rs.float(), thr.float())
    with pytest.raises(RuntimeError, match="buffer size is too small"):
        ops.create_dec_config(ctx, 128, cs, rs, thr)
    cfg = ops.create_dec_config(ctx, 8, cs, rs, thr)
    with pytest.raises(RuntimeError, match="Mismatched data types between input tensor and DECConfig"):
        ops.dec(cfg, x.float(), y.float())
    with pytest.raises(RuntimeError, match="does not match with DECConfig"):
        ops.dec(cfg, x[:, :, :512].contiguous(), y)
    ops.destroy_dec_config(cfg)


def test_residual_on_device_and_graph_capture(ops):
    """q_residual may live on the GPU (reference: warning, no zero-copy); the fused call is
    capturable in a CUDA graph and replays with new activations."""
    N, K = 512, 2048
    L = P.random_bcq_layer(N, K, 3, 128, seed=5)
    cs, rs = P.random_residual(N, K, seed=6)
    thr = P.make_thresholds(K)
    ctx, rows, acts = _ctx(ops, 8, 1024, "fp16")
    cfg = ops.create_dec_config(ctx, 16, cs.cuda(), rs.cuda(), thr)
    qw, al, qb = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda()
    xbuf = P.make_activation(K, seed=7).cuda()
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        ops.dec_lutgemm(cfg, xbuf, y, qw, al, qb, 3, 128)     # warm-up allocates the stream's workspace
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y.zero_()
        ops.dec_lutgemm(cfg, xbuf, y, qw, al, qb, 3, 128)
    for seed in (8, 9):
        x = P.make_activation(K, seed=seed)
        xbuf.copy_(x.cuda())
        g.replay()
        torch.cuda.synchronize()
        exp_rows, exp_acts, _ = P.expected_selection(x, thr, 16, "fp16")
        delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
        _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x), None, delta), "fp16", "graph replay")


def test_graphs_captured_on_fresh_streams_have_their_own_workspace(ops):
    """A stream that the library first sees during capture cannot allocate; it is given one of the workspaces set aside
    at the device's first call.  Two graphs captured on two such streams, with layers of the same width (so that they
    would meet on the same accumulator words if they shared a workspace), are replayed side by side on two streams many
    times and must both keep giving the eager result bit for bit (the packed sums do not depend on arrival order)."""
    N, K = 4096, 4096
    layers, want, ys, graphs = [], [], [], []
    for seed in (31, 32):
        L = P.random_bcq_layer(N, K, 3, 128, seed=seed)
        x = P.make_activation(K, seed=seed + 10).cuda()
        t = (x, L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda())
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        ops.lutgemm_gemv(t[0], y, t[1], t[2], t[3], 3, 128)           # eager, on the current stream
        layers.append(t)
        want.append(y.clone())
    torch.cuda.synchronize()
    for t in layers:
        cap = torch.cuda.Stream()                                      # never used before the capture
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=cap):
            y.zero_()
            ops.lutgemm_gemv(t[0], y, t[1], t[2], t[3], 3, 128)
        ys.append(y)
        graphs.append(g)
    run = [torch.cuda.Stream(), torch.cuda.Stream()]
    for _ in range(200):
        for g, s in zip(graphs, run):
            with torch.cuda.stream(s):
                g.replay()
    torch.cuda.synchronize()
    for y, w in zip(ys, want):
        assert torch.equal(y, w)
    assert ops.stream_status() == 0


def test_wait_that_runs_out_is_reported_and_recoverable(ops):
    """Device-side failure handling without a GPU fault: under a test-only launch flag the producer of the pipelined
    binary-coded GEMV never issues its last stage (nothing is in flight for it), so the consumers' wait for that stage,
    given a 2 ms limit, runs out.  The launch must return, leave y untouched, raise the stream's error word, make the
    next call fail loudly, and after a reset the stream must compute correctly again."""
    N, K = 1024, 2048
    L = P.random_bcq_layer(N, K, 3, 128, seed=77)
    x = P.make_activation(K, seed=78)
    y0 = _y0(N, "fp16")
    y = y0.clone().cuda()
    qw, al, qb, xd = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), x.cuda()
    ops.lutgemm_gemv(xd, torch.zeros_like(y), qw, al, qb, 3, 128)      # workspace exists, kernel configured
    torch.cuda.synchronize()
    assert ops.stream_status() == 0
    os.environ["DECDEC_TEST_WITHHOLD_STAGE"] = "1"
    os.environ["DECDEC_PIPE_WAIT_NS"] = "2000000"
    try:
        ops.lutgemm_gemv(xd, y, qw, al, qb, 3, 128)
        torch.cuda.synchronize()
    finally:
        del os.environ["DECDEC_TEST_WITHHOLD_STAGE"]
        del os.environ["DECDEC_PIPE_WAIT_NS"]
    assert ops.stream_status() == 1, "the wait that ran out was not reported"
    assert torch.equal(y.cpu(), y0), "an unfinished launch must not touch the output"
    with pytest.raises(RuntimeError, match="gave up waiting"):
        ops.lutgemm_gemv(xd, y, qw, al, qb, 3, 128)
    ops.stream_reset()
    assert ops.stream_status() == 0
    ops.lutgemm_gemv(xd, y, qw, al, qb, 3, 128)
    torch.cuda.synchronize()
    _assert_close(y, ofw.layer_output(L["w_hat"], P.to_np(x), P.to_np(y0)), "fp16", "call after reset")
