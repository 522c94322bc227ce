"""GPU parity at the shapes and launch geometries the benchmark and the named model configurations use.

The fused entry point is checked at
  * the timed Llama-3-8B launches (fused wqkv 4096->6144, w1w3 4096->28672, w2 14336->4096, wo 4096->4096) with
    k_chunk 32 at a thread-block budget of 96 and at the tuner's operating point (budget 16, k_chunk 5 / 3);
  * Phi-3-medium shapes (hidden 5120, FFN 17920 = 17.5 selection chunks, k_chunk 16): the partial last chunk goes
    through the fetch, not only through the selection;
  * Llama-3-70B shapes (hidden 8192, FFN 28672, k_chunk 32), whole and as the tensor-parallel shards of 2, 4 and 8
    ranks: every rank's shard runs through the CUDA kernels in turn on one GPU, the partial outputs are summed in
    fp32 and compared with the unsharded oracle, and the union of the ranks' selected channels must equal the
    single-GPU selection;
  * 4-bit binary-coded weights fused with compensation, and the mixed 3-bit / 4-bit set-up with one context per
    bit width (end-to-end/generate.py:225-233, model.py:182-198).
Outputs of wide layers are compared on a seeded subset of rows (the float64 oracle of all rows would need gigabytes);
the channel selection is always compared completely.
"""
import numpy as np
import pytest
import torch

from oracle import forward as ofw
from oracle import formats
from tests import problems as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from decdec_b200 import ops as _ops
    return _ops


def _rand_layer(N, K, bits, group, seed):
    """Random planes / alpha / bias as torch tensors (no dense matrix: rows are dequantized on demand)."""
    rng = np.random.default_rng(seed)
    qw = torch.from_numpy(rng.integers(-2**31, 2**31, size=(K // 32, bits, N), dtype=np.int64).astype(np.int32))
    alpha = torch.from_numpy(rng.random((K // group, bits, N), dtype=np.float32) * 0.01).half()
    qb = torch.from_numpy((rng.random((K // group, N), dtype=np.float32) - 0.5) * 0.01).half()
    return qw, alpha, qb


def _rand_residual(N, K, seed):
    rng = np.random.default_rng(seed)
    cs = torch.from_numpy(rng.integers(-2**31, 2**31, size=(K, N // 8), dtype=np.int64).astype(np.int32))
    rs = torch.from_numpy(rng.random(N, dtype=np.float32) * 1e-3 + 2e-4).half()
    return cs, rs


def _oracle_rows(qw, alpha, qb, group, x, idx, delta=None):
    """float64 outputs of the rows `idx` of a binary-coded layer (+ compensation term)."""
    w_hat = formats.bcq_dequant(qw[:, :, idx].numpy(), P.to_np(alpha[:, :, idx]), P.to_np(qb[:, idx]), group)
    y = ofw.layer_output(w_hat, P.to_np(x))
    return y if delta is None else y + delta[idx]


def _check_rows(y, ref, idx, what, tol=(1e-2, 1e-3)):
    got = P.to_np(y).reshape(-1)[idx]
    ma = float(np.abs(got - ref).max())
    rl = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
    assert ma <= tol[0] and rl <= tol[1], f"{what}: max abs {ma:.3e}, rel L2 {rl:.3e}"


def _fused(ops, N, K, bits, k_chunk, n_tb, seed, rows_checked=1536):
    qw, alpha, qb = _rand_layer(N, K, bits, 128, seed)
    cs, rs = _rand_residual(N, K, seed + 1)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=seed + 2)
    k = k_chunk * K // 1024
    rows = torch.full((max(k, 1),), -1, dtype=torch.int32, device="cuda")
    acts = torch.zeros(max(k, 1), dtype=torch.float16, device="cuda")
    ctx = ops.create_dec_context(n_tb, rows, acts)
    cfg = ops.create_dec_config(ctx, k_chunk, cs, rs, thr)
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.dec_lutgemm(cfg, x.cuda(), y, qw.cuda(), alpha.cuda(), qb.cuda(), bits, 128)
    torch.cuda.synchronize()
    assert ops.stream_status() == 0
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
    assert np.array_equal(rows[:k].cpu().numpy(), exp_rows), "selected channels differ from the oracle"
    assert np.array_equal(P.to_np(acts[:k]), exp_acts)
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    idx = np.sort(np.random.default_rng(seed).choice(N, size=min(N, rows_checked), replace=False))
    _check_rows(y, _oracle_rows(qw, alpha, qb, 128, x, idx, delta), idx, f"dec_lutgemm {N}x{K} b{bits} kc={k_chunk} n_tb={n_tb}")
    # second call on the same output: the workspace was left clean, the result doubles
    ops.dec_lutgemm(cfg, x.cuda(), y, qw.cuda(), alpha.cuda(), qb.cuda(), bits, 128)
    torch.cuda.synchronize()
    _check_rows(y, 2.0 * _oracle_rows(qw, alpha, qb, 128, x, idx, delta), idx, "second accumulating call", tol=(2e-2, 1e-3))
    ops.destroy_dec_config(cfg)


@pytest.mark.parametrize("N,K,k_chunk,n_tb", [
    (6144, 4096, 32, 96), (4096, 4096, 32, 96), (28672, 4096, 32, 96), (4096, 14336, 32, 96),      # the timed launches
    (28672, 4096, 5, 16), (4096, 14336, 3, 16), (6144, 4096, 3, 16), (4096, 4096, 2, 16),          # the tuner's regime
])
def test_fused_at_the_timed_geometry(ops, N, K, k_chunk, n_tb):
    _fused(ops, N, K, 3, k_chunk, n_tb, seed=N + K + k_chunk)


@pytest.mark.parametrize("N,K", [(7680, 5120), (5120, 5120), (35840, 5120), (5120, 17920)])
def test_fused_phi3_medium_shapes(ops, N, K):
    """hidden 5120 (5 chunks), FFN 17920 (17.5 chunks: the last chunk selects k_chunk / 2 channels), k_chunk 16."""
    _fused(ops, N, K, 3, 16, 40, seed=N + K)


@pytest.mark.parametrize("N,K", [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)])
def test_fused_llama3_70b_shapes(ops, N, K):
    _fused(ops, N, K, 3, 32, 96, seed=N + K, rows_checked=1024)


@pytest.mark.parametrize("N,K", [(4096, 4096), (6144, 4096), (1024, 2048)])
def test_fused_four_bit(ops, N, K):
    """4-bit binary-coded planes (the pipelined kernel's 4-plane instance) fused with compensation."""
    _fused(ops, N, K, 4, 16, 24, seed=N + K + 4)


def test_mixed_precision_two_contexts(ops):
    """Half of the layers 3-bit, half 4-bit, one context (thread-block budget) and one k_chunk set per bit width,
    all sharing the selection buffers - the "3.5-bit" set-up of the reference (generate.py:225-233)."""
    K, N = 4096, 4096
    rows = torch.full((32 * 1024,), -1, dtype=torch.int32, device="cuda")
    acts = torch.zeros(32 * 1024, dtype=torch.float16, device="cuda")
    ctx = {3: ops.create_dec_context(16, rows, acts), 4: ops.create_dec_context(32, rows, acts)}
    k_chunk = {3: 8, 4: 24}
    thr = P.make_thresholds(K)
    layers = []
    for li, bits in enumerate([3, 4, 4, 3]):
        qw, alpha, qb = _rand_layer(N, K, bits, 128, 100 + li)
        cs, rs = _rand_residual(N, K, 200 + li)
        cfg = ops.create_dec_config(ctx[bits], k_chunk[bits], cs, rs, thr)
        layers.append((bits, qw, alpha, qb, cs, rs, cfg))
    idx = np.sort(np.random.default_rng(3).choice(N, size=1024, replace=False))
    for li, (bits, qw, alpha, qb, cs, rs, cfg) in enumerate(layers):
        x = P.make_activation(K, seed=300 + li)
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        ops.dec_lutgemm(cfg, x.cuda(), y, qw.cuda(), alpha.cuda(), qb.cuda(), bits, 128)
        torch.cuda.synchronize()
        kc = k_chunk[bits]
        exp_rows, exp_acts, _ = P.expected_selection(x, thr, kc, "fp16")
        assert np.array_equal(rows[:kc * 4].cpu().numpy(), exp_rows)
        info = ops.read_dec_config(cfg)
        assert info["k_chunk"] == kc
        delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
        _check_rows(y, _oracle_rows(qw, alpha, qb, 128, x, idx, delta), idx, f"layer {li} ({bits}-bit)")
    for layer in layers:
        ops.destroy_dec_config(layer[-1])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode,N,K", [("col", 10240, 8192), ("row", 8192, 8192), ("row", 8192, 28672), ("row", 4096, 4096)])
def test_tensor_parallel_shards_on_one_gpu(ops, world, mode, N, K):
    """Every rank's shard (decdec_b200.tp) through the CUDA kernels, one after the other on this GPU; the fp32 sum
    of the partial outputs (row-parallel) or their concatenation (column-parallel) is the unsharded layer, and the
    ranks together select exactly the channels the single GPU selects."""
    from decdec_b200 import tp
    k_chunk = 32
    qw, alpha, qb = _rand_layer(N, K, 3, 128, N + K + world)
    cs, rs = _rand_residual(N, K, N + K + world + 1)
    thr = P.make_thresholds(K)
    x = P.make_activation(K, seed=world)
    exp_rows, exp_acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
    delta = ofw.dec_delta(P.to_np(x), exp_rows, cs.numpy(), P.to_np(rs), exp_acts)
    total = torch.zeros(N, dtype=torch.float32)
    selected = []
    for rank in range(world):
        w = tp.shard_bcq(qw, alpha, qb, 128, mode, rank, world)
        r = tp.shard_residual(cs, rs, thr, k_chunk, mode, rank, world)
        xs = tp.shard_input(x, mode, rank, world)
        n_loc, k_loc = w["qweight"].shape[2], w["qweight"].shape[0] * 32
        k = k_chunk * k_loc // 1024
        rows = torch.full((k,), -1, dtype=torch.int32, device="cuda")
        acts = torch.zeros(k, dtype=torch.float16, device="cuda")
        cfg = ops.create_dec_config(ops.create_dec_context(max(8, 96 // world), rows, acts), k_chunk, r["q_residual"],
                                    r["reordered_scales"], r["thresholds"])
        y = torch.zeros(1, 1, n_loc, dtype=torch.float16, device="cuda")
        ops.dec_lutgemm(cfg, xs.cuda(), y, w["qweight"].cuda(), w["alpha"].cuda(), w["q_bias"].cuda(), 3, 128)
        torch.cuda.synchronize()
        if mode == "row":
            k0 = tp.row_plan(K, N, world)[rank][0]
            n0, n1 = r["n_range"]
            total[n0:n1] += y.float().cpu().reshape(-1)
            selected.append((rows.cpu().numpy() + k0, (n0, n1)))
        else:
            n0, n1 = tp.split_even(N, world, 32)[rank]
            total[n0:n1] = y.float().cpu().reshape(-1)
            assert np.array_equal(rows.cpu().numpy(), exp_rows), "column-parallel ranks must select identically"
        ops.destroy_dec_config(cfg)
    if mode == "row":
        # ranks that share a chunk (fewer chunks than ranks) select the same channels; over the distinct input
        # ranges the union is the single-GPU selection
        union = np.unique(np.concatenate([s for s, _ in selected]))
        assert np.array_equal(union, np.sort(exp_rows)), "the ranks' selections do not add up to the single-GPU selection"
    idx = np.sort(np.random.default_rng(world).choice(N, size=1024, replace=False))
    ref = _oracle_rows(qw, alpha, qb, 128, x, idx, delta)
    got = total.numpy().astype(np.float64)[idx]
    # every rank rounds its partial output to fp16 once
    ma = float(np.abs(got - ref).max())
    rl = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    assert ma <= 1e-2 * max(1, world // 2) and rl <= 1e-3 * max(1, world // 2), f"tp{world} {mode} {N}x{K}: max abs {ma:.3e}, rel L2 {rl:.3e}"
