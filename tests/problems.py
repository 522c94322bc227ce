"""Seeded synthetic problems for the parity tests (shapes and value distributions of the
benchmark configurations: N(0,1) activations with a fixed 1% of channels scaled x20, N(0,0.02) weights; they stand in for
real checkpoints and calibration data)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import formats, residual, selection

TORCH_DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def outlier_channels(K: int) -> np.ndarray:
    """The fixed 1% subset of channels that carry x20 outliers (same for calibration and test)."""
    return np.random.default_rng(1234 + K).choice(K, size=max(1, K // 100), replace=False)


def make_activation(K: int, seed: int, dtype: str = "fp16") -> torch.Tensor:
    """x[1,1,K] ~ N(0,1) with the outlier subset scaled x20, rounded to `dtype`."""
    x = np.random.default_rng(seed).standard_normal(K).astype(np.float32)
    x[outlier_channels(K)] *= 20.0
    return torch.from_numpy(x).to(TORCH_DT[dtype]).reshape(1, 1, K)


def make_thresholds(K: int, dtype: str = "fp16", n_calib: int = 256, seed: int = 99) -> torch.Tensor:
    """thresholds[K] from seeded calibration activations (statistic of thresholds.py:162-175)."""
    rng = np.random.default_rng(seed)
    acts = rng.standard_normal((n_calib, K)).astype(np.float32)
    acts[:, outlier_channels(K)] *= 20.0
    acts = torch.from_numpy(acts).to(TORCH_DT[dtype]).float().numpy()
    return torch.from_numpy(residual.thresholds_from_calibration(acts)).to(TORCH_DT[dtype])


def to_np(t: torch.Tensor) -> np.ndarray:
    """Exact float64 view of a torch tensor of any float dtype."""
    return t.detach().cpu().to(torch.float64).numpy()


def make_weight(N: int, K: int, seed: int) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal((N, K)) * 0.02).astype(np.float16).astype(np.float32)


def random_residual(N: int, K: int, seed: int, dtype: str = "fp16"):
    """Random packed residual (nibbles 1..15) and scales: enough for kernel parity at large shapes."""
    rng = np.random.default_rng(seed)
    q = rng.integers(-7, 8, size=(N, K), dtype=np.int8)
    scales = (rng.random(N).astype(np.float32) * 1e-3 + 2e-4)
    scales_t = torch.from_numpy(scales).to(TORCH_DT[dtype])
    cs, rs = residual.pack_cheatsheet(q, scales_t.float().numpy())
    return torch.from_numpy(cs.copy()), torch.from_numpy(rs.copy()).to(TORCH_DT[dtype])


def quantized_residual(w: np.ndarray, w_fake: np.ndarray, dtype: str = "fp16"):
    """Residual of a real quantization, through the reference's quantizer math (cheatsheet.py)."""
    err = torch.from_numpy(w.astype(np.float32) - w_fake.astype(np.float32)).to(torch.float16)
    q, scales = residual.quantize_residual(err)
    cs, rs = residual.pack_cheatsheet(q.numpy(), scales.float().numpy())
    return torch.from_numpy(cs.copy()), torch.from_numpy(rs.copy()).to(TORCH_DT[dtype])


def bcq_layer(N: int, K: int, bits: int, group: int, seed: int, dtype: str = "fp16"):
    """Uniform group quantization converted to binary-coded tensors; returns torch tensors + dense W_hat."""
    w = make_weight(N, K, seed)
    w_fake, s, z, codes = formats.pseudo_quantize_uniform(w, bits, group)
    qw, alpha, qb = formats.uniform_to_bcq(s, z, codes, bits)
    alpha_t = torch.from_numpy(alpha).to(TORCH_DT[dtype])
    qb_t = torch.from_numpy(qb).to(TORCH_DT[dtype])
    w_hat = formats.bcq_dequant(qw, to_np(alpha_t), to_np(qb_t), group)
    return dict(w=w, w_fake=w_fake, qweight=torch.from_numpy(qw.copy()), alpha=alpha_t, q_bias=qb_t, w_hat=w_hat)


def random_bcq_layer(N: int, K: int, bits: int, group: int, seed: int, dtype: str = "fp16"):
    """Random planes / alpha / bias (no quantizer): exercises the kernel at any bit width quickly."""
    rng = np.random.default_rng(seed)
    qw = rng.integers(-2**31, 2**31, size=(K // 32, bits, N), dtype=np.int64).astype(np.int32)
    alpha = torch.from_numpy((rng.random((K // group, bits, N), dtype=np.float32) * 0.01)).to(TORCH_DT[dtype])
    qb = torch.from_numpy(((rng.random((K // group, N), dtype=np.float32) - 0.5) * 0.01)).to(TORCH_DT[dtype])
    w_hat = formats.bcq_dequant(qw, to_np(alpha), to_np(qb), group)
    return dict(qweight=torch.from_numpy(qw), alpha=alpha, q_bias=qb, w_hat=w_hat)


def lut_layer(N: int, K: int, bits: int, seed: int, dtype: str = "fp16", fmt: str = "anyprec", real: bool = True):
    """Per-row LUT quantization packed for the any-precision or SqueezeLLM kernels."""
    rng = np.random.default_rng(seed)
    if real:
        w = make_weight(N, K, seed)
        lut, codes = formats.lut_quantize(w, bits)
        lut_t = torch.from_numpy(lut).to(TORCH_DT[dtype])
    else:
        w = None
        codes = rng.integers(0, 2 ** bits, size=(N, K), dtype=np.int64).astype(np.int32)
        lut_t = torch.from_numpy((rng.standard_normal((N, 2 ** bits)) * 0.02).astype(np.float32)).to(TORCH_DT[dtype])
    w_hat = formats.lut_dequant(to_np(lut_t), codes)
    if fmt == "anyprec":
        qw = formats.anyprec_pack(codes, bits)
    else:
        qw = formats.sqllm_pack(codes, bits)
    return dict(w=w, codes=codes, qweight=torch.from_numpy(qw.copy()), lut=lut_t, w_hat=w_hat)


def expected_selection(x: torch.Tensor, thresholds: torch.Tensor, k_chunk: int, dtype: str):
    K = x.numel()
    k = k_chunk * K // 1024
    if k == 0:
        return np.zeros(0, np.int32), np.zeros(0), None
    thr = to_np(thresholds)
    return selection.select(to_np(x).reshape(-1), thr[0], thr[k - 1], k_chunk, dtype)


def errors(y: torch.Tensor, ref: np.ndarray):
    d = to_np(y).reshape(-1) - ref
    return float(np.abs(d).max()), float(np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-30))
