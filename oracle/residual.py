"""4-bit residual ("cheatsheet") quantizer, packer and threshold statistic (CPU oracle).

Test infrastructure only.  Paths are relative to the SNU-ARC/DecDEC repository.
"""
from __future__ import annotations

import numpy as np
import torch


@torch.no_grad()
def quantize_residual(error: torch.Tensor):
    """Per-output-row 4-bit symmetric quantizer with a 32-point scale grid search.

    Follows `decdec_setup/cheatsheet.py:59-86` (bit_width = 4 branch) operation by operation, in the
    same torch dtypes (fp16 residual, float32 candidate scales and MSE), vectorised over a block of
    rows instead of one Python iteration per row.

    error: [N, K] torch tensor (fp16 in the reference flow).  Returns (q int8 [N,K] in [-7,7],
    scales fp16 [N]).
    """
    n, k = error.shape
    positive_levels = 7
    grid = 32
    scales = torch.zeros(n, dtype=torch.float16)
    q = torch.zeros((n, k), dtype=torch.int8)
    for r in range(n):
        row = error[r]
        max_scale = torch.max(torch.abs(row)) / positive_levels
        to_try = torch.linspace(max_scale / grid, max_scale, grid)
        cand = torch.clamp(torch.round(row.unsqueeze(0) / to_try.unsqueeze(1)), -positive_levels, positive_levels)
        recon = cand * to_try.unsqueeze(1)
        mse = torch.mean((row.unsqueeze(0).float() - recon.float()) ** 2, dim=1)
        best = torch.argmin(mse)
        scales[r] = to_try[best]
        q[r] = cand[best].to(torch.int8)
    return q, scales


def pack_cheatsheet(q: np.ndarray, scales: np.ndarray):
    """Pack residual codes for the DEC kernel.

    Follows `decdec_setup/cheatsheet.py:99-125`: stored nibble = q + 8; word [k, c] holds output
    rows 8c..8c+7 with row 8c+i at bits 4i; reordered_scales[i*N/8 + c] = scales[8c+i].

    q: [N, K] ints in [-8, 7].  Returns (cheatsheet int32 [K, N/8], reordered_scales [N]).
    """
    q = np.asarray(q)
    n, k = q.shape
    assert n % 8 == 0
    nib = ((q.astype(np.int64) + 8) & 0xF).T.reshape(k, n // 8, 8).astype(np.uint64)  # [K, N/8, 8]
    words = (nib << (4 * np.arange(8, dtype=np.uint64))).sum(-1).astype(np.uint32)
    reordered = np.asarray(scales).reshape(n // 8, 8).T.reshape(-1).copy()
    return words.view(np.int32), reordered


def unpack_cheatsheet(cheatsheet: np.ndarray, reordered_scales: np.ndarray):
    """Inverse of `pack_cheatsheet`; nibble decode as in `decdec_extension/dec.cu:245-249`.
    Returns (q int32 [N, K] in [-8, 7], scales [N])."""
    k, nc = cheatsheet.shape
    w = cheatsheet.view(np.uint32)
    nib = ((w[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.int32) - 8
    q = nib.reshape(k, nc * 8).T.copy()
    scales = np.asarray(reordered_scales).reshape(8, nc).T.reshape(-1).copy()
    return q, scales


def thresholds_from_calibration(acts: np.ndarray) -> np.ndarray:
    """thresholds[r] = max over calibration tokens of the r-th largest |activation|.

    Follows the forward hook of `decdec_setup/thresholds.py:162-175`.  acts: [tokens, K].
    """
    s = -np.sort(-np.abs(np.asarray(acts, np.float32)), axis=1)
    return s.max(axis=0)
