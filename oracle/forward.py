"""Reference arithmetic of one decode-step linear layer with error compensation (CPU oracle).

Test infrastructure only.  `dec_delta`/`layer_output` give float64 ground truth for the parity
tests; `cpu_reference_linear` is the reference's PyTorch math (dequantise, exact per-chunk top-k,
two mat-vecs) used as the timed CPU baseline.  Paths are relative to the SNU-ARC/DecDEC repository.
"""
from __future__ import annotations

import numpy as np
import torch

from . import formats, residual, selection


def dec_delta(x: np.ndarray, rows: np.ndarray, cheatsheet: np.ndarray, reordered_scales: np.ndarray,
              acts: np.ndarray | None = None) -> np.ndarray:
    """Compensation term added to the layer output, float64 [N].

    delta[8c+i] = scale[8c+i] * sum_r (nibble_i(cheatsheet[r, c]) - 8) * act_r over the selected
    rows r (`decdec_extension/dec.cu:231-256`).  `acts` defaults to x[rows] (what `dec_kernel`
    gathers, `dec.cu:346`); the fused kernel uses the activations recorded at selection time.
    """
    x = np.asarray(x, np.float64).reshape(-1)
    rows = np.asarray(rows, np.int64)
    if acts is None:
        acts = x[rows]
    w = cheatsheet.view(np.uint32)[rows]  # [k, N/8]
    nib = ((w[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.float64) - 8.0
    nc = cheatsheet.shape[1]
    s = (nib * np.asarray(acts, np.float64)[:, None, None]).sum(0)  # [N/8, 8]
    scales = np.asarray(reordered_scales, np.float64).reshape(8, nc).T  # [N/8, 8]
    return (s * scales).reshape(-1)


def layer_output(w_hat: np.ndarray, x: np.ndarray, y0: np.ndarray | None = None,
                 delta: np.ndarray | None = None) -> np.ndarray:
    """y = y0 + W_hat @ x (+ delta) in float64.  All entry points accumulate into the output
    (`end-to-end/APLinear.py:51`, `evaluation/evaltools.py:355-359`)."""
    y = np.asarray(w_hat, np.float64) @ np.asarray(x, np.float64).reshape(-1)
    if y0 is not None:
        y = y + np.asarray(y0, np.float64).reshape(-1)
    if delta is not None:
        y = y + delta
    return y


# ----------------------------------------------------------------------------------------------
# Timed CPU baseline: the reference's PyTorch math on host cores (float32)
# ----------------------------------------------------------------------------------------------


@torch.no_grad()
def torch_bcq_dequant(qweight: torch.Tensor, alpha: torch.Tensor, q_bias: torch.Tensor, group: int) -> torch.Tensor:
    """`evaluation/evaltools.py:546-580` / `end-to-end/LUTGEMMLinear.py:41-82` in float32 on CPU.
    Returns W^T [K, N]."""
    kw, b, n = qweight.shape
    k = kw * 32
    shifts = torch.arange(32, dtype=torch.int32)
    bits = ((qweight.unsqueeze(-1) >> shifts) & 1).to(torch.uint8)
    bits = bits.permute(0, 3, 1, 2).reshape(k, b, n)
    delta = bits.to(torch.float32).mul_(2).sub_(1)
    gidx = torch.div(torch.arange(k), group, rounding_mode="floor").long()
    delta.mul_(alpha.float()[gidx])
    return delta.sum(dim=1) + q_bias.float()[gidx]


@torch.no_grad()
def torch_lut_dequant(codes: torch.Tensor, lut: torch.Tensor) -> torch.Tensor:
    """`decdec_setup/conv_sqllm.py:76-87`: W[n,k] = lut[n, codes[n,k]] (float32)."""
    return lut.float().gather(1, codes.long())


@torch.no_grad()
def torch_unpack_residual(cheatsheet: torch.Tensor, reordered_scales: torch.Tensor) -> torch.Tensor:
    """Dense residual R^T [K, N] float32 from the packed format of `decdec_setup/cheatsheet.py:99-125`."""
    k, nc = cheatsheet.shape
    sh = (torch.arange(8, dtype=torch.int32) * 4)
    nib = ((cheatsheet.unsqueeze(-1) >> sh) & 0xF).to(torch.float32) - 8.0  # [K, N/8, 8]
    scales = reordered_scales.float().reshape(8, nc).t()  # [N/8, 8]
    return (nib * scales).reshape(k, nc * 8)


@torch.no_grad()
def cpu_reference_linear(x: torch.Tensor, wt: torch.Tensor, rt: torch.Tensor | None, k_chunk: int) -> torch.Tensor:
    """One decode-step linear on CPU: y = x @ W^T + x[sel] @ R^T[sel], with `sel` the exact top
    k_chunk of |x| inside every 1024-channel chunk (`evaluation/evaltools.py:327-343` applied per
    chunk).  x: [K] float32, wt: [K, N] float32, rt: [K, N] float32 or None."""
    y = x @ wt
    if rt is not None and k_chunk > 0:
        K = x.shape[0]
        sel = []
        for s in range(0, K, 1024):
            e = min(s + 1024, K)
            kq = k_chunk * (e - s) // 1024
            if kq:
                sel.append(torch.topk(x[s:e].abs(), kq).indices + s)
        if sel:
            idx = torch.cat(sel)
            y = y + x[idx] @ rt[idx]
    return y


__all__ = [
    "dec_delta", "layer_output", "torch_bcq_dequant", "torch_lut_dequant", "torch_unpack_residual",
    "cpu_reference_linear", "formats", "residual", "selection",
]
