"""Producers and loaders of the compensation artifacts (`cheatsheet.pt`, `thresholds.pt`).

The kernels consume three tensors per linear layer: `q_residual int32 [K, N/8]` (4-bit residual, eight output
rows per word), `reordered_scales [N]` (per-output-row scale, stored nibble-major: entry i*N/8 + c belongs to output
row 8c + i) and `thresholds [K]` (calibration statistic of which entries [0] and [k-1] become the bucket bounds).
The reference produces them offline with `decdec_setup/cheatsheet.py` and `decdec_setup/thresholds.py` and assembles
them per model layer in `end-to-end/loader.py:112-195`.  This module provides the same pieces as a library (torch
tensors on any device), with two defects of that loader resolved:

  * fused projections (q/k/v -> wqkv, gate/up -> w1w3): the residual words concatenate along the output dimension,
    but `reordered_scales` cannot be concatenated as stored, because the nibble-major layout depends on the TOTAL
    output width (the loader does concatenate them, `loader.py:130-137,162-168`).  `fuse_projections` un-reorders
    every part, concatenates, and reorders for the fused width.
  * the down projection (`w2`) gets its `q_residual` and `scales` entries too (the loader's binary-coded branch only
    sets its thresholds, `loader.py:145-150,193`).

File formats are the reference's: `cheatsheet.pt` = list over layers of {module_name: {'cheatsheet', 'reordered_scales'}}
(`cheatsheet.py:125,239`), `thresholds.pt` = list over layers of {module_name: tensor[K]} (`thresholds.py:158-208`).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Sequence, Tuple

import torch

POSITIVE_LEVELS = 7      # 4-bit symmetric: codes -7..7 (nibble = code + 8)
SCALE_GRID = 32          # candidate scales per output row


# ---------------------------------------------------------------------------------------------------------
# residual quantizer and packer
# ---------------------------------------------------------------------------------------------------------

@torch.no_grad()
def quantize_residual(error: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """4-bit residual of one layer: per output row, the scale among 32 candidates (max|row|/7 * j/32) with the
    smallest squared reconstruction error (`decdec_setup/cheatsheet.py:59-86`).

    error: [N, K] = W - dequant(W), normally fp16.  Returns (codes int8 [N, K] in [-7, 7], scales fp16 [N]).
    The arithmetic keeps the reference's dtypes (fp16 residual, fp32 candidates and error), one row at a time.
    """
    if error.dim() != 2:
        raise ValueError("error must be [out_features, in_features]")
    n, k = error.shape
    scales = torch.zeros(n, dtype=torch.float16, device=error.device)
    codes = torch.zeros((n, k), dtype=torch.int8, device=error.device)
    for r in range(n):
        row = error[r]
        top = torch.max(torch.abs(row)) / POSITIVE_LEVELS
        candidates = torch.linspace(top / SCALE_GRID, top, SCALE_GRID).to(error.device)
        q = torch.clamp(torch.round(row.unsqueeze(0) / candidates.unsqueeze(1)), -POSITIVE_LEVELS, POSITIVE_LEVELS)
        mse = torch.mean((row.unsqueeze(0).float() - (q * candidates.unsqueeze(1)).float()) ** 2, dim=1)
        best = torch.argmin(mse)
        scales[r] = candidates[best]
        codes[r] = q[best].to(torch.int8)
    return codes, scales


def reorder_scales(scales: torch.Tensor) -> torch.Tensor:
    """Natural order [N] -> stored order: entry i*N/8 + c = scales[8c + i] (`cheatsheet.py:119-123`)."""
    n = scales.numel()
    if n % 8:
        raise ValueError("out_features must be a multiple of 8")
    return scales.reshape(n // 8, 8).t().reshape(-1).contiguous()


def unreorder_scales(reordered: torch.Tensor) -> torch.Tensor:
    """Stored order -> natural order [N]."""
    n = reordered.numel()
    if n % 8:
        raise ValueError("out_features must be a multiple of 8")
    return reordered.reshape(8, n // 8).t().reshape(-1).contiguous()


def pack_cheatsheet(codes: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """codes [N, K] in [-8, 7], scales [N]  ->  (q_residual int32 [K, N/8], reordered_scales [N]).
    Word [k, c] holds output rows 8c..8c+7 of input channel k, row 8c+i at bits 4i, stored nibble = code + 8
    (`cheatsheet.py:99-125`; decoded by the kernels as nibble - 8, `dec.cu:245-249`)."""
    n, k = codes.shape
    if n % 8:
        raise ValueError("out_features must be a multiple of 8")
    nib = ((codes.to(torch.int64) + 8) & 0xF).t().reshape(k, n // 8, 8)
    shifts = 4 * torch.arange(8, dtype=torch.int64, device=codes.device)
    words = (nib << shifts).sum(-1)                                  # 0 .. 2^32 - 1
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words.contiguous(), reorder_scales(scales)


def unpack_cheatsheet(q_residual: torch.Tensor, reordered_scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of `pack_cheatsheet`: (codes int32 [N, K] in [-8, 7], scales [N] in natural order)."""
    k, nc = q_residual.shape
    w = q_residual.to(torch.int64) & 0xFFFFFFFF
    shifts = 4 * torch.arange(8, dtype=torch.int64, device=q_residual.device)
    nib = ((w.unsqueeze(-1) >> shifts) & 0xF).to(torch.int32) - 8      # [K, N/8, 8]
    return nib.reshape(k, nc * 8).t().contiguous(), unreorder_scales(reordered_scales)


def residual_matrix(q_residual: torch.Tensor, reordered_scales: torch.Tensor) -> torch.Tensor:
    """Dense fp32 [N, K] residual that the packed tensors stand for."""
    codes, scales = unpack_cheatsheet(q_residual, reordered_scales)
    return codes.float() * scales.float().unsqueeze(1)


# ---------------------------------------------------------------------------------------------------------
# thresholds
# ---------------------------------------------------------------------------------------------------------

class ThresholdAccumulator:
    """thresholds[r] = max over calibration tokens of the r-th largest |activation| of the token
    (the forward hook of `decdec_setup/thresholds.py:162-175`); feed activation batches, read `.value`."""

    def __init__(self, in_features: int, device=None):
        self.value = torch.zeros(in_features, dtype=torch.float32, device=device)

    @torch.no_grad()
    def update(self, activations: torch.Tensor) -> None:
        a = activations.reshape(-1, activations.shape[-1]).abs().float()
        ranked = torch.sort(a, dim=1, descending=True).values
        self.value = torch.maximum(self.value, ranked.max(dim=0).values.to(self.value.device))


def thresholds_from_calibration(activations: torch.Tensor) -> torch.Tensor:
    acc = ThresholdAccumulator(activations.shape[-1], device=activations.device)
    acc.update(activations)
    return acc.value


# ---------------------------------------------------------------------------------------------------------
# fused projections and per-model assembly
# ---------------------------------------------------------------------------------------------------------

def fuse_projections(parts: Sequence[Mapping[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Fuse projections that share their input (q/k/v, gate/up) along the output dimension.
    parts: [{'cheatsheet': int32 [K, N_i/8], 'reordered_scales': [N_i]}, ...] in output order."""
    q = torch.cat([p["cheatsheet"] for p in parts], dim=1).contiguous()
    natural = torch.cat([unreorder_scales(p["reordered_scales"]) for p in parts], dim=0)
    return {"cheatsheet": q, "reordered_scales": reorder_scales(natural)}


_ATTN_PARTS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")
_MLP_PARTS = ("mlp.gate_proj", "mlp.up_proj")


def assemble(cheatsheet_layers: Sequence[Mapping], thresholds_layers: Sequence[Mapping]) -> Dict[str, torch.Tensor]:
    """Per-layer tensors under the names the reference model uses (`end-to-end/loader.py:119-195`):
    `layers.{i}.attention.wqkv|wo.{q_residual,scales,thresholds}`, `layers.{i}.feed_forward.w1w3|w2.{...}`.
    Accepts fused (`self_attn.qkv_proj`, `mlp.gate_up_proj`) or separate projections."""
    out: Dict[str, torch.Tensor] = {}
    for i, layer in enumerate(cheatsheet_layers):
        qkv = layer["self_attn.qkv_proj"] if "self_attn.qkv_proj" in layer else fuse_projections([layer[m] for m in _ATTN_PARTS])
        w13 = layer["mlp.gate_up_proj"] if "mlp.gate_up_proj" in layer else fuse_projections([layer[m] for m in _MLP_PARTS])
        for name, entry in ((f"layers.{i}.attention.wqkv", qkv), (f"layers.{i}.attention.wo", layer["self_attn.o_proj"]),
                            (f"layers.{i}.feed_forward.w1w3", w13), (f"layers.{i}.feed_forward.w2", layer["mlp.down_proj"])):
            out[name + ".q_residual"] = entry["cheatsheet"]
            out[name + ".scales"] = entry["reordered_scales"]
    for i, layer in enumerate(thresholds_layers):
        # fused projections share their input, hence one statistic (the first part's)
        out[f"layers.{i}.attention.wqkv.thresholds"] = layer["self_attn.qkv_proj"] if "self_attn.qkv_proj" in layer else layer["self_attn.q_proj"]
        out[f"layers.{i}.attention.wo.thresholds"] = layer["self_attn.o_proj"]
        out[f"layers.{i}.feed_forward.w1w3.thresholds"] = layer["mlp.gate_up_proj"] if "mlp.gate_up_proj" in layer else layer["mlp.gate_proj"]
        out[f"layers.{i}.feed_forward.w2.thresholds"] = layer["mlp.down_proj"]
    return out


def build_layer_cheatsheet(weights: Mapping[str, torch.Tensor], dequantized: Mapping[str, torch.Tensor]) -> Dict[str, Dict[str, torch.Tensor]]:
    """One layer's entry of `cheatsheet.pt`: {module_name: {'cheatsheet', 'reordered_scales'}} from the original and
    the dequantized weights [N, K] of each module (`cheatsheet.py:_process_layer`)."""
    out = {}
    for name, w in weights.items():
        err = (w.to(torch.float16) - dequantized[name].to(torch.float16))
        codes, scales = quantize_residual(err)
        q, rs = pack_cheatsheet(codes, scales)
        out[name] = {"reordered_scales": rs.cpu(), "cheatsheet": q.cpu()}
    return out


def save_cheatsheet(path: str, layers: Sequence[Mapping]) -> None:
    torch.save(list(layers), path)


def save_thresholds(path: str, layers: Sequence[Mapping]) -> None:
    torch.save([{k: v.cpu() for k, v in layer.items()} for layer in layers], path)


def load(cheatsheet_path: str, thresholds_path: str, map_location="cpu") -> Dict[str, torch.Tensor]:
    return assemble(torch.load(cheatsheet_path, map_location=map_location), torch.load(thresholds_path, map_location=map_location))
