"""The reference's `decdec_ext` function set (decdec_extension/bindings.cpp:17-41) over torch tensors.

Same names, positional arguments, in-place (+=) semantics and error behaviour (RuntimeError with the
reference's messages) as the pybind module of the reference; the work is done by the C ABI of
libdecdec_b200.so through `decdec_b200.capi`.  Tensors supply device memory and the current stream,
nothing else.  Handles are plain Python ints, as in the reference.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi

_DT = {torch.float32: capi.FP32, torch.float16: capi.FP16, torch.bfloat16: capi.BF16}

# Python objects the C side borrows (thresholds storage, selection buffers) are kept alive here,
# keyed by handle, because callers of the reference API are free to drop their own references.
_KEEP: dict[int, tuple] = {}


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _dt(t: torch.Tensor) -> int:
    _check(t.dtype in _DT, "Unsupported data type.")
    return _DT[t.dtype]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _call(name: str, *args) -> None:
    try:
        capi.call(name, *args)
    except capi.DecdecError as e:  # same exception type the pybind module raises
        raise RuntimeError(str(e)) from None


def _io_checks(input: torch.Tensor, output: torch.Tensor) -> None:
    _check(input.dtype == output.dtype,
           f"Mismatched data types between input and output tensors. input type: {input.dtype}, output type: {output.dtype}")
    _check(input.is_cuda and output.is_cuda, "input and output tensors must be on GPU.")
    _check(input.dim() == 3, "input tensor must be of shape (batch_size, seq_len, hidden_size).")
    _check(output.dim() == 3, "output tensor must be of shape (batch_size, seq_len, hidden_size).")
    _check(input.size(0) == 1, "Batch size must be 1 for input tensor.")
    _check(output.size(0) == 1, "Batch size must be 1 for output tensor.")
    _check(input.size(1) == 1, "Sequence length must be 1 for input tensor.")
    _check(output.size(1) == 1, "Sequence length must be 1 for output tensor.")
    _check(input.is_contiguous(), "input tensor must be contiguous.")
    _check(output.is_contiguous(), "output tensor must be contiguous.")


# ---- context / config ---------------------------------------------------------------------------

def create_dec_context(num_tb: int, selected_rows_buffer: torch.Tensor, selected_activations_buffer: torch.Tensor) -> int:
    """reference: dec_context.cu:62-103"""
    _check(selected_rows_buffer.is_cuda, "selected_rows_buffer must be on GPU.")
    _check(selected_activations_buffer.is_cuda, "selected_activations_buffer must be on GPU.")
    _check(selected_rows_buffer.numel() == selected_activations_buffer.numel(),
           "selected_rows_buffer and selected_activations_buffer must be of the same size.")
    _check(selected_rows_buffer.dtype == torch.int32, "selected_rows_buffer must be of type int.")
    _check(selected_rows_buffer.is_contiguous(), "selected_rows_buffer must be contiguous.")
    _check(selected_activations_buffer.is_contiguous(), "selected_activations_buffer must be contiguous.")
    h = C.c_size_t(0)
    with torch.cuda.device(selected_rows_buffer.device):
        _call("decdec_create_context", int(num_tb), selected_rows_buffer.data_ptr(),
              selected_activations_buffer.data_ptr(), selected_activations_buffer.numel(),
              _dt(selected_activations_buffer), C.byref(h))
    _KEEP[h.value] = (selected_rows_buffer, selected_activations_buffer)
    return int(h.value)


def create_dec_config(dec_context: int, k_chunk: int, q_residual: torch.Tensor, reordered_scales: torch.Tensor,
                      thresholds: torch.Tensor) -> int:
    """reference: dec_config.cu:247-292"""
    _check(thresholds.device.type == "cpu", "thresholds must be on CPU.")
    _check(reordered_scales.dtype == thresholds.dtype, "reordered_scales and thresholds must have the same data type.")
    _check(q_residual.dtype == torch.int32, "q_residual must be of type int.")
    _check(q_residual.is_contiguous(), "q_residual must be contiguous.")
    _check(reordered_scales.is_contiguous(), "reordered_scales must be contiguous.")
    _check(thresholds.is_contiguous(), "thresholds must be contiguous.")
    _check(q_residual.dim() == 2 and reordered_scales.dim() == 1, "q_residual must be [K, N/8] and reordered_scales [N].")
    K, N = q_residual.size(0), reordered_scales.size(0)
    _check(q_residual.size(1) * 8 == N, "q_residual must have out_features / 8 columns.")
    _check(thresholds.numel() >= K, "thresholds must have in_features entries.")
    if q_residual.is_cuda:
        print("DecDEC WARNING: q_residual is on GPU. This is NOT the intended setup; zero-copy memory will NOT be used.")
    h = C.c_size_t(0)
    dev = q_residual.device if q_residual.is_cuda else (reordered_scales.device if reordered_scales.is_cuda else None)
    ctx_bufs = _KEEP.get(int(dec_context))
    if dev is None and ctx_bufs is not None:
        dev = ctx_bufs[0].device
    with torch.cuda.device(dev):
        _call("decdec_create_config", int(dec_context), int(k_chunk), q_residual.data_ptr(), int(q_residual.is_cuda),
              K, N, reordered_scales.data_ptr(), int(reordered_scales.is_cuda), thresholds.data_ptr(),
              _dt(reordered_scales), C.byref(h))
    _KEEP[h.value] = (thresholds, q_residual if q_residual.is_cuda else None)
    return int(h.value)


def read_dec_config(dec_config: int) -> dict:
    """reference: dec_config.cu:337-354"""
    info = capi.ConfigInfo()
    _call("decdec_read_config", int(dec_config), C.byref(info))
    return info.as_dict()


def update_dec_config(dec_config: int, new_dec_context: int, k_chunk: int) -> None:
    """reference: dec_config.cu:295-326"""
    _call("decdec_update_config", int(dec_config), int(new_dec_context), int(k_chunk))


def destroy_dec_config(dec_config: int) -> None:
    """reference: dec_config.cu:329-334"""
    _call("decdec_destroy_config", int(dec_config))
    _KEEP.pop(int(dec_config), None)


# ---- compensation alone ---------------------------------------------------------------------------

def dec(dec_config: int, input: torch.Tensor, output: torch.Tensor) -> None:
    """reference: decdec.cu:93-146"""
    _io_checks(input, output)
    with torch.cuda.device(input.device):
        _call("decdec_dec", int(dec_config), input.data_ptr(), output.data_ptr(), input.size(2), output.size(2),
              _dt(input), _stream())


def unfused_dec(dec_config: int, input: torch.Tensor, output: torch.Tensor) -> None:
    """reference: decdec.cu:196-245"""
    _io_checks(input, output)
    with torch.cuda.device(input.device):
        _call("decdec_unfused_dec", int(dec_config), input.data_ptr(), output.data_ptr(), input.size(2),
              output.size(2), _dt(input), _stream())


# ---- base GEMVs --------------------------------------------------------------------------------------

def _anyprec_checks(input, output, qweight, lut, bitwidth):
    _check(3 <= bitwidth <= 8, "Bitwidth must be between 3 and 8.")
    _check(input.dtype == lut.dtype and input.dtype == output.dtype,
           "Mismatched data types between input, lut, and output tensors.")
    _check(qweight.dtype == torch.int32, "qweight tensor must be of type int.")
    _io_checks(input, output)
    _check(lut.dim() == 2 and lut.size(1) == (1 << bitwidth) and lut.size(0) == output.size(2),
           f"lut tensor must be of shape (output_feat, 2 ** bitwidth). Expected ({output.size(2)}, {1 << bitwidth}), "
           f"got ({lut.size(0)}, {lut.size(1) if lut.dim() > 1 else -1}).")
    _check(qweight.dim() == 3 and qweight.size(0) >= bitwidth and qweight.size(2) == input.size(2) // 32
           and qweight.size(1) == output.size(2),
           "qweight tensor must be of shape (>=bitwidth, output_feat, input_feat / 32).")
    _check(qweight.is_contiguous(), "qweight tensor must be contiguous.")
    _check(lut.is_contiguous(), "lut tensor must be contiguous.")
    _check(input.dtype != torch.float32,
           "Any-Precision GEMV does not support float data type. Please use half or bfloat16.")


def anyprec_gemv(input, output, qweight, lut, bitwidth: int) -> None:
    """reference: decdec.cu:275-333"""
    _anyprec_checks(input, output, qweight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_anyprec_gemv", input.data_ptr(), output.data_ptr(), qweight.data_ptr(), qweight.size(0),
              lut.data_ptr(), output.size(2), input.size(2), int(bitwidth), _dt(input), _stream())


def anyprec_dequant(qweight, lut, bitwidth: int) -> torch.Tensor:
    """reference: decdec.cu:339-393; returns dense [N, K] weights in lut.dtype."""
    _check(lut.dtype != torch.float32,
           "Any-Precision Dequantization does not support float data type. Please use half or bfloat16.")
    _check(qweight.dim() == 3 and qweight.dtype == torch.int32 and qweight.is_cuda and lut.is_cuda,
           "qweight must be a 3-D int tensor on GPU")
    n, k = qweight.size(1), qweight.size(2) * 32
    out = torch.empty((n, k), dtype=lut.dtype, device=qweight.device)
    with torch.cuda.device(qweight.device):
        _call("decdec_anyprec_dequant", qweight.data_ptr(), lut.data_ptr(), out.data_ptr(), n, k, int(bitwidth),
              _dt(lut), _stream())
    return out


def lutgemm_dequant(q_weight, alpha, q_bias, bitwidth: int, group_size: int) -> torch.Tensor:
    """Dense [K, N] weights of a binary-coded layer (the right operand of the prefill `x @ W`); same arithmetic as the
    reference's tensor expression, end-to-end/LUTGEMMLinear.py:41-82.  No counterpart in the reference binding."""
    _check(q_weight.dim() == 3 and q_weight.dtype == torch.int32 and q_weight.is_cuda and alpha.is_cuda and q_bias.is_cuda,
           "q_weight must be a 3-D int tensor on GPU")
    _check(alpha.dtype == q_bias.dtype, "Mismatched data types between alpha and q_bias tensors.")
    _check(q_weight.is_contiguous() and alpha.is_contiguous() and q_bias.is_contiguous(), "tensors must be contiguous.")
    k, n = q_weight.size(0) * 32, q_weight.size(2)
    _check(q_weight.size(1) == bitwidth and tuple(alpha.shape) == (k // group_size, bitwidth, n)
           and tuple(q_bias.shape) == (k // group_size, n), "q_weight/alpha/q_bias shapes do not match bitwidth and group_size.")
    out = torch.empty((k, n), dtype=alpha.dtype, device=q_weight.device)
    with torch.cuda.device(q_weight.device):
        _call("decdec_lutgemm_dequant", q_weight.data_ptr(), alpha.data_ptr(), q_bias.data_ptr(), out.data_ptr(), n, k,
              int(bitwidth), int(group_size), _dt(alpha), _stream())
    return out


def _lutgemm_checks(input, output, q_weight, alpha, q_bias, bitwidth, group_size):
    _check(1 <= bitwidth <= 8, "Bitwidth must be between 1 and 8.")
    _check(input.dtype == alpha.dtype and input.dtype == q_bias.dtype and input.dtype == output.dtype,
           "Mismatched data types between input, alpha, q_bias, and output tensors.")
    _io_checks(input, output)
    _check(q_weight.is_contiguous(), "q_weight tensor must be contiguous.")
    _check(alpha.is_contiguous(), "alpha tensor must be contiguous.")
    _check(q_bias.is_contiguous(), "q_bias tensor must be contiguous.")
    k, m = input.size(2), output.size(2)
    groups = k // group_size
    _check(q_weight.dim() == 3 and q_weight.size(0) == k // 32 and q_weight.size(1) == bitwidth and q_weight.size(2) == m,
           "q_weight tensor must be of shape (input_feat / 32, bitwidth, output_feat).")
    _check(alpha.dim() == 3 and alpha.size(0) == groups and alpha.size(1) == bitwidth and alpha.size(2) == m,
           "alpha tensor must be of shape (num_groups, bitwidth, output_feat).")
    _check(q_bias.dim() == 2 and q_bias.size(0) == groups and q_bias.size(1) == m,
           "q_bias tensor must be of shape (num_groups, output_feat).")


def lutgemm_gemv(input, output, q_weight, alpha, q_bias, bitwidth: int, group_size: int) -> None:
    """reference: decdec.cu:430-496"""
    _lutgemm_checks(input, output, q_weight, alpha, q_bias, bitwidth, group_size)
    with torch.cuda.device(input.device):
        _call("decdec_lutgemm_gemv", input.data_ptr(), output.data_ptr(), q_weight.data_ptr(), alpha.data_ptr(),
              q_bias.data_ptr(), output.size(2), input.size(2), int(bitwidth), int(group_size), _dt(input), _stream())


def _sqllm_checks(input, output, qweight, lut, bitwidth):
    _check(bitwidth in (3, 4), "Bitwidth must be 3 or 4.")
    _check(input.dtype == lut.dtype and input.dtype == output.dtype,
           "Mismatched data types between input, lut, and output tensors.")
    _check(qweight.dtype == torch.int32, "qweight tensor must be of type int.")
    _io_checks(input, output)
    _check(lut.dim() == 2 and lut.size(1) == (1 << bitwidth) and lut.size(0) == output.size(2),
           "lut tensor must be of shape (output_feat, 2 ** bitwidth).")
    _check(qweight.dim() == 2 and qweight.size(1) == lut.size(0) and qweight.size(0) == input.size(2) * bitwidth // 32,
           "qweight tensor must be of shape (input_feat * bitwidth / 32, output_feat).")
    _check(qweight.is_contiguous(), "qweight tensor must be contiguous.")
    _check(lut.is_contiguous(), "lut tensor must be contiguous.")


def sqllm_gemv(input, output, qweight, lut, bitwidth: int) -> None:
    """reference: decdec.cu:544-603"""
    _sqllm_checks(input, output, qweight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_sqllm_gemv", input.data_ptr(), output.data_ptr(), qweight.data_ptr(), lut.data_ptr(),
              output.size(2), input.size(2), int(bitwidth), _dt(input), _stream())


# ---- fused -------------------------------------------------------------------------------------------

def dec_anyprec(dec_config: int, input, output, qweight, lut, bitwidth: int) -> None:
    """reference: decdec.cu:609-659"""
    _check(input.dtype in (torch.float16, torch.bfloat16), "Unsupported data type.")
    _anyprec_checks(input, output, qweight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_dec_anyprec", int(dec_config), input.data_ptr(), output.data_ptr(), qweight.data_ptr(),
              qweight.size(0), lut.data_ptr(), output.size(2), input.size(2), int(bitwidth), _dt(input), _stream())


def dec_lutgemm(dec_config: int, input, output, q_weight, alpha, q_bias, bitwidth: int, group_size: int) -> None:
    """reference: decdec.cu:665-721"""
    _lutgemm_checks(input, output, q_weight, alpha, q_bias, bitwidth, group_size)
    with torch.cuda.device(input.device):
        _call("decdec_dec_lutgemm", int(dec_config), input.data_ptr(), output.data_ptr(), q_weight.data_ptr(),
              alpha.data_ptr(), q_bias.data_ptr(), output.size(2), input.size(2), int(bitwidth), int(group_size),
              _dt(input), _stream())


def dec_sqllm(dec_config: int, input, output, q_weight, lut, bitwidth: int) -> None:
    """reference: decdec.cu:727-779"""
    _sqllm_checks(input, output, q_weight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_dec_sqllm", int(dec_config), input.data_ptr(), output.data_ptr(), q_weight.data_ptr(),
              lut.data_ptr(), output.size(2), input.size(2), int(bitwidth), _dt(input), _stream())


# ---- GEMV beside an SM-occupying busy kernel ------------------------------------------------------------

def dummy_anyprec(input, output, qweight, lut, bitwidth: int, dummy_sm: int, dummy_iters: int) -> None:
    """reference: decdec.cu:874-893"""
    _check(input.dtype in (torch.float16, torch.bfloat16), "dummy_anyprec supports FP16/BF16 only.")
    _anyprec_checks(input, output, qweight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_dummy_anyprec", input.data_ptr(), output.data_ptr(), qweight.data_ptr(), qweight.size(0),
              lut.data_ptr(), output.size(2), input.size(2), int(bitwidth), _dt(input), int(dummy_sm),
              int(dummy_iters), _stream())


def dummy_lutgemm(input, output, qweight, alpha, qbias, bitwidth: int, group_size: int, dummy_sm: int,
                  dummy_iters: int) -> None:
    """reference: decdec.cu:930-956"""
    _lutgemm_checks(input, output, qweight, alpha, qbias, bitwidth, group_size)
    with torch.cuda.device(input.device):
        _call("decdec_dummy_lutgemm", input.data_ptr(), output.data_ptr(), qweight.data_ptr(), alpha.data_ptr(),
              qbias.data_ptr(), output.size(2), input.size(2), int(bitwidth), int(group_size), _dt(input),
              int(dummy_sm), int(dummy_iters), _stream())


def dummy_sqllm(input, output, qweight, lut, bitwidth: int, dummy_sm: int, dummy_iters: int) -> None:
    """reference: decdec.cu:990-1013"""
    _check(bitwidth in (3, 4), "SQLLM bitwidth must be 3 or 4.")
    _sqllm_checks(input, output, qweight, lut, bitwidth)
    with torch.cuda.device(input.device):
        _call("decdec_dummy_sqllm", input.data_ptr(), output.data_ptr(), qweight.data_ptr(), lut.data_ptr(),
              output.size(2), input.size(2), int(bitwidth), _dt(input), int(dummy_sm), int(dummy_iters), _stream())


__all__ = [
    "create_dec_context", "create_dec_config", "read_dec_config", "update_dec_config", "destroy_dec_config",
    "dec", "unfused_dec", "anyprec_dequant", "anyprec_gemv", "lutgemm_gemv", "sqllm_gemv",
    "dec_anyprec", "dec_lutgemm", "dec_sqllm", "dummy_anyprec", "dummy_lutgemm", "dummy_sqllm",
]


# ---- additions without a counterpart in the reference binding -------------------------------------------

def stream_status() -> int:
    """Error word of the current stream's workspace (0 = fine; 1 = a bounded wait inside a kernel ran out,
    2 = a launch did not get the shared-memory layout it was sized for).  Does not synchronise."""
    err = C.c_uint32(0)
    _call("decdec_stream_status", _stream(), C.byref(err))
    return int(err.value)


def stream_reset() -> None:
    """Waits for the current stream, clears its error word and its accumulator workspace."""
    _call("decdec_stream_reset", _stream())

