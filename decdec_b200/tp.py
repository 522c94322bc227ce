"""Tensor-parallel sharding of one quantized linear layer with error compensation.

The reference is single-GPU (no collective anywhere in SNU-ARC/DecDEC); this module defines how its
per-layer tensors are cut so that the same kernels run unchanged on every rank:

  column-parallel (q/k/v, gate/up): outputs N are split.  Every rank sees the full activation, so
      the channel selection is identical on all ranks and nothing is exchanged.  The residual shard
      is q_residual[:, n0/8:n1/8]; `reordered_scales` is re-derived per shard because its layout
      [nibble][N_local/8] depends on the shard width (decdec_extension/dec.cu:223-224).
  row-parallel (o, down): inputs K are split at multiples of the 1024-channel selection chunk
      (decdec_extension/macros.h:8) so that chunk-local selection equals the single-GPU selection.
      Only thresholds[0] and thresholds[k-1] are read by the kernel (decdec_extension/decdec.cu:66-67),
      so a shard keeps the global bucket bounds by carrying those two values at [0] and [k_local-1].
      Partial outputs are summed with one all-reduce of [N] values.

The sharding functions are pure tensor slicing (torch, CPU or GPU).  `PushAllReduce` is the collective for
the row-parallel outputs on GPUs of one node: a one-shot push over NVLink peer memory (CUDA kernel behind
`decdec_tp_allreduce`), set up through any `torch.distributed` process group.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

CHUNK = 1024


def split_even(total: int, world: int, unit: int) -> List[Tuple[int, int]]:
    """Cut [0, total) into `world` contiguous ranges whose sizes are multiples of `unit` and differ by
    at most one unit (total must be a multiple of unit)."""
    if total % unit:
        raise ValueError(f"{total} is not a multiple of {unit}")
    units = total // unit
    base, extra = divmod(units, world)
    out, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * unit
        out.append((start, start + n))
        start += n
    return out


def k_ranges(K: int, world: int, group: int = 128) -> List[Tuple[int, int]]:
    """Row-parallel input ranges: chunk-aligned when K has at least `world` chunks, else aligned to the
    larger of 32 (one packed word) and the scale group, with the partial-chunk selection rule applied
    inside each shard (decdec_extension/dec.cu:84-86)."""
    if K % CHUNK == 0 and K // CHUNK >= world:
        return split_even(K, world, CHUNK)
    return split_even(K, world, max(32, group))


def unreorder_scales(reordered: torch.Tensor) -> torch.Tensor:
    n = reordered.numel()
    return reordered.reshape(8, n // 8).t().reshape(-1)


def reorder_scales(scales: torch.Tensor) -> torch.Tensor:
    n = scales.numel()
    return scales.reshape(n // 8, 8).t().reshape(-1).contiguous()


def shard_residual(q_residual: torch.Tensor, reordered_scales: torch.Tensor, thresholds: torch.Tensor, k_chunk: int,
                   mode: str, rank: int, world: int, group: int = 128) -> Dict[str, torch.Tensor]:
    """Residual tensors of one rank.  q_residual [K, N/8] int32, reordered_scales [N], thresholds [K]."""
    K, N = q_residual.shape[0], reordered_scales.numel()
    if mode == "col":
        n0, n1 = split_even(N, world, 32)[rank]
        scales = unreorder_scales(reordered_scales)[n0:n1]
        return {"q_residual": q_residual[:, n0 // 8:n1 // 8].contiguous(), "reordered_scales": reorder_scales(scales),
                "thresholds": thresholds.clone(), "k_chunk": k_chunk}
    if mode != "row":
        raise ValueError(mode)
    k0, k1 = k_ranges(K, world, group)[rank]
    k_glob = k_chunk * K // CHUNK
    k_loc = k_chunk * (k1 - k0) // CHUNK
    thr = thresholds[k0:k1].clone()
    if k_glob > 0 and k_loc > 0:
        thr[0] = thresholds[0]
        thr[k_loc - 1] = thresholds[k_glob - 1]
    return {"q_residual": q_residual[k0:k1].contiguous(), "reordered_scales": reordered_scales.clone(),
            "thresholds": thr, "k_chunk": k_chunk}


def shard_bcq(qweight: torch.Tensor, alpha: torch.Tensor, q_bias: torch.Tensor, group: int, mode: str, rank: int,
              world: int) -> Dict[str, torch.Tensor]:
    """Binary-coded weights of one rank.  qweight [K/32, bits, N], alpha [K/group, bits, N], q_bias [K/group, N]."""
    K, N = qweight.shape[0] * 32, qweight.shape[2]
    if mode == "col":
        n0, n1 = split_even(N, world, 32)[rank]
        return {"qweight": qweight[:, :, n0:n1].contiguous(), "alpha": alpha[:, :, n0:n1].contiguous(),
                "q_bias": q_bias[:, n0:n1].contiguous()}
    k0, k1 = k_ranges(K, world, group)[rank]
    return {"qweight": qweight[k0 // 32:k1 // 32].contiguous(), "alpha": alpha[k0 // group:k1 // group].contiguous(),
            "q_bias": q_bias[k0 // group:k1 // group].contiguous()}


def shard_anyprec(qweight: torch.Tensor, lut: torch.Tensor, mode: str, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """Any-precision weights of one rank.  qweight [planes, N, K/32], lut [N, 2^bits].  Row-parallel
    shards must start and end on 1024-channel blocks, because the bit-to-channel map of a tail block
    depends on the row length (decdec_extension/anyprec.cu:297-300)."""
    N, K = qweight.shape[1], qweight.shape[2] * 32
    if mode == "col":
        n0, n1 = split_even(N, world, 32)[rank]
        return {"qweight": qweight[:, n0:n1].contiguous(), "lut": lut[n0:n1].contiguous()}
    k0, k1 = split_even(K, world, CHUNK)[rank]
    return {"qweight": qweight[:, :, k0 // 32:k1 // 32].contiguous(), "lut": lut}


def shard_input(x: torch.Tensor, mode: str, rank: int, world: int, group: int = 128) -> torch.Tensor:
    """Activation seen by a rank: everything (column-parallel) or its K range (row-parallel)."""
    if mode == "col":
        return x
    K = x.shape[-1]
    k0, k1 = k_ranges(K, world, group)[rank]
    return x[..., k0:k1].contiguous()


class PushAllReduce:
    """In-place sum of a [.., n] fp16/bf16/fp32 CUDA tensor over the ranks of `group`, one kernel per rank.

    Every rank allocates an exchange buffer in the CUDA library, the 64-byte IPC handles travel once through
    the process group, and each call pushes this rank's vector into the peers' buffers, waits (bounded) for
    theirs and sums in rank order - identical results on all ranks, capturable in CUDA graphs.  All ranks must
    make the same sequence of calls, and no rank may reach a call more than the bounded wait (about a second) after
    the others - put a barrier after uneven set-up work.  `check()` raises if a wait ever ran out.
    """

    _DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

    def __init__(self, max_n: int, group=None, device=None):
        import ctypes as C
        import torch.distributed as dist
        from . import capi
        self._capi, self._C = capi, C
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        handle = (C.c_ubyte * 64)()
        comm = C.c_size_t(0)
        with torch.cuda.device(self.device):
            capi.call("decdec_tp_create", self.world, self.rank, int(max_n), C.byref(comm), C.cast(handle, C.c_void_p))
        self._comm = comm.value
        mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=self.device)
        gathered = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(gathered, mine, group=group)
        blob = bytes(torch.stack(gathered).cpu().flatten().tolist())
        if self.world > 1:
            buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
            with torch.cuda.device(self.device):
                capi.call("decdec_tp_connect_ipc", self._comm, C.cast(buf, C.c_void_p))
        dist.barrier(group=group)          # every buffer is zeroed and mapped before the first push

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        if not y.is_cuda or not y.is_contiguous():
            raise ValueError("PushAllReduce needs a contiguous CUDA tensor")
        stream = torch.cuda.current_stream(y.device).cuda_stream
        self._capi.call("decdec_tp_allreduce", self._comm, y.data_ptr(), y.numel(), self._DT[y.dtype], stream)
        return y

    def status(self):
        calls, err = self._C.c_uint32(0), self._C.c_uint32(0)
        self._capi.call("decdec_tp_status", self._comm, self._C.byref(calls), self._C.byref(err))
        return int(calls.value), int(err.value)

    def check(self) -> None:
        calls, err = self.status()
        if err:
            raise RuntimeError(f"PushAllReduce: a wait for a peer ran out (after {calls} completed calls); outputs were left unsummed")

    def close(self) -> None:
        if self._comm:
            self._capi.call("decdec_tp_destroy", self._comm)
            self._comm = 0
