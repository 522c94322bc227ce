"""Tensor-parallel sharding of one quantized linear layer with error compensation.

The reference is single-GPU (no collective anywhere in SNU-ARC/DecDEC); this module defines how its
per-layer tensors are cut so that the same kernels run unchanged on every rank:

  column-parallel (q/k/v, gate/up): outputs N are split.  Every rank sees the full activation, so
      the channel selection is identical on all ranks and nothing is exchanged.  The residual shard
      is q_residual[:, n0/8:n1/8]; `reordered_scales` is re-derived per shard because its layout
      [nibble][N_local/8] depends on the shard width (decdec_extension/dec.cu:223-224).
  row-parallel (o, down): inputs K are split at multiples of the 1024-channel selection chunk
      (decdec_extension/macros.h:8) so that chunk-local selection equals the single-GPU selection; with
      fewer chunks than ranks the ranks that share a chunk split its outputs (`row_plan`).
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


def row_plan(K: int, N: int, world: int) -> List[Tuple[int, int, int, int]]:
    """Row-parallel plan: (k0, k1, n0, n1) per rank.  The input range of a rank is a whole number of
    1024-channel selection chunks, so that chunk-local selection equals the single-GPU selection.
      * K has at least `world` chunks: the chunks are dealt out as evenly as they go (28 chunks over 8 ranks:
        4,4,4,4,3,3,3,3) and every rank produces all N outputs;
      * fewer chunks than ranks: every chunk is shared by world / chunks ranks, which split its OUTPUTS
        (a rank computes the partial sums of its output range over its chunk); world must be a multiple of
        the chunk count.
    In both cases the partial outputs, written into a zeroed [N] vector, are summed by one all-reduce.
    A shard narrower than one chunk would select other channels than the unsharded layer
    (decdec_extension/dec.cu:84-86 applies the quota per chunk), so it is refused."""
    if K % CHUNK:
        raise ValueError(f"row-parallel sharding needs in_features to be a multiple of {CHUNK} (got {K}): a partial chunk "
                         "cannot be cut without changing the channel selection")
    chunks = K // CHUNK
    if chunks >= world:
        return [(k0, k1, 0, N) for k0, k1 in split_even(K, world, CHUNK)]
    if world % chunks:
        raise ValueError(f"{chunks} selection chunks cannot be shared evenly by {world} ranks")
    per = world // chunks
    n_ranges = split_even(N, per, 128 if N % (128 * per) == 0 else 32)
    return [(c * CHUNK, (c + 1) * CHUNK, *n_ranges[i]) for c in range(chunks) for i in range(per)]


def k_ranges(K: int, world: int, group: int = 128) -> List[Tuple[int, int]]:
    """Input ranges of `row_plan` (outputs ignored)."""
    return [(k0, k1) for k0, k1, _, _ in row_plan(K, 32 * world, world)]


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
    k0, k1, n0, n1 = row_plan(K, N, world)[rank]
    k_glob = k_chunk * K // CHUNK
    k_loc = k_chunk * (k1 - k0) // CHUNK
    thr = thresholds[k0:k1].clone()
    if k_glob > 0 and k_loc > 0:
        if k_loc == 1 and k_glob > 1:
            raise ValueError("a shard that selects a single channel cannot carry both global bucket bounds (the kernel reads "
                             "thresholds[0] and thresholds[k-1]); use k_chunk >= 2 or fewer ranks")
        thr[0] = thresholds[0]
        thr[k_loc - 1] = thresholds[k_glob - 1]
    scales = reordered_scales.clone()
    if (n0, n1) != (0, N):
        scales = reorder_scales(unreorder_scales(reordered_scales)[n0:n1])
    return {"q_residual": q_residual[k0:k1, n0 // 8:n1 // 8].contiguous(), "reordered_scales": scales,
            "thresholds": thr, "k_chunk": k_chunk, "n_range": (n0, n1)}


def shard_bcq(qweight: torch.Tensor, alpha: torch.Tensor, q_bias: torch.Tensor, group: int, mode: str, rank: int,
              world: int) -> Dict[str, torch.Tensor]:
    """Binary-coded weights of one rank.  qweight [K/32, bits, N], alpha [K/group, bits, N], q_bias [K/group, N]."""
    K, N = qweight.shape[0] * 32, qweight.shape[2]
    if mode == "col":
        n0, n1 = split_even(N, world, 32)[rank]
        return {"qweight": qweight[:, :, n0:n1].contiguous(), "alpha": alpha[:, :, n0:n1].contiguous(),
                "q_bias": q_bias[:, n0:n1].contiguous()}
    k0, k1, n0, n1 = row_plan(K, N, world)[rank]
    return {"qweight": qweight[k0 // 32:k1 // 32, :, n0:n1].contiguous(), "alpha": alpha[k0 // group:k1 // group, :, n0:n1].contiguous(),
            "q_bias": q_bias[k0 // group:k1 // group, n0:n1].contiguous(), "n_range": (n0, n1)}


def shard_anyprec(qweight: torch.Tensor, lut: torch.Tensor, mode: str, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """Any-precision weights of one rank.  qweight [planes, N, K/32], lut [N, 2^bits].  Row-parallel
    shards must start and end on 1024-channel blocks, because the bit-to-channel map of a tail block
    depends on the row length (decdec_extension/anyprec.cu:297-300)."""
    N, K = qweight.shape[1], qweight.shape[2] * 32
    if mode == "col":
        n0, n1 = split_even(N, world, 32)[rank]
        return {"qweight": qweight[:, n0:n1].contiguous(), "lut": lut[n0:n1].contiguous()}
    k0, k1, n0, n1 = row_plan(K, N, world)[rank]
    return {"qweight": qweight[:, n0:n1, k0 // 32:k1 // 32].contiguous(), "lut": lut[n0:n1].contiguous(), "n_range": (n0, n1)}


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
