"""Tensor-parallel sharding on CPU ranks (gloo, world size 2): the shard planner plus one all-reduce
reproduces the unsharded layer, checked with the oracle arithmetic on every rank."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, K, N, k_chunk):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from decdec_b200 import tp
        from oracle import forward as ofw, formats
        from tests import problems as P
        L = P.random_bcq_layer(N, K, 3, 128, seed=5)
        cs, rs = P.random_residual(N, K, seed=6)
        thr = P.make_thresholds(K)
        x = P.make_activation(K, seed=7)
        # unsharded ground truth
        rows, acts, _ = P.expected_selection(x, thr, k_chunk, "fp16")
        full = ofw.layer_output(L["w_hat"], P.to_np(x), None, ofw.dec_delta(P.to_np(x), rows, cs.numpy(), P.to_np(rs), acts))
        # this rank's shard
        w = tp.shard_bcq(L["qweight"], L["alpha"], L["q_bias"], 128, mode, rank, world)
        r = tp.shard_residual(cs, rs, thr, k_chunk, mode, rank, world)
        xs = tp.shard_input(x, mode, rank, world)
        w_hat = formats.bcq_dequant(w["qweight"].numpy(), P.to_np(w["alpha"]), P.to_np(w["q_bias"]), 128)
        srows, sacts, _ = P.expected_selection(xs, r["thresholds"], r["k_chunk"], "fp16")
        delta = ofw.dec_delta(P.to_np(xs), srows, r["q_residual"].numpy(), P.to_np(r["reordered_scales"]), sacts)
        part = torch.from_numpy(ofw.layer_output(w_hat, P.to_np(xs), None, delta))
        if mode == "row":
            n0, n1 = r["n_range"]
            whole = torch.zeros(N, dtype=part.dtype)
            whole[n0:n1] = part                        # partial sums go into a zeroed [N] vector ...
            dist.all_reduce(whole)                     # ... and one all-reduce is the only exchange of the path
            assert np.allclose(whole.numpy(), full, rtol=1e-9, atol=1e-9)
            # same channels as the single-GPU selection, seen from this rank's K range
            k0, k1 = tp.k_ranges(K, world)[rank]
            glob = np.sort(rows[(rows >= k0) & (rows < k1)])
            assert np.array_equal(np.sort(srows + k0), glob)
        else:
            gathered = [torch.zeros_like(part) for _ in range(world)]
            dist.all_gather(gathered, part)            # test-only: the path itself needs no exchange here
            assert np.allclose(torch.cat(gathered).numpy(), full, rtol=1e-9, atol=1e-9)
            assert np.array_equal(srows, rows)         # identical selection on every rank
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,K,N,world", [("col", 2048, 256, 2), ("row", 4096, 128, 2), ("row", 3072, 64, 2),
                                            ("row", 1024, 256, 2)])      # last: fewer chunks than ranks, outputs split
def test_tp_shards_reproduce_the_layer(mode, K, N, world):
    mp.spawn(_worker, args=(world, _free_port(), mode, K, N, 16), nprocs=world, join=True)


def test_split_planner():
    from decdec_b200 import tp
    assert tp.k_ranges(28672, 8) == [(0, 4096), (4096, 8192), (8192, 12288), (12288, 16384), (16384, 19456), (19456, 22528),
                                     (22528, 25600), (25600, 28672)]          # 28 chunks -> 4,4,4,4,3,3,3,3
    # fewer chunks than ranks: two ranks share a chunk and split its outputs, never the chunk
    assert tp.row_plan(4096, 4096, 8) == [(c * 1024, (c + 1) * 1024, h * 2048, (h + 1) * 2048) for c in range(4) for h in range(2)]
    assert tp.row_plan(8192, 8192, 8) == [(i * 1024, (i + 1) * 1024, 0, 8192) for i in range(8)]
    with pytest.raises(ValueError):
        tp.row_plan(3072, 4096, 8)              # 3 chunks, 8 ranks
    with pytest.raises(ValueError):
        tp.row_plan(4096 + 512, 4096, 2)        # a partial chunk cannot be sharded
    assert tp.split_even(6144, 4, 32) == [(0, 1536), (1536, 3072), (3072, 4608), (4608, 6144)]
    s = torch.arange(64.0)
    assert torch.equal(tp.unreorder_scales(tp.reorder_scales(s)), s)
    with pytest.raises(ValueError):
        tp.split_even(100, 3, 32)


def test_single_channel_shard_is_refused():
    """A shard that selects one channel would have to carry both bucket bounds in one threshold entry."""
    from decdec_b200 import tp
    K, N = 4096, 64
    q = torch.zeros(K, N // 8, dtype=torch.int32)
    with pytest.raises(ValueError, match="single channel"):
        tp.shard_residual(q, torch.ones(N).half(), torch.linspace(4, 0.1, K).half(), 1, "row", 0, 4)
    r = tp.shard_residual(q, torch.ones(N).half(), torch.linspace(4, 0.1, K).half(), 2, "row", 1, 4)
    assert float(r["thresholds"][0]) == 4.0 and r["q_residual"].shape == (1024, N // 8)
