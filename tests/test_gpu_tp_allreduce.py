"""Push all-reduce of the row-parallel outputs (decdec_tp_allreduce), through the C ABI.

On one GPU the peer is emulated by staging what it would have pushed (its vector as self-validating lines
{payload, call, payload, call}) into this rank's exchange buffer BEFORE the launch, so no kernel ever waits for another kernel on the same GPU.  The
failure path is a wait that runs out (flags nobody sets) with a short limit; the kernel returns an error status
and the context stays usable.  With two or more GPUs the real exchange runs as two processes and is compared
with NCCL's all-reduce.
"""
import ctypes as C
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def _layout(capi, world, max_n):
    f, s, st, b = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    capi.call("decdec_tp_layout", world, max_n, C.byref(f), C.byref(s), C.byref(st), C.byref(b))
    return f.value, s.value, st.value, b.value


def _create(capi, world, rank, max_n):
    comm = C.c_size_t(0)
    capi.call("decdec_tp_create", world, rank, max_n, C.byref(comm), None)
    ptr = C.c_void_p()
    capi.call("decdec_tp_local_ptr", comm.value, C.byref(ptr))
    return comm.value, ptr.value


def _status(capi, comm):
    calls, err = C.c_uint32(0), C.c_uint32(0)
    capi.call("decdec_tp_status", comm, C.byref(calls), C.byref(err))
    return calls.value, err.value


@pytest.fixture(scope="module")
def capi():
    assert torch.cuda.is_available()
    from decdec_b200 import capi as _c
    return _c


def test_world_of_one_is_identity(capi):
    comm, _ = _create(capi, 1, 0, 4096)
    y = torch.randn(4096, device="cuda").half()
    ref = y.clone()
    capi.call("decdec_tp_allreduce", comm, y.data_ptr(), y.numel(), DT[y.dtype], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(y, ref)
    assert _status(capi, comm) == (1, 0)
    capi.call("decdec_tp_destroy", comm)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 7)])
def test_staged_peers_sum_in_rank_order(capi, dtype, world, rank):
    n, max_n = 4096 + 512, 8192
    flags_off, slots_off, stride, nbytes = _layout(capi, world, max_n)
    comm, ptr = _create(capi, world, rank, max_n)
    mine = torch.as_tensor(_Raw(ptr, nbytes), device="cuda")
    # the peers' buffers are plain device tensors here: this rank's pushes land in them and can be inspected
    peers = {s: torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for s in range(world) if s != rank}
    table = (C.c_size_t * world)(*[(ptr if s == rank else peers[s].data_ptr()) for s in range(world)])
    capi.call("decdec_tp_connect_ptrs", comm, table)
    esz = torch.empty(0, dtype=dtype).element_size()
    g = torch.Generator(device="cuda").manual_seed(world * 10 + rank)
    stream = torch.cuda.current_stream().cuda_stream

    def lines(vec, call):
        """The slot image of a vector: payload words interleaved with the call number."""
        words = vec.contiguous().view(torch.int32)
        return torch.stack([words, torch.full_like(words, call)], dim=1).reshape(-1)

    for call in (1, 2, 3):
        half = call & 1
        vecs = [torch.randn(n, device="cuda", generator=g).to(dtype) for _ in range(world)]
        nwords = n * esz // 4
        for s in range(world):
            if s == rank:
                continue
            off = slots_off + (half * world + s) * stride
            mine[off:off + nwords * 8].view(torch.int32).copy_(lines(vecs[s], call))        # what peer s would have pushed
        y = vecs[rank].clone()
        torch.cuda.synchronize()
        capi.call("decdec_tp_allreduce", comm, y.data_ptr(), n, DT[dtype], stream)
        torch.cuda.synchronize()
        acc = torch.zeros(n, dtype=torch.float32, device="cuda")
        for s in range(world):
            acc += vecs[s].float()
        assert torch.equal(y, acc.to(dtype)), f"call {call}: sum differs"
        assert _status(capi, comm) == (call, 0)
        # this rank's lines arrived in every peer's buffer, in its own slot of this call's half
        for s, buf in peers.items():
            off = slots_off + (half * world + rank) * stride
            assert torch.equal(buf[off:off + nwords * 8].view(torch.int32), lines(vecs[rank], call))
    capi.call("decdec_tp_destroy", comm)


def test_wait_runs_out_and_context_survives(capi):
    os.environ["DECDEC_TP_WAIT_POLLS"] = "2000"          # a few milliseconds
    try:
        comm, ptr = _create(capi, 2, 0, 4096)
    finally:
        del os.environ["DECDEC_TP_WAIT_POLLS"]
    _, _, _, nbytes = _layout(capi, 2, 4096)
    peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    table = (C.c_size_t * 2)(ptr, peer.data_ptr())
    capi.call("decdec_tp_connect_ptrs", comm, table)
    y = torch.randn(4096, device="cuda").half()
    ref = y.clone()
    capi.call("decdec_tp_allreduce", comm, y.data_ptr(), 4096, DT[y.dtype], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()                               # returns: the wait is bounded
    calls, err = _status(capi, comm)
    assert err == 1 and calls == 1
    assert torch.equal(y, ref), "an unsummed output must be left as it was"
    # the device is still usable
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
    capi.call("decdec_tp_destroy", comm)


def test_gemv_behind_a_slow_exchange_does_not_give_up(capi):
    """A GEMV launched behind an exchange becomes resident while the exchange still waits for a peer, and its producer
    fills every stage slot at once.  Its bounded waits for a free slot must start only after the exchange has ended:
    here the exchange waits tens of milliseconds for a peer that never pushes (bounded; it reports and returns), the
    GEMV's own limit is 1 ms, and the GEMV must still finish with the right answer."""
    from decdec_b200 import ops
    from tests import problems as P
    from oracle import forward as ofw
    os.environ["DECDEC_TP_WAIT_POLLS"] = "60000"
    try:
        comm, ptr = _create(capi, 2, 0, 4096)
    finally:
        del os.environ["DECDEC_TP_WAIT_POLLS"]
    _, _, _, nbytes = _layout(capi, 2, 4096)
    peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    capi.call("decdec_tp_connect_ptrs", comm, (C.c_size_t * 2)(ptr, peer.data_ptr()))
    N, K = 8192, 4096                       # 64 stages per K slice: the producer has to wait for free slots
    L = P.random_bcq_layer(N, K, 3, 128, seed=5)
    x = P.make_activation(K, seed=6)
    qw, al, qb, xd = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda(), x.cuda()
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.lutgemm_gemv(xd, torch.zeros_like(y), qw, al, qb, 3, 128)
    torch.cuda.synchronize()
    v = torch.randn(4096, device="cuda").half()
    stream = torch.cuda.current_stream().cuda_stream
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    os.environ["DECDEC_PIPE_WAIT_NS"] = "1000000"
    try:
        a.record()
        capi.call("decdec_tp_allreduce", comm, v.data_ptr(), 4096, DT[v.dtype], stream)
        b.record()
        ops.lutgemm_gemv(xd, y, qw, al, qb, 3, 128)
        torch.cuda.synchronize()
    finally:
        del os.environ["DECDEC_PIPE_WAIT_NS"]
    assert _status(capi, comm)[1] == 1                      # the exchange did give up on its peer ...
    assert a.elapsed_time(b) > 3.0, "the exchange did not outlast the GEMV's own limit; the test shows nothing"
    assert ops.stream_status() == 0                         # ... and the GEMV behind it did not
    want = ofw.layer_output(L["w_hat"], P.to_np(x), None)
    max_abs, _ = P.errors(y, want)
    assert max_abs <= 1e-2
    capi.call("decdec_tp_destroy", comm)


def test_argument_checks(capi):
    from decdec_b200.capi import DecdecError
    comm, _ = _create(capi, 2, 0, 1024)
    y = torch.zeros(1024, device="cuda").half()
    with pytest.raises(DecdecError):       # peers not connected
        capi.call("decdec_tp_allreduce", comm, y.data_ptr(), 1024, 1, None)
    capi.call("decdec_tp_destroy", comm)
    comm, _ = _create(capi, 1, 0, 1024)
    with pytest.raises(DecdecError):       # longer than max_n
        capi.call("decdec_tp_allreduce", comm, y.data_ptr(), 2048, 1, None)
    with pytest.raises(DecdecError):       # not a multiple of 16 bytes
        capi.call("decdec_tp_allreduce", comm, y.data_ptr(), 1001, 1, None)
    capi.call("decdec_tp_destroy", comm)
    with pytest.raises(DecdecError):
        _create(capi, 9, 0, 1024)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _same(y, ref32):
    """The push kernel adds the ranks' fp16 vectors in fp32 in rank order and rounds once; NCCL's fp32 sum may use
    another order, so the two may differ by one fp16 ulp of the result."""
    return bool(torch.allclose(y.float(), ref32, rtol=2.0 ** -10, atol=2.0 ** -12))


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from decdec_b200.tp import PushAllReduce
    ar = PushAllReduce(8192)
    ok = True
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for i, n in enumerate([4096, 8192, 4096, 1024, 4096]):
        y = torch.randn(n, device=dev, generator=g).half()
        ref = y.float().clone()
        dist.all_reduce(ref)
        ar(y)
        torch.cuda.synchronize()
        ok &= _same(y, ref)
        # every rank sums in rank order: the result is bit-identical on all of them
        mine = y.view(torch.int32).clone()      # two fp16 values per word (NCCL has no 16-bit integer type)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok &= bool(torch.equal(lo, hi))
    # graph replay with changing inputs
    s = torch.cuda.Stream()
    yb = torch.zeros(4096, device=dev).half()
    with torch.cuda.stream(s):
        ar(yb)
        s.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            ar(yb)
        for i in range(4):
            src = torch.randn(4096, device=dev, generator=g).half()
            ref = src.float().clone()
            dist.all_reduce(ref)
            yb.copy_(src)
            gr.replay()
            s.synchronize()
            ok &= _same(yb, ref)
    ar.check()
    calls, err = ar.status()
    dist.barrier()
    torch.cuda.synchronize()
    q.put((rank, ok, calls, err))
    del gr
    ar.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_real_gpus_match_nccl(world):
    """One process per GPU, the real exchange over NVLink peer memory, eager and graph-replayed, against ncclAllReduce."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, calls, err in res:
        assert ok and err == 0 and calls == 10, (rank, ok, calls, err)
