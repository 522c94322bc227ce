"""Push all-reduce of the row-parallel outputs (decdec_tp_allreduce), through the C ABI.

On one GPU the peer is emulated by staging what it would have pushed (its vector and its flags) into this
rank's exchange buffer BEFORE the launch, so no kernel ever waits for another kernel on the same GPU.  The
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
    ept = 16 // esz
    n_cta = -(-n // (256 * ept))
    g = torch.Generator(device="cuda").manual_seed(world * 10 + rank)
    stream = torch.cuda.current_stream().cuda_stream
    for call in (1, 2, 3):
        half = call & 1
        vecs = [torch.randn(n, device="cuda", generator=g).to(dtype) for _ in range(world)]
        for s in range(world):
            if s == rank:
                continue
            off = slots_off + (half * world + s) * stride
            mine[off:off + n * esz].view(dtype).copy_(vecs[s])                     # what peer s would have pushed
            fl = mine[flags_off:flags_off + world * 64 * 4].view(torch.int32).view(world, 64)
            fl[s, :n_cta] = call                                                    # ... and its flags
        y = vecs[rank].clone()
        torch.cuda.synchronize()
        capi.call("decdec_tp_allreduce", comm, y.data_ptr(), n, DT[dtype], stream)
        torch.cuda.synchronize()
        acc = torch.zeros(n, dtype=torch.float32, device="cuda")
        for s in range(world):
            acc += vecs[s].float()
        assert torch.equal(y, acc.to(dtype)), f"call {call}: sum differs"
        assert _status(capi, comm) == (call, 0)
        # this rank's vector and flags arrived in every peer's buffer
        for s, buf in peers.items():
            off = slots_off + (half * world + rank) * stride
            assert torch.equal(buf[off:off + n * esz].view(dtype), vecs[rank])
            fl = buf[flags_off:flags_off + world * 64 * 4].view(torch.int32).view(world, 64)
            assert (fl[rank, :n_cta] == call).all() and (fl[rank, n_cta:] == 0).all()
    capi.call("decdec_tp_destroy", comm)


@pytest.mark.parametrize("with_dec", [False, True])
def test_exchange_folded_into_the_gemv_finalizer(capi, with_dec):
    """decdec_tp_bind_next + a binary-coded GEMV: the finalizing thread blocks push fp32 tile sums, wait for the
    (staged) peer's, and round once.  World of two, this process is rank 0; the peer's sums and flags are staged."""
    import numpy as np
    from decdec_b200 import ops
    from oracle import forward as ofw
    from tests import problems as P
    N, K, world, rank, max_n = 4096, 2048, 2, 0, 8192
    flags_off, slots_off, stride, nbytes = _layout(capi, world, max_n)
    comm, ptr = _create(capi, world, rank, max_n)
    mine = torch.as_tensor(_Raw(ptr, nbytes), device="cuda")
    peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    capi.call("decdec_tp_connect_ptrs", comm, (C.c_size_t * 2)(ptr, peer.data_ptr()))
    L = P.bcq_layer(N, K, 3, 128, seed=5)
    x = P.make_activation(K, seed=6)
    own = ofw.layer_output(L["w_hat"], P.to_np(x))
    cfg = None
    if with_dec:
        cs, rs = P.random_residual(N, K, seed=7)
        thr = P.make_thresholds(K)
        rows = torch.zeros(4096, dtype=torch.int32, device="cuda")
        acts = torch.zeros(4096, dtype=torch.float16, device="cuda")
        ctx = ops.create_dec_context(8, rows, acts)
        cfg = ops.create_dec_config(ctx, 8, cs, rs, thr)
        er, ea, _ = P.expected_selection(x, thr, 8, "fp16")
        own = own + ofw.dec_delta(P.to_np(x), er, cs.numpy(), P.to_np(rs), ea)
    qw, al, qb = L["qweight"].cuda(), L["alpha"].cuda(), L["q_bias"].cuda()
    g = torch.Generator(device="cuda").manual_seed(11)
    for call in (1, 2):
        half = call & 1
        other = torch.randn(N, device="cuda", generator=g)                        # the peer's fp32 partial sums
        off = slots_off + (half * world + 1) * stride
        mine[off:off + N * 4].view(torch.float32).copy_(other)
        mine[flags_off:flags_off + world * 64 * 4].view(torch.int32).view(world, 64)[1, :] = call
        y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        capi.call("decdec_tp_bind_next", comm)
        if with_dec:
            ops.dec_lutgemm(cfg, x.cuda(), y, qw, al, qb, 3, 128)
        else:
            ops.lutgemm_gemv(x.cuda(), y, qw, al, qb, 3, 128)
        torch.cuda.synchronize()
        assert _status(capi, comm) == (call, 0)
        ref = own + other.double().cpu().numpy()
        err = np.abs(y.float().cpu().numpy().reshape(-1) - ref)
        assert err.max() <= 1e-2 and np.linalg.norm(err) / np.linalg.norm(ref) <= 1e-3
        # this rank's fp32 sums reached the peer's buffer, with one flag per output tile
        off0 = slots_off + (half * world + 0) * stride
        pushed = peer[off0:off0 + N * 4].view(torch.float32).double().cpu().numpy()
        assert np.abs(pushed - own).max() <= 1e-2
        fl = peer[flags_off:flags_off + world * 64 * 4].view(torch.int32).view(world, 64)[0]
        n_set = int((fl == call).sum())
        assert 1 <= n_set <= 64 and bool((fl[:n_set] == call).all())
    # an unbound call afterwards is a plain GEMV again
    y = torch.zeros(1, 1, N, dtype=torch.float16, device="cuda")
    ops.lutgemm_gemv(x.cuda(), y, qw, al, qb, 3, 128)
    torch.cuda.synchronize()
    base = ofw.layer_output(L["w_hat"], P.to_np(x))
    assert np.abs(y.float().cpu().numpy().reshape(-1) - base).max() <= 1e-2
    assert _status(capi, comm)[0] == 2
    if cfg is not None:
        ops.destroy_dec_config(cfg)
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
        ok &= bool(torch.equal(y, ref.half()))
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
            ok &= bool(torch.equal(yb, ref.half()))
    # exchange folded into a row-parallel binary-coded GEMV (each rank holds half of K)
    from decdec_b200 import ops
    Kl, N = 2048, 4096
    gw = torch.Generator(device=dev).manual_seed(500 + rank)
    qw = torch.randint(-2**31, 2**31 - 1, (Kl // 32, 3, N), dtype=torch.int32, device=dev, generator=gw)
    al = (torch.rand(Kl // 128, 3, N, device=dev, generator=gw) * 0.01).half()
    qb = ((torch.rand(Kl // 128, N, device=dev, generator=gw) - 0.5) * 0.01).half()
    fused_calls = 0
    for i in range(3):
        xl = torch.randn(1, 1, Kl, device=dev, generator=gw).half()
        part = torch.zeros(1, 1, N, dtype=torch.float16, device=dev)
        ops.lutgemm_gemv(xl, part, qw, al, qb, 3, 128)
        ref = part.float().clone()
        dist.all_reduce(ref)
        yf = torch.zeros(1, 1, N, dtype=torch.float16, device=dev)
        ar.bind_next()
        ops.lutgemm_gemv(xl, yf, qw, al, qb, 3, 128)
        torch.cuda.synchronize()
        fused_calls += 1
        d = (yf.float() - ref).abs()
        ok &= bool(d.max() <= 2e-2) and bool(d.norm() / ref.norm() <= 2e-3)
        # every rank holds the same bits
        both = [torch.empty_like(yf) for _ in range(world)]
        dist.all_gather(both, yf)
        ok &= bool(torch.equal(both[0], both[1]))
    ar.check()
    calls, err = ar.status()
    calls -= fused_calls
    dist.barrier()
    torch.cuda.synchronize()
    q.put((rank, ok, calls, err))
    del gr
    ar.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_match_nccl():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, calls, err in res:
        assert ok and err == 0 and calls == 10, (rank, ok, calls, err)
