"""Row-sharded products on two GPUs: one process per GPU, each holding a row shard on its device; the partial
results of t(y) X, t(X) X and t(X)(X v) are all-reduced (the path's only exchange step) with NCCL and with the library's
own kernel over peer memory, and checked against the dense product; X v stays row partitioned. Skipped where fewer than two GPUs are visible."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

from systemds_b200 import datagen, shard
from tests.util import TOL, dense_of, rel_err

pytestmark = pytest.mark.gpu
KINDS = ("ddc",) * 12 + ("ddc2", "sdc", "rle", "ole", "unc", "const", "sdcsz", "ddc_char")
NROWS = 200_003


def _rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from systemds_b200 import native
    from systemds_b200.native import check
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    L = native.lib()
    dev = torch.device("cuda", rank)
    cmb = datagen.random_cmb(44, NROWS, KINDS)
    rng = np.random.default_rng(2)
    y = rng.standard_normal((3, cmb.rlen))
    v = rng.standard_normal(cmb.clen)
    a, b = shard.shard_bounds(cmb.rlen, world)[rank]
    part = shard.slice_rows(cmb, a, b).to_device(rank)
    h, n = part.handle(), cmb.clen
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    yd = torch.from_numpy(np.ascontiguousarray(y[:, a:b])).to(dev)
    vd = torch.from_numpy(v).to(dev)
    lmm = torch.empty((3, n), dtype=torch.float64, device=dev)
    tsmm = torch.empty((n, n), dtype=torch.float64, device=dev)
    chain = torch.empty(n, dtype=torch.float64, device=dev)
    u = torch.empty(b - a, dtype=torch.float64, device=dev)
    check(L.cla_lmm_dev(h, P(yd), 3, P(lmm), s))
    check(L.cla_tsmm_dev(h, P(tsmm), s))
    check(L.cla_mmchain_dev(h, P(vd), None, 0, P(chain), None, s))
    check(L.cla_rmm_dev(h, P(vd), n, 1, P(u), s))
    # the same sums through the library's own exchange over peer memory (cla_allreduce_dev), before NCCL touches them
    from systemds_b200.comm import PeerAllReduce, torch_exchange
    comm = PeerAllReduce(rank, world, rank, n * n, torch_exchange(dev))
    peer = [t.clone() for t in (lmm, tsmm, chain)]
    for _ in range(3):  # repeated calls walk both slot parities
        again = [t.clone() for t in (lmm, tsmm, chain)]
        for t in again:
            comm(t.data_ptr(), t.numel(), s.value)
    for t in peer:
        comm(t.data_ptr(), t.numel(), s.value)
    comm.status()
    same = all(torch.equal(a_, b_) for a_, b_ in zip(peer, again))
    for t in (lmm, tsmm, chain):
        dist.all_reduce(t)
    torch.cuda.synchronize()
    # every rank holds identical bits of the peer sums (rank-ordered addition), and they agree with NCCL's to rounding
    bits = [torch.zeros_like(t) for t in peer]
    for b_, t in zip(bits, peer):
        b_.copy_(t)
        dist.broadcast(b_, 0)
    same = same and all(torch.equal(a_, b_) for a_, b_ in zip(peer, bits))
    close = all(bool(((a_ - b_).abs() <= 1e-12 * (a_.abs() + b_.abs()) + 1e-300).all()) or
                float((a_ - b_).abs().max()) <= 1e-9 * float(b_.abs().max()) for a_, b_ in zip(peer, (lmm, tsmm, chain)))
    ok = torch.tensor([int(same), int(close)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    comm.close()
    st = part.stats()
    if rank == 0:
        q.put([lmm.cpu().numpy(), tsmm.cpu().numpy(), chain.cpu().numpy(), u.cpu().numpy(), st["kernel_launches"],
               ok.cpu().tolist()])
    dist.barrier()
    part.free()
    dist.destroy_process_group()


def test_two_gpu_partials_add_up(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    lmm, tsmm, chain, u0, launches, peer_ok = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert launches > 0
    assert peer_ok == [1, 1], "peer-memory all-reduce: [identical on all ranks and between calls, agrees with NCCL]"
    cmb = datagen.random_cmb(44, NROWS, KINDS)
    X = dense_of(cmb)
    aX = np.abs(X)
    rng = np.random.default_rng(2)
    y = rng.standard_normal((3, cmb.rlen))
    v = rng.standard_normal(cmb.clen)
    assert rel_err(lmm, oracle.dense_lmm_ld(X, y), np.abs(y) @ aX) < TOL
    assert rel_err(tsmm, oracle.dense_tsmm_ld(X), aX.T @ aX) < TOL
    assert rel_err(chain.ravel(), X.T @ (X @ v), aX.T @ (aX @ np.abs(v))) < 10 * TOL
    a, b = shard.shard_bounds(cmb.rlen, 2)[0]
    assert rel_err(u0.ravel(), (X @ v)[a:b], (aX @ np.abs(v))[a:b] + 1e-300) < TOL
