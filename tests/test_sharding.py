"""Row sharding: shards decompress to the right rows, and partial products add up -- on CPU, with a real
two-rank gloo all-reduce for the exchange step."""
import os
import socket

import numpy as np
import pytest

from systemds_b200 import datagen, shard
from tests.util import TOL, dense_of, rel_err


def test_shard_bounds():
    b = shard.shard_bounds(1000, 3)
    assert b[0][0] == 0 and b[-1][1] == 1000 and all(x[1] == y[0] for x, y in zip(b, b[1:]))
    assert all(x[0] % 128 == 0 for x in b)
    assert shard.shard_bounds(100, 8)[-1] == (100, 100)  # more shards than 128-row blocks: empty tails


@pytest.mark.parametrize("nShards", [2, 3])
def test_slices_decompress_to_the_right_rows(oracle, nShards):
    cmb = datagen.random_cmb(21, 70001, datagen.KINDS + ("ddcfor", "sdcfor"))
    X = dense_of(cmb)
    for (a, b), s in zip(shard.shard_bounds(cmb.rlen, nShards), shard.shard(cmb, nShards)):
        assert s.rlen == b - a
        assert np.array_equal(dense_of(s), X[a:b])
        assert rel_err(oracle.OracleMatrix(s).decompress(), X[a:b]) < 1e-14


def _rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cmb = datagen.random_cmb(33, 20000, ("ddc", "ddc2", "sdc", "rle", "ole", "unc", "const", "sdcsz"))
    rng = np.random.default_rng(1)
    y = rng.standard_normal((2, cmb.rlen))
    v = rng.standard_normal(cmb.clen)
    a, b = shard.shard_bounds(cmb.rlen, world)[rank]
    om = o.OracleMatrix(shard.slice_rows(cmb, a, b), threads=1)
    parts = [torch.from_numpy(om.lmm(y[:, a:b])), torch.from_numpy(om.tsmm()), torch.from_numpy(om.mmchain(v))]
    for p in parts:  # the one exchange step of the path
        dist.all_reduce(p)
    u = torch.from_numpy(om.rmm(v))  # RMM: no exchange, output stays row partitioned
    gathered = [torch.zeros(bb - aa, 1, dtype=torch.float64) for aa, bb in shard.shard_bounds(cmb.rlen, world)]
    dist.all_gather(gathered, u) if all(g.shape == gathered[0].shape for g in gathered) else None
    if rank == 0:
        q.put([p.numpy() for p in parts] + [u.numpy()])
    dist.destroy_process_group()


def test_two_rank_gloo_partials_add_up(oracle):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    lmm, tsmm, chain, u0 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cmb = datagen.random_cmb(33, 20000, ("ddc", "ddc2", "sdc", "rle", "ole", "unc", "const", "sdcsz"))
    X = dense_of(cmb)
    aX = np.abs(X)
    rng = np.random.default_rng(1)
    y = rng.standard_normal((2, cmb.rlen))
    v = rng.standard_normal(cmb.clen)
    assert rel_err(lmm, oracle.dense_lmm_ld(X, y), np.abs(y) @ aX) < TOL
    assert rel_err(tsmm, oracle.dense_tsmm_ld(X), aX.T @ aX) < TOL + 20000 * 1.2e-16
    assert rel_err(chain.ravel(), X.T @ (X @ v), aX.T @ (aX @ np.abs(v))) < 10 * TOL
    a, b = shard.shard_bounds(cmb.rlen, 2)[0]
    assert rel_err(u0.ravel(), (X @ v)[a:b], (aX @ np.abs(v))[a:b] + 1e-300) < TOL


def _exchange_rank(rank, world, port, q):
    import torch.distributed as dist
    from systemds_b200.comm import HANDLE_BYTES, torch_exchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    got = torch_exchange(None)(bytes([rank + 1]) * HANDLE_BYTES)  # what the ranks do with their 64-byte IPC handles
    q.put((rank, [g[0] for g in got], [len(g) for g in got]))
    dist.destroy_process_group()


def test_handle_exchange_over_gloo():
    """The host-side half of the peer-memory all-reduce setup: every rank ends up with all ranks' handles, in rank
    order (the device half needs GPUs and is covered by the gpu tests)."""
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_exchange_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, firsts, lens in res:
        assert firsts == [1, 2] and lens == [64, 64]
