"""The peer-memory all-reduce on one GPU: a world of one, argument checks, and the bounded wait (a rank that never
arrives ends the kernel with an error status and a NaN result; nothing hangs and the comm stays usable). The exchange
between two GPUs is covered by tests/test_multi_gpu.py."""
import numpy as np
import pytest

from systemds_b200 import CLAError
from systemds_b200.comm import PeerAllReduce

pytestmark = pytest.mark.gpu


def test_world_of_one_is_the_identity():
    import torch
    comm = PeerAllReduce(0, 1, 0, 1000)
    x = torch.randn(1000, dtype=torch.float64, device="cuda:0")
    want = x.clone()
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(5):  # both parities of the slot, several times
        comm(x.data_ptr(), 1000, s)
    comm(x.data_ptr(), 0, s)
    comm.status()
    assert torch.equal(x, want)
    with pytest.raises(CLAError):
        comm(x.data_ptr(), 1001, s)  # more than the comm was created for
    comm.close()
    with pytest.raises(CLAError):
        PeerAllReduce(2, 2, 0, 10)  # rank outside the world


def test_a_rank_that_never_arrives_times_out():
    import time
    import torch
    comm = PeerAllReduce(0, 2, 0, 256)  # rank 1 does not exist: nothing ever raises its flag
    comm.set_timeout_ms(50)
    x = torch.ones(256, dtype=torch.float64, device="cuda:0")
    t0 = time.perf_counter()
    comm(x.data_ptr(), 256, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(CLAError) as e:
        comm.status()
    assert time.perf_counter() - t0 < 5.0
    assert "rank 1" in str(e.value)
    assert bool(torch.isnan(x).all())  # the failure is visible in the result as well
    comm.status()  # the error has been reported once; the context and the comm are intact
    y = torch.arange(8, dtype=torch.float64, device="cuda:0")
    assert float((y * 2).sum()) == 56.0
    comm.close()
