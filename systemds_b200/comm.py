"""The small all-reduce that ends a product on a row-sharded block, over NVLink peer memory (``cla_allreduce_dev``).

One process per GPU. Every rank creates a comm, the ranks exchange the 64-byte IPC handles of their buffers (here
through ``torch.distributed``, which is only the messenger), connect, and from then on sum device vectors in place with
one kernel per rank. All ranks receive identical bits (the sum is formed in rank order on every rank).
"""
from __future__ import annotations

import ctypes as C

from . import native
from .native import check

HANDLE_BYTES = 64


def torch_exchange(device):
    """Returns ``exchange(my_bytes) -> [bytes of rank 0, bytes of rank 1, ...]`` over the default process group."""
    import torch
    import torch.distributed as dist

    def exchange(b: bytes):
        world = dist.get_world_size()
        on_gpu = dist.get_backend() == "nccl"
        dev = device if on_gpu else torch.device("cpu")
        mine = torch.frombuffer(bytearray(b), dtype=torch.uint8).to(dev)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        return [bytes(p.cpu().numpy().tobytes()) for p in parts]

    return exchange


class PeerAllReduce:
    """``comm(ptr, n, stream)`` sums ``n`` doubles at device address ``ptr`` over all ranks, in place."""

    def __init__(self, rank: int, world: int, device: int, max_doubles: int, exchange=None, connect: bool = True):
        self.L = native.lib()
        self._buf = C.create_string_buffer(HANDLE_BYTES)
        self.h = check(self.L.cla_comm_create(device, rank, world, max_doubles, self._buf))
        self.rank, self.world, self.max_doubles = rank, world, max_doubles
        if connect:
            try:
                self.connect(exchange)
            except Exception:
                self.close()
                raise

    @property
    def handle_bytes(self) -> bytes:
        """This rank's 64-byte IPC handle (what the ranks exchange)."""
        return self._buf.raw

    def connect(self, exchange=None, handles=None) -> None:
        """Maps the peers' buffers. ``handles``: the 64-byte handles of all ranks in rank order, or ``exchange`` to fetch
        them; neither: every rank maps to this rank's own buffer (single-process checks)."""
        if handles is None and exchange is not None:
            handles = exchange(self._buf.raw)
        if handles is None:
            check(self.L.cla_comm_connect(self.h, None))
            return
        if len(handles) != self.world or any(len(x) != HANDLE_BYTES for x in handles):
            raise native.CLAError(-2, "one 64-byte handle per rank is needed")
        check(self.L.cla_comm_connect(self.h, C.c_char_p(b"".join(handles))))

    def set_timeout_ms(self, ms: int) -> None:
        check(self.L.cla_comm_set_timeout_ms(self.h, ms))

    def __call__(self, ptr: int, n: int, stream: int = 0) -> None:
        check(self.L.cla_allreduce_dev(self.h, C.c_void_p(ptr), n, C.c_void_p(stream)))

    def status(self) -> None:
        """Synchronises the device and raises CLAError (DEVICE_CHECK) if a rank failed to arrive in an earlier call."""
        check(self.L.cla_comm_status(self.h))

    def close(self) -> None:
        if self.h:
            self.L.cla_comm_destroy(self.h)
            self.h = 0
