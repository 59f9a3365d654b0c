"""Host side of the tensor-parallel exchange: one process per GPU, torch.distributed carries the bootstrap bytes.

The library has two all-reduce paths (csrc/tp_nccl.c, csrc/tp_p2p.cu): NCCL for any size and a one-shot push kernel
over CUDA-IPC peer memory for small vectors.  Both need a few bytes to reach every rank before the first step: the
128-byte NCCL id of rank 0 and the 64-byte IPC handle of every rank's exchange buffer.
"""
from __future__ import annotations

import ctypes as C


def _err(lib) -> str:
    lib.ckb200_last_error_message.restype = C.c_char_p
    return lib.ckb200_last_error_message().decode()


def setup(lib, rank: int, world: int, device=None, p2p_floats: int = 0) -> None:
    """Create the library's NCCL communicator and, if p2p_floats > 0, the peer-memory exchange buffer for vectors of
    up to that many floats.  `device`: where the bootstrap tensors live (a CUDA device for an NCCL process group,
    None for gloo)."""
    import torch
    import torch.distributed as dist

    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_char * 128)()
        if lib.ckb200_tp_unique_id(buf) != 0:
            raise RuntimeError(_err(lib))
        uid = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    if device is not None:
        uid = uid.to(device)
    dist.broadcast(uid, 0)
    if lib.ckb200_tp_init(rank, world, bytes(uid.cpu().numpy().tobytes())) != 0:
        raise RuntimeError(_err(lib))
    if p2p_floats <= 0 or world < 2:
        return
    lib.ckb200_tp_p2p_create.argtypes = [C.c_int, C.c_int, C.c_size_t, C.c_void_p]
    lib.ckb200_tp_p2p_connect.argtypes = [C.c_void_p]
    handle = (C.c_char * 64)()
    if lib.ckb200_tp_p2p_create(rank, world, (p2p_floats + 3) // 4 * 4, handle) != 0:
        raise RuntimeError(_err(lib))
    mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).clone()
    if device is not None:
        mine = mine.to(device)
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    raw = b"".join(bytes(t.cpu().numpy().tobytes()) for t in everyone)
    if lib.ckb200_tp_p2p_connect(raw) != 0:
        raise RuntimeError(_err(lib))
    dist.barrier()          # every rank has mapped every buffer before anyone's first push


class PeerLeft(RuntimeError):
    """A tensor-parallel peer announced that it stopped, or stopped reporting, before this step."""


class Membership:
    """Host-side liveness of the tensor-parallel group, checked BEFORE a step is launched.

    The exchange kernels wait for their peers' stores; a rank that is gone would leave the others in a bounded wait (seconds) and with an
    error to clean up.  So every rank records the number of the step it is about to launch in a key-value store shared by the group
    (a torch.distributed store: TCPStore, FileStore, or the store behind the default process group), and launches step s only after every
    peer has announced step s too (one store round trip per step; a peer that merely finished step s - 1 may still be about to leave).  A
    rank leaves only between steps: it calls leave(), which the others see instead of its next announcement; a rank that dies silently is
    noticed when the time limit runs out.  No kernel, collective or device is involved.
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "ckb200/tp"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self.store.set(self._key("step", rank), "0")

    def _key(self, what: str, rank: int) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def leave(self, reason: str = "left") -> None:
        self.store.set(self._key("left", self.rank), reason)

    def _peer_state(self, peer: int):
        """(step reached, reason it left or None); keys that do not exist yet read as step -1"""
        left = None
        if self.store.check([self._key("left", peer)]):
            left = self.store.get(self._key("left", peer)).decode()
        step = int(self.store.get(self._key("step", peer)).decode()) if self.store.check([self._key("step", peer)]) else -1
        return step, left

    def before_step(self, step: int) -> None:
        """Announce `step`, then wait (up to the time limit) until every peer has announced it as well.  Raises PeerLeft."""
        import time

        self.store.set(self._key("step", self.rank), str(step))
        deadline = time.monotonic() + self.timeout_s
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                reached, left = self._peer_state(peer)
                if reached >= step:                    # the peer is about to launch (or has launched) the same step
                    break
                if left is not None:
                    raise PeerLeft(f"rank {peer} {left} after step {reached}; step {step} not launched on rank {self.rank}")
                if time.monotonic() > deadline:
                    raise PeerLeft(f"rank {peer} has not reported for {self.timeout_s:.1f} s (last step {reached}); step {step} not launched on rank {self.rank}")
                time.sleep(0.002)
