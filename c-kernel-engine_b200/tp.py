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
