"""Tensor-parallel decode on 2 GPUs: one process per GPU, the NCCL all-reduce after o_proj and down_proj,
logits of every rank against the unsharded CPU step.  Skipped on a box with a single GPU."""
from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest

from test_tp_sharding_gloo import TP_CFG

pytestmark = pytest.mark.gpu


def _gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank: int, world: int, port: int, out_dir: str):
    import ctypes as C

    import torch
    import torch.distributed as dist

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    import __graft_entry__ as graft
    import cases
    import step_oracle as so

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    lib = graft.load_package().load_lib()
    assert lib.ckb200_init(rank) == 0
    so.bind_model_api(lib)
    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_char * 128)()
        assert lib.ckb200_tp_unique_id(buf) == 0
        uid = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    dist.broadcast(uid, 0)
    raw = bytes(uid.numpy().tobytes())
    assert lib.ckb200_tp_init(rank, world, raw) == 0, lib.ckb200_last_error_message()

    cpu = so.CpuModel(TP_CFG, seed=5)
    cpu.prefill_kv(20, seed=6)
    shard = so.TpShard(cpu, rank, world)
    st = so.make_cfg(TP_CFG, batch=1, tp_rank=rank, tp_size=world)
    handle = lib.ckb200_model_create(C.byref(st))
    assert handle, lib.ckb200_last_error_message()
    lib.ckb200_model_use_tp.argtypes = [C.c_void_p]
    lib.ckb200_model_use_tp(handle)
    so.upload_shard(lib, handle, shard)
    assert lib.ckb200_model_set_pos(handle, 20) == 0
    outs = []
    for tok in (7, 123):
        ids = np.array([tok], dtype=np.int32)
        logits = np.zeros((1, TP_CFG["vocab_size"]), np.float32)
        assert lib.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, lib.ckb200_last_error_message()
        outs.append(logits[0].copy())
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), np.stack(outs))
    dist.barrier()
    lib.ckb200_model_free(handle)
    lib.ckb200_tp_shutdown()
    dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_tensor_parallel_decode(tmp_path, orc):
    import torch.multiprocessing as mp

    import step_oracle as so

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    cpu = so.CpuModel(TP_CFG, seed=5)
    cpu.prefill_kv(20, seed=6)
    want = np.stack([cpu.decode(orc, tok, 20 + i) for i, tok in enumerate((7, 123))])
    for rank in range(2):
        got = np.load(tmp_path / f"rank{rank}.npy")
        for a, b in zip(got, want):
            cos = float(a.astype(np.float64) @ b.astype(np.float64) / (np.linalg.norm(a) * np.linalg.norm(b)))
            assert cos >= 0.9999, (rank, cos)
