"""Tensor-parallel decode on 2, 4 and 8 GPUs: one process per GPU, the all-reduce after o_proj and down_proj (peer-memory
push kernel checked against NCCL, then used by the step),
logits of every rank against the unsharded CPU step.  Skipped on a box with fewer GPUs."""
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


def _worker(rank: int, world: int, port: int, out_dir: str, cfg: dict):
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
    pkg = graft.load_package()
    pkg.tp.setup(lib, rank, world, None, p2p_floats=4096)
    assert lib.ckb200_tp_p2p_ready() == 1

    # the exchange step alone: the peer-memory kernel against NCCL on the same vectors (both sum in fp32; two
    # ranks: one addition, so bit-exact), several calls in a row to cross both buffer parities, ragged counts
    lib.ckb200_tp_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    for call, count in enumerate((4096, 1000, 4, 4096, 2052, 1)):
        x = torch.from_numpy(np.random.default_rng(100 * call + rank).standard_normal(count).astype(np.float32)).cuda()
        got, want = x.clone(), x.clone()
        torch.cuda.synchronize()
        lib.ckb200_tune_set(b"tp_p2p", 1)
        assert lib.ckb200_tp_allreduce(None, got.data_ptr(), count, None) == 0, lib.ckb200_last_error_message()
        lib.ckb200_tune_set(b"tp_p2p", 0)
        assert lib.ckb200_tp_allreduce(None, want.data_ptr(), count, None) == 0, lib.ckb200_last_error_message()
        assert lib.ckb200_synchronize() == 0, lib.ckb200_last_error_message()
        if world == 2:
            assert torch.equal(got, want), (rank, call, count)
        else:                                             # more than two addends: NCCL's order of additions is its own
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-5), (rank, call, count)
    lib.ckb200_tune_set(b"tp_p2p", 1)

    cpu = so.CpuModel(cfg, seed=5)
    cpu.prefill_kv(20, seed=6)
    shard = so.TpShard(cpu, rank, world)
    lib.ckb200_model_use_tp.argtypes = [C.c_void_p]

    def run(fused: int):
        """Two decode steps of a fresh model; fused: the exchange inside the norm kernel (1) or the all-reduce kernel (0)."""
        lib.ckb200_tune_set(b"tp_fused_norm", fused)
        st = so.make_cfg(cfg, batch=1, tp_rank=rank, tp_size=world)
        handle = lib.ckb200_model_create(C.byref(st))
        assert handle, lib.ckb200_last_error_message()
        lib.ckb200_model_use_tp(handle)
        so.upload_shard(lib, handle, shard)
        assert lib.ckb200_model_set_pos(handle, 20) == 0
        outs = []
        for tok in (7, 123):
            ids = np.array([tok], dtype=np.int32)
            logits = np.zeros((1, cfg["vocab_size"]), np.float32)
            assert lib.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, lib.ckb200_last_error_message()
            outs.append(logits[0].copy())
        dist.barrier()
        lib.ckb200_model_free(handle)
        return np.stack(outs)

    launches0 = lib.ckb200_launch_count()
    fused = run(1)
    launches_fused = lib.ckb200_launch_count() - launches0
    unfused = run(0)
    launches_unfused = lib.ckb200_launch_count() - launches0 - launches_fused
    lib.ckb200_tune_set(b"tp_fused_norm", -1)
    assert launches_fused < launches_unfused, (launches_fused, launches_unfused)     # the fused form really ran
    assert np.array_equal(fused, unfused)            # same sums in the same order: the two forms agree bit for bit
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), fused)
    dist.barrier()
    lib.ckb200_tp_shutdown()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_decode(tmp_path, orc, world):
    import torch.multiprocessing as mp

    import step_oracle as so

    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    # whole KV heads per rank, and per-rank attention and FFN widths that are multiples of 256
    cfg = TP_CFG if world == 2 else dict(TP_CFG, num_heads=4 * world, num_kv_heads=world, intermediate_size=256 * world)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path), cfg), nprocs=world, join=True)
    cpu = so.CpuModel(cfg, seed=5)
    cpu.prefill_kv(20, seed=6)
    want = np.stack([cpu.decode(orc, tok, 20 + i) for i, tok in enumerate((7, 123))])
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npy")
        for a, b in zip(got, want):
            cos = float(a.astype(np.float64) @ b.astype(np.float64) / (np.linalg.norm(a) * np.linalg.norm(b)))
            assert cos >= 0.9999, (rank, cos)
