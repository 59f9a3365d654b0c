"""Tensor-parallel decode on CPU, world_size 2 over gloo: each process holds one shard (column-parallel
q/k/v/gate/up, row-parallel o/down cut at 256-element block boundaries), runs the step with the oracle's
kernels and all-reduces the two partial outputs per layer.  The logits must match the unsharded step;
the integer stages are untouched by the split, only the fp32 sum order changes."""
from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest

TP_CFG = dict(embed_dim=512, num_heads=8, num_kv_heads=2, head_dim=64, intermediate_size=1024, num_layers=2, vocab_size=300,
              max_seq_len=48, rms_eps=1e-5, rope_theta=1.0e4, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch
    import torch.distributed as dist

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    import __graft_entry__ as graft
    import step_oracle as so

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    orc = graft.oracle_loader().load_oracle()
    cpu = so.CpuModel(TP_CFG, seed=5)
    cpu.prefill_kv(20, seed=6)
    shard = so.TpShard(cpu, rank, world)

    def allreduce(vec):
        t = torch.from_numpy(vec)
        dist.all_reduce(t)

    outs = [shard.decode(orc, tok, 20 + i, allreduce) for i, tok in enumerate((7, 123))]
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), np.stack(outs))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_step_matches_unsharded(tmp_path, orc):
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
        scale = float(np.max(np.abs(want)))
        assert float(np.max(np.abs(got - want))) <= 2e-3 * scale, rank
        for a, b in zip(got, want):
            cos = float(a.astype(np.float64) @ b.astype(np.float64) / (np.linalg.norm(a) * np.linalg.norm(b)))
            assert cos >= 0.9999


def test_shard_shapes_cover_the_whole_matrix():
    """Row shards concatenate back to the matrix; column shards split every row at block boundaries."""
    import step_oracle as so

    cpu = so.CpuModel(TP_CFG, seed=1)
    lay = cpu.layers[0]
    parts = [so.shard_layer(TP_CFG, lay, r, 2) for r in range(2)]
    assert np.array_equal(np.concatenate([p["WQ"][3] for p in parts]), lay["WQ"][3])
    fmt, rows, cols, data = lay["WO"]
    back = np.concatenate([p["WO"][3].reshape(rows, -1) for p in parts], axis=1).reshape(-1)
    assert np.array_equal(back, data)
    I = TP_CFG["intermediate_size"]
    rb = lay["W1"][3].size // (2 * I)
    w1 = lay["W1"][3].reshape(2 * I, rb)
    assert np.array_equal(parts[1]["W1"][3].reshape(I, rb)[:I // 2], w1[I // 2:I])          # gate rows of rank 1
    assert np.array_equal(parts[1]["W1"][3].reshape(I, rb)[I // 2:], w1[I + I // 2:])      # up rows of rank 1
