"""Failure detection of the tensor-parallel group on the host (tp.Membership), with gloo ranks on CPU: a rank that leaves between steps, a rank
that dies without a word, and the undisturbed case.  No GPU, no kernel is made to wait."""
from __future__ import annotations

import multiprocessing as mp
import os
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, port, scenario, out):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g

    tp = g.load_package().tp
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, wait_for_workers=False)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    m = tp.Membership(store, rank, world, timeout_s=1.0)
    launched = 0
    try:
        for step in range(1, 7):
            if scenario == "leave" and rank == 1 and step == 4:
                m.leave("left")                       # between steps: nothing of this rank is in flight
                break
            if scenario == "vanish" and rank == 1 and step == 4:
                os._exit(0)                           # no good-bye: the others notice the silence
            m.before_step(step)
            t = torch.ones(4) * (rank + 1)            # the step itself: an exchange every rank takes part in
            dist.all_reduce(t)
            assert float(t[0]) == sum(range(1, world + 1))
            launched = step
        out.put((rank, launched, "done"))
    except tp.PeerLeft as e:
        out.put((rank, launched, str(e)))
    if scenario == "ok":
        dist.barrier()
    time.sleep(0.2 if rank else 0.6)                  # rank 0 hosts the store: it goes last


@pytest.mark.parametrize("scenario,world", [("ok", 2), ("leave", 2), ("leave", 3), ("vanish", 2)])
def test_membership(scenario, world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + (os.getpid() % 200) + {"ok": 0, "leave": 1, "vanish": 2}[scenario] * 200 + world
    procs = [ctx.Process(target=_rank, args=(r, world, port, scenario, out)) for r in range(world)]
    for p in procs:
        p.start()
    want = world - (1 if scenario == "vanish" else 0)
    got = {}
    deadline = time.time() + 60
    while len(got) < want and time.time() < deadline:
        try:
            r, launched, msg = out.get(timeout=1.0)
            got[r] = (launched, msg)
        except Exception:
            pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert len(got) == want, got
    if scenario == "ok":
        assert all(v == (6, "done") for v in got.values()), got
    else:
        survivors = [r for r in range(world) if r != 1]
        for r in survivors:
            launched, msg = got[r]
            assert launched == 3 and "step 4 not launched" in msg, got      # the step after the departure was never launched
            assert ("rank 1 left after step 3" in msg) if scenario == "leave" else ("has not reported" in msg), got
        if scenario == "leave":
            assert got[1] == (3, "done")
