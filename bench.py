#!/usr/bin/env python
"""Benchmark of the quantised GEMV hot path: Q4_K x Q8_K dequant-dot GEMV GB/s on B200.

One step = one pass over the quant-format GEMV sweep for Q4_K - out x in of 4096x4096, 14336x4096,
4096x14336 and 151936x896 (K padded to 1024), batch 1 - where every launch reads a different
resident copy of its weight matrix; the copies of a shape total more than 4x the L2 size, so no
launch is served from L2.  `value` = algorithmic bytes of the step (weights + Q8_K activations +
fp32 outputs) / device time, inputs already in HBM.  `e2e` = the same sweep through the
reference-named host-pointer entry point gemv_q4_k_q8_k(y, W, x_q8, M, K): weights registered
(resident, as after model load), activations copied in from pinned host memory and outputs copied
back inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--detail]

Under torchrun every rank runs the sweep on its own GPU over its own shard of rows (no collective
in the data path; weak scaling); the time is the max over ranks.
--impl reference times the reference's own CPU thread-pool path on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402

pkg = graft.load_package()
synth = pkg.synth

METRIC = "q4_k_gemv_hbm_gbs"
UNIT = "GB/s"
L2_BYTES_X4 = 4 * 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0


def sweep(fmt: str):
    return [(m, synth.k_for(fmt, k), k) for (m, k) in synth.SWEEP_SHAPES]


def sweep_config():
    """The workload both arms (this library on the GPU, the reference on the host cores) are timed on."""
    return {"workload": "quant-format GEMV sweep, Q4_K x Q8_K, batch 1",
            "shapes": [[m, k] for m, k, _ in sweep("q4_k")],
            "inputs": "Q4_K weights with fp16 d~U(0,0.02), dmin~U(0,0.01), uniform random scale and quant bytes; x fp32 N(0,1) quantised to Q8_K; "
                      "K = 896 zero-padded to 1024"}


vptr, fptr = pkg.model_api.vptr, pkg.model_api.fptr


def cpu_quantize_q8_k(lib, prefix, x):
    """quantize_row_q8_k of a CPU library (the reference build or the oracle port)."""
    out = np.zeros(synth.row_bytes("q8_k", x.size), dtype=np.uint8)
    f = getattr(lib, prefix + "quantize_row_q8_k")
    f.restype = None
    f(fptr(np.ascontiguousarray(x)), vptr(out), C.c_int(x.size))
    return out


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        import threading

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def count(self) -> int:
        return len(self.lines)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)
        text = "".join(self.lines)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in text.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------- reference arm

def run_reference(args, rank: int):
    if rank != 0:
        return
    loader = graft.oracle_loader()
    threads = loader.host_threads()
    os.environ["CK_NUM_THREADS"] = str(threads)
    ref = loader.load_reference()
    kind = "reference"
    if ref is None:
        ref, kind = loader.load_oracle(), "port"
        threads = 1
    shapes = sweep("q4_k")
    prefix = "" if kind == "reference" else "oracle_"
    work = []
    for m, k, k_raw in shapes:
        w = synth.make_weights("q4_k", m, k, seed=0)
        x = synth.make_x(k, seed=0, k_valid=k_raw if k_raw != k else None)
        xq = cpu_quantize_q8_k(ref, prefix, x)
        y = np.zeros(m, dtype=np.float32)
        work.append((m, k, w, xq, y))
    if kind == "reference":
        ref.ck_parallel_decode_init()
        fn = ref.gemv_q4_k_q8_k_parallel_dispatch       # the reference's own thread-pool path
    else:
        fn = ref.oracle_gemv_q4_k_q8_k
    fn.restype = None
    bytes_per_step = sum(synth.gemv_bytes("q4_k", m, k) for m, k, *_ in work)

    def step():
        for m, k, w, xq, y in work:
            fn(fptr(y), vptr(w), vptr(xq), C.c_int(m), C.c_int(k))

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = bytes_per_step * args.steps / dt / 1e9
    sample = "one GEMV per sweep shape per step (no weight rotation; the largest matrix alone exceeds the host caches)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 dot, fp32 accumulate", "data": "synthetic",
        "config": sweep_config(),
        "path": "gemv_q4_k_q8_k_parallel_dispatch on the reference thread pool" if kind == "reference" else "scalar port",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_sample(budget_s: float = 12.0):
    """Rank 0, N=1: the reference's thread-pool GEMV on a bounded sample of the same sweep."""
    loader = graft.oracle_loader()
    threads = loader.host_threads()
    os.environ["CK_NUM_THREADS"] = str(threads)
    ref = loader.load_reference()
    kind = "reference" if ref is not None else "port"
    if ref is None:
        ref, threads = loader.load_oracle(), 1
    prefix = "" if kind == "reference" else "oracle_"
    if kind == "reference":
        ref.ck_parallel_decode_init()
        fn = ref.gemv_q4_k_q8_k_parallel_dispatch
    else:
        fn = ref.oracle_gemv_q4_k_q8_k
    fn.restype = None
    total_b, total_t, used = 0, 0.0, []
    for m, k, k_raw in sweep("q4_k"):
        w = synth.make_weights("q4_k", m, k, seed=0)
        xq = cpu_quantize_q8_k(ref, prefix, synth.make_x(k, seed=0, k_valid=k_raw if k_raw != k else None))
        y = np.zeros(m, dtype=np.float32)
        args = (fptr(y), vptr(w), vptr(xq), C.c_int(m), C.c_int(k))
        fn(*args)
        reps, t0 = 0, time.perf_counter()
        while True:
            fn(*args)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > budget_s / 4 or reps >= 50:
                break
        total_b += reps * synth.gemv_bytes("q4_k", m, k)
        total_t += dt
        used.append(f"{m}x{k}:{reps}")
    return {"value": total_b / total_t / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": "Q4_K sweep shapes, repetitions " + " ".join(used) + " (up to 3 s or 50 runs each, after one warm-up)"}


# ------------------------------------------------------------------------------------- decode steps

QWEN2_05B = dict(embed_dim=896, num_heads=14, num_kv_heads=2, head_dim=64, intermediate_size=4864, num_layers=24, vocab_size=151936,
                 max_seq_len=2048, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
LLAMA3_70B = dict(embed_dim=8192, num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=28672, num_layers=80, vocab_size=128256,
                  max_seq_len=4352, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)


def decode_bench(lib, name, cfg, ctx, steps, peak, batch=1, tp_rank=0, tp_size=1, dist=None, keep_logits=None, kv_f16=False):
    """Decode tokens/s of a model SHAPE with random weights (device-generated) and a synthetic N(0,1) KV cache of `ctx` tokens.
    With keep_logits (a list) the logits of one extra step at position ctx are appended to it as a device tensor.
    kv_f16: the executor keeps IEEE fp16 caches (the reference's kv_cache_store_f16 / _f16cache attention pair)."""
    import torch

    so = pkg.model_api
    so.bind_model_api(lib)
    st = so.make_cfg(cfg, batch=batch, tp_rank=tp_rank, tp_size=tp_size)
    lib.ckb200_tune_set(b"model_kv_f16", int(kv_f16))
    try:
        handle = lib.ckb200_model_create(C.byref(st))
    finally:
        lib.ckb200_tune_set(b"model_kv_f16", 0)
    if not handle:
        msg = lib.ckb200_last_error_message().decode()
        lib.ckb200_clear_error()
        return {"error": msg}
    try:
        if tp_size > 1:
            lib.ckb200_model_use_tp(handle)
        # the same seed on every rank: the replicated tensors (norm weights, LM head) must agree, and a rank's shard of the
        # others is random data either way
        assert lib.ckb200_model_fill_synthetic(handle, 1) == 0
        assert lib.ckb200_model_fill_kv_synthetic(handle, ctx, 2) == 0
        ids = np.full(batch, 11, dtype=np.int32)
        launches0 = lib.ckb200_launch_count()
        assert lib.ckb200_model_decode(handle, vptr(ids), None) == 0          # eager warm-up + capture + first replay
        launches = (lib.ckb200_launch_count() - launches0) // 2
        assert lib.ckb200_model_decode_repeat(handle, 3) == 0
        assert lib.ckb200_synchronize() == 0
        lstream = torch.cuda.ExternalStream(lib.ckb200_stream())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        assert lib.ckb200_model_set_pos(handle, ctx) == 0
        if dist:
            dist.barrier()
        e0.record(lstream)
        assert lib.ckb200_model_decode_repeat(handle, steps) == 0
        e1.record(lstream)
        lstream.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if dist:
            t = torch.tensor([ms], device=torch.device("cuda", torch.cuda.current_device()))
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        wbytes = lib.ckb200_model_weight_bytes(handle)                    # this rank's shard
        kv_bytes = 2 * cfg["num_layers"] * max(1, cfg["num_kv_heads"] // tp_size) * (ctx + steps // 2) * cfg["head_dim"] * (2 if kv_f16 else 4) * batch
        gbs = (wbytes + kv_bytes) / ms / 1e6
        # end to end: token id from the host, logits back to the host, every step
        logits = np.zeros((batch, cfg["vocab_size"]), np.float32)
        assert lib.ckb200_model_set_pos(handle, ctx) == 0
        t0 = time.perf_counter()
        n_e2e = max(5, steps // 2)
        for _ in range(n_e2e):
            assert lib.ckb200_model_decode(handle, vptr(ids), vptr(logits)) == 0
        e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
        if keep_logits is not None:
            assert lib.ckb200_model_set_pos(handle, ctx) == 0
            assert lib.ckb200_model_decode(handle, vptr(ids), vptr(logits)) == 0
            keep_logits.append(torch.from_numpy(logits[0].copy()).to(torch.device("cuda", torch.cuda.current_device())))
        return {"model_shape": name, "batch": batch, "context": ctx, "tp": tp_size, "kv_cache": "f16" if kv_f16 else "f32", "tok_s": batch * 1e3 / ms, "ms_per_token": ms, "launches_per_token": int(launches),
                "weight_bytes": int(wbytes), "kv_bytes": int(kv_bytes), "hbm_gbs_per_gpu": gbs, "frac_of_measured_peak": gbs / peak,
                "e2e_tok_s": batch * 1e3 / e2e_ms, "e2e_ms_per_token": e2e_ms}
    finally:
        lib.ckb200_model_free(handle)


# ------------------------------------------------------------------------------------- CUDA arm

# DRAM traffic of the Q4_K GEMV kernels relative to their algorithmic bytes, from the ncu capture summarised in
# profiles/gemv_q4k_pair_14336x4096.md (dram__bytes_read.sum + dram__bytes_write.sum of one launch / algorithmic bytes of that
# launch).  Traffic grows with the bytes streamed (every weight byte is read once), so a step's traffic is this ratio times its bytes.
Q4K_DRAM_TRAFFIC_RATIO = 0.999

# sweep name -> (weight format, resident layout, device entry point)
SWEEPS = {
    "q4_k": ("q4_k", None, "ckb200_dev_gemv_q4_k_q8_k"),
    "q6_k_planar": ("q6_k", "planar", "ckb200_dev_gemv_q6_k_planar_q8_k"),
    "q6_k_reference_layout": ("q6_k", None, "ckb200_dev_gemv_q6_k_q8_k"),
    "q8_0_planar": ("q8_0", "planar", "ckb200_dev_gemv_q8_0_planar_q8_0"),
    "q8_0_reference_layout": ("q8_0", None, "ckb200_dev_gemv_q8_0_q8_0"),
    "q5_0_planar": ("q5_0", "planar", "ckb200_dev_gemv_q5_0_planar_q8_0"),
    "q5_0_reference_layout": ("q5_0", None, "ckb200_dev_gemv_q5_0_q8_0"),
}
DEFAULT_SWEEPS = ["q4_k", "q6_k_planar", "q6_k_reference_layout", "q8_0_planar", "q8_0_reference_layout"]


def run_cuda(args, rank: int, world: int, local_rank: int):
    import torch

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = pkg.load_lib()
    if lib.ckb200_init(local_rank) != 0:
        raise RuntimeError(lib.ckb200_last_error_message().decode())
    lib.ckb200_launch_count.restype = C.c_longlong
    lib.ckb200_stream.restype = C.c_void_p

    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.Stream(device=dev)             # graphs cannot be captured on the default stream
    torch.cuda.set_stream(stream)
    sp = C.c_void_p(stream.cuda_stream)
    side_streams = [torch.cuda.Stream(device=dev) for _ in range(max(0, args.streams - 1))]

    names = list(DEFAULT_SWEEPS) + (["q5_0_planar", "q5_0_reference_layout"] if args.detail else [])
    if world > 1:
        names = ["q4_k"]                                # the scaling runs time the headline sweep only
    planar_fns = {"q6_k": (lib.ckb200_q6_k_planar_bytes, lib.ckb200_dev_q6_k_to_planar),
                  "q8_0": (lib.ckb200_q8_0_planar_bytes, lib.ckb200_dev_q8_0_to_planar),
                  "q5_0": (lib.ckb200_q5_0_planar_bytes, lib.ckb200_dev_q5_0_to_planar)}
    for size_fn, _ in planar_fns.values():
        size_fn.restype = C.c_size_t

    results = {}
    for name in names:
        fmt, layout, entry = SWEEPS[name]
        gemv = getattr(lib, entry)
        quant = lib.ckb200_dev_quantize_q8_0 if fmt in ("q8_0", "q5_0") else lib.ckb200_dev_quantize_q8_k
        plan = []
        for m, k, k_raw in sweep(fmt):
            w_host = synth.make_weights(fmt, m, k, seed=rank)          # every rank holds its own shard of rows
            nbytes = w_host.nbytes
            copies = max(2, -(-L2_BYTES_X4 // nbytes))
            slot = (nbytes + 255) & ~255
            src = torch.from_numpy(w_host).to(dev)
            if layout == "planar":                     # resident Q6_K / Q8_0 / Q5_0 weights in the library's row-planar layout (same bits)
                size_fn, conv_fn = planar_fns[fmt]
                nbytes = size_fn(m, k)
                slot = (nbytes + 255) & ~255
                planar = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                assert conv_fn(C.c_void_p(planar.data_ptr()), C.c_void_p(src.data_ptr()), m, k, sp) == 0
                src = planar
            wbuf = torch.empty(copies * slot + 256, dtype=torch.uint8, device=dev)
            for c in range(copies):
                wbuf[c * slot:c * slot + nbytes].copy_(src)
            x = torch.from_numpy(synth.make_x(k, seed=rank, k_valid=k_raw if k_raw != k else None)).to(dev)
            xq = torch.empty(synth.row_bytes("q8_0" if fmt in ("q8_0", "q5_0") else "q8_k", k) + 64, dtype=torch.uint8, device=dev)
            y = torch.empty(copies, m, dtype=torch.float32, device=dev)
            assert quant(C.c_void_p(x.data_ptr()), C.c_void_p(xq.data_ptr()), 1, k, sp) == 0
            plan.append(dict(m=m, k=k, copies=copies, slot=slot, wbuf=wbuf, xq=xq, y=y, bytes=synth.gemv_bytes(fmt, m, k),
                             w_host=w_host if name == "q4_k" else None))
        torch.cuda.synchronize()

        def step(plan=plan, gemv=gemv, nstreams=1):
            """One pass over the sweep.  The launches are independent GEMVs (own weights, own output); with nstreams > 1
            they are dealt round-robin to that many streams, which a graph capture turns into parallel branches."""
            lanes = [stream] + side_streams[:nstreams - 1]
            for s2 in lanes[1:]:
                s2.wait_stream(stream)
            i = 0
            for p in plan:
                base = p["wbuf"].data_ptr()
                for c in range(p["copies"]):
                    rc = gemv(C.c_void_p(p["y"][c].data_ptr()), C.c_void_p(base + c * p["slot"]),
                              C.c_void_p(p["xq"].data_ptr()), p["m"], p["k"], C.c_void_p(lanes[i % len(lanes)].cuda_stream))
                    i += 1
                    if rc != 0:
                        raise RuntimeError(lib.ckb200_last_error_message().decode())
            for s2 in lanes[1:]:
                stream.wait_stream(s2)

        def timed_graph(g, reps):
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                g.replay()
            b.record(stream)
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        launches_before = lib.ckb200_launch_count()
        step()                                             # un-captured: sets kernel attributes, warms caches
        launches_per_step = lib.ckb200_launch_count() - launches_before
        torch.cuda.synchronize()
        # Independent launches on several streams run best when each takes one CTA per SM (kernels of different launches are then
        # resident together and one launch's ramp-up and tail hide behind the others' streaming); a dependent chain wants the full
        # occupancy.  The grid size is fixed when the launch is captured.
        lib.ckb200_tune_set(b"gemv_occ_cap", 1 if args.streams > 1 else 0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step(nstreams=args.streams)
        lib.ckb200_tune_set(b"gemv_occ_cap", 0)
        sampler = ClockSampler(local_rank) if name == "q4_k" else None
        for _ in range(args.warmup):
            graph.replay()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        clocks = None
        if sampler:
            # the timed region is a few milliseconds, the sampler's period 100 ms (and nvidia-smi needs a moment to start): the same
            # step keeps running, untimed, until the sampler has seen it three times
            t_load = time.time()
            while sampler.proc and sampler.count() < 3 and time.time() - t_load < 4.0:
                for _ in range(20):
                    graph.replay()
                torch.cuda.synchronize()
            clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        if dist:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        step_bytes = sum(p["bytes"] * p["copies"] for p in plan)
        serial_gbs = None
        if args.streams > 1:                               # the same step as ONE dependent chain on one stream at full occupancy
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=stream):
                step(nstreams=1)
            serial_gbs = step_bytes / timed_graph(g1, max(3, args.steps // 2)) / 1e6
        per_shape = {}
        if args.detail:
            for p in plan:                                 # per-shape timing, graph of one rotation of that shape
                g = torch.cuda.CUDAGraph()
                lib.ckb200_tune_set(b"gemv_occ_cap", 1 if args.streams > 1 else 0)
                with torch.cuda.graph(g, stream=stream):
                    step(plan=[p], nstreams=args.streams)
                lib.ckb200_tune_set(b"gemv_occ_cap", 0)
                t_ms = timed_graph(g, max(3, args.steps // 2))
                per_shape[f"{p['m']}x{p['k']}"] = {"gbs": p["bytes"] * p["copies"] / t_ms / 1e6, "us_per_launch": t_ms * 1e3 / p["copies"]}
        rc = lib.ckb200_synchronize()
        if rc != 0:
            raise RuntimeError(lib.ckb200_last_error_message().decode())
        results[name] = dict(ms=ms, step_bytes=step_bytes, launches=launches_per_step, clocks=clocks, per_shape=per_shape, serial_gbs=serial_gbs,
                             plan=plan if name == "q4_k" else None, rotation="/".join(str(p["copies"]) for p in plan))
        del graph
        if name != "q4_k":
            del plan
            torch.cuda.empty_cache()

    # ---- end to end through the reference-named host-pointer entry point (Q4_K): resident weights (registered once, as after
    # model load) on rotating copies like the device leg, Q8_K activations in from pinned host memory, fp32 outputs back to it
    plan = results["q4_k"]["plan"]
    fn = lib.gemv_q4_k_q8_k
    fn.restype = None
    lib.ckb200_host_alloc.restype = C.c_void_p
    pinned = []
    for p in plan:
        rot = max(2, min(p["copies"], 16))                          # at most 16 host copies per shape (more than L2 in total for every shape)
        w_rot = np.ascontiguousarray(np.tile(p["w_host"], rot))
        assert lib.ckb200_register_weights(vptr(w_rot), C.c_size_t(w_rot.nbytes)) == 0
        xq_bytes = synth.row_bytes("q8_k", p["k"])
        hx = lib.ckb200_host_alloc(C.c_size_t(xq_bytes))
        hy = lib.ckb200_host_alloc(C.c_size_t(4 * p["m"]))
        xq_host = p["xq"][:xq_bytes].cpu().numpy()
        C.memmove(hx, xq_host.ctypes.data, xq_bytes)
        pinned.append(dict(p=p, w=w_rot, rot=rot, one=p["w_host"].nbytes, hx=hx, hy=hy, xq_bytes=xq_bytes))
    e2e_calls = [0]

    def e2e_step():
        i = e2e_calls[0]
        for q in pinned:
            fn(C.c_void_p(q["hy"]), C.c_void_p(q["w"].ctypes.data + (i % q["rot"]) * q["one"]), C.c_void_p(q["hx"]), q["p"]["m"], q["p"]["k"])
        e2e_calls[0] = i + 1

    for _ in range(max(3, args.warmup)):
        e2e_step()
    if dist:
        dist.barrier()
    lstream = torch.cuda.ExternalStream(lib.ckb200_stream())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(args.steps, 20)
    e0.record(lstream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(lstream)
    lstream.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    if dist:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_bytes = sum(p["bytes"] for p in plan)
    e2e = {"value": world * e2e_bytes * e2e_steps / e2e_ms / 1e6, "unit": UNIT,
           "h2d_bytes_per_step": sum(q["xq_bytes"] for q in pinned), "d2h_bytes_per_step": sum(4 * q["p"]["m"] for q in pinned),
           "call": "gemv_q4_k_q8_k(y_host, W_host_registered, x_q8_host, M, K), one call per sweep shape per step, weights rotating over "
                   + "/".join(str(q["rot"]) for q in pinned) + " resident copies",
           "ms_per_step": e2e_ms / e2e_steps}
    for q in pinned:
        lib.ckb200_unregister_weights(vptr(q["w"]))
        lib.ckb200_host_free(C.c_void_p(q["hx"]))
        lib.ckb200_host_free(C.c_void_p(q["hy"]))
    pinned.clear()
    pkg.check(lib)

    decode_tp = None
    if world > 1 and not args.no_decode:
        try:
            pkg.tp.setup(lib, rank, world, dev, p2p_floats=32 * LLAMA3_70B["embed_dim"])
            decode_tp = []
            kept = []
            forms = ((1, 1, "peer-memory exchange fused into the residual-add + RMSNorm + quantise kernel"),
                     (1, 0, "one-shot push all-reduce kernel over peer memory"), (0, 0, "NCCL all-reduce"))
            for p2p, fused, how in forms:
                lib.ckb200_tune_set(b"tp_p2p", p2p)
                lib.ckb200_tune_set(b"tp_fused_norm", fused)
                d = decode_bench(lib, f"Llama-3-70B shape, Q4_K_M mix, TP={world}", LLAMA3_70B, 4096, 20, measured_peak()[0],
                                 batch=1, tp_rank=rank, tp_size=world, dist=dist, keep_logits=kept)
                d["exchange"] = how
                if "error" not in d and len(kept) == len(decode_tp) + 1:
                    # correctness carried with the number: the replicated LM head must see the same hidden state on every rank, and the
                    # three exchange forms must agree with each other
                    mine = kept[-1]
                    hi, lo = mine.clone(), mine.clone()
                    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                    first = kept[0].double()
                    cos = float((first @ mine.double()) / (first.norm() * mine.double().norm()))
                    d["logits_check"] = {"max_abs_spread_across_ranks": float((hi - lo).abs().max().item()), "finite": bool(torch.isfinite(mine).all().item()),
                                         "cosine_vs_first_form_rank0": cos, "max_abs_logit": float(mine.abs().max().item())}
                decode_tp.append(d)
            lib.ckb200_tune_set(b"tp_p2p", 1)
            lib.ckb200_tune_set(b"tp_fused_norm", -1)                    # the library's own choice by rank count
            d = decode_bench(lib, f"Llama-3-70B shape, Q4_K_M mix, TP={world}, batch 1 (default exchange)", LLAMA3_70B, 4096, 20, measured_peak()[0],
                             batch=1, tp_rank=rank, tp_size=world, dist=dist)
            d["exchange"] = "default"
            decode_tp.append(d)
            d = decode_bench(lib, f"Llama-3-70B shape, Q4_K_M mix, TP={world}, batch 32", LLAMA3_70B, 4096, 4, measured_peak()[0],
                             batch=32, tp_rank=rank, tp_size=world, dist=dist)
            d["exchange"] = "default"
            decode_tp.append(d)
        except Exception as exc:
            decode_tp = {"error": repr(exc)}
            lib.ckb200_clear_error()

    if rank == 0:
        r = results["q4_k"]
        peak, peak_kind = measured_peak()
        gbs_one = r["step_bytes"] * args.steps / r["ms"] / 1e6
        value = gbs_one * world
        sweeps = {}
        for name, rr in results.items():
            g = rr["step_bytes"] * args.steps / rr["ms"] / 1e6
            sweeps[name] = {"gbs": g, "frac": g / peak, "serial_chain_gbs": rr["serial_gbs"], "frac_serial_chain": rr["serial_gbs"] / peak if rr["serial_gbs"] else None,
                            "bytes_per_step": rr["step_bytes"], "launches_per_step": int(rr["launches"]), "rotation": rr["rotation"], "entry_point": SWEEPS[name][2]}
            if rr["per_shape"]:
                sweeps[name]["per_shape"] = rr["per_shape"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": r["ms"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 dot (dp4a), fp32 accumulate", "data": "synthetic",
            "config": sweep_config(),
            "method": {"l2": "every launch reads a different weight copy; copies per shape total > 4x L2 (rotation " + r["rotation"] + ")",
                       "sharding": "each rank streams its own shard of rows; no collective in the data path",
                       "timing": "CUDA graph of one step replayed; CUDA events on the launching stream; max over ranks",
                       "schedule": f"the launches of a step are independent GEMVs and are dealt round-robin to {args.streams} stream(s) "
                                   "(parallel branches of the graph, one CTA per SM per launch), as the step executor does with q/k/v; "
                                   "frac_serial_chain is the same step as one dependent chain on one stream at full occupancy"},
            "serial_chain_gbs": (r["serial_gbs"] * world) if r["serial_gbs"] else None,
            "clocks": {k: r["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")} if r["clocks"] else None,
            "e2e": e2e,
            "gpu_launches": int(sum(rr["launches"] for rr in results.values()) * args.steps),
            "roofline": {"bound": "hbm", "achieved": gbs_one, "peak": peak, "unit": "GB/s", "frac": gbs_one / peak,
                         "frac_serial_chain": r["serial_gbs"] / peak if r["serial_gbs"] else None,
                         "traffic": Q4K_DRAM_TRAFFIC_RATIO * r["step_bytes"],
                         "traffic_note": "DRAM bytes per step = measured DRAM / algorithmic ratio of one launch (ncu, 14336x4096) x the step's algorithmic bytes",
                         "peak_kind": peak_kind, "kernel": "Q4_K GEMV (all sweep shapes)", "bytes_per_step": r["step_bytes"]},
            "sweeps": sweeps,
        }
        if world == 1 and not args.no_decode:
            try:
                line["decode"] = [decode_bench(lib, "Qwen2-0.5B shape, Q4_K_M mix", QWEN2_05B, 1024, 200, peak),
                                  decode_bench(lib, "Llama-3-70B shape, Q4_K_M mix, 1 GPU", LLAMA3_70B, 4096, 10, peak),
                                  decode_bench(lib, "Llama-3-70B shape, Q4_K_M mix, 1 GPU, batch 8", LLAMA3_70B, 4096, 6, peak, batch=8),
                                  decode_bench(lib, "Llama-3-70B shape, Q4_K_M mix, 1 GPU, batch 32", LLAMA3_70B, 4096, 4, peak, batch=32),
                                  decode_bench(lib, "Llama-3-70B shape, Q4_K_M mix, 1 GPU, batch 32, fp16 cache", LLAMA3_70B, 4096, 4, peak, batch=32,
                                               kv_f16=True)]
            except Exception as exc:                      # the headline metric above must survive a failure here
                line["decode"] = {"error": repr(exc)}
                lib.ckb200_clear_error()
            try:
                line["attention"] = attention_bench(lib, torch, peak)
            except Exception as exc:
                line["attention"] = {"error": repr(exc)}
                lib.ckb200_clear_error()
            try:
                line["prefill"] = prefill_bench(lib, 512, 20, sp, torch, measured_tensor_peak())
                line["prefill"]["whole_stack"] = prefill_step_bench(lib)
            except Exception as exc:
                line["prefill"] = {"error": repr(exc)}
                lib.ckb200_clear_error()
        if decode_tp is not None:
            line["decode_tp"] = decode_tp
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


PREFILL_SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336)]      # (N, K) of the Llama-3-8B projections


def prefill_bench(lib, m_tokens, iters, stream_ptr, torch, tensor_peak):
    """Batched quantised GEMM C[M,N] = A_q8k[M,K] . W_q4k[N,K]^T at prefill size (tcgen05 kernel), per projection shape."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {"workload": f"Llama-3-8B-shaped prefill GEMM, Q4_K x Q8_K, M={m_tokens}", "shapes": {}}
    flops_total, ms_total = 0.0, 0.0
    for n, k in PREFILL_SHAPES:
        w = torch.from_numpy(synth.make_weights("q4_k", n, k, seed=3)).to(dev)
        a = torch.from_numpy(synth.make_x(k, seed=3, rows=m_tokens)).to(dev)
        aq = torch.empty(m_tokens * synth.row_bytes("q8_k", k) + 64, dtype=torch.uint8, device=dev)
        c = torch.empty(m_tokens, n, dtype=torch.float32, device=dev)
        assert lib.ckb200_dev_quantize_q8_k(C.c_void_p(a.data_ptr()), C.c_void_p(aq.data_ptr()), m_tokens, k, stream_ptr) == 0

        def run():
            rc = lib.ckb200_dev_gemm_nt_q4_k_q8_k(C.c_void_p(aq.data_ptr()), C.c_void_p(w.data_ptr()), None, C.c_void_p(c.data_ptr()),
                                                  m_tokens, n, k, stream_ptr)
            if rc != 0:
                raise RuntimeError(lib.ckb200_last_error_message().decode())

        for _ in range(3):
            run()
        torch.cuda.synchronize()
        if stream_ptr is None:                             # launches go to the library's own stream: time on that one
            lib.ckb200_stream.restype = C.c_void_p
            st = torch.cuda.ExternalStream(lib.ckb200_stream())
        else:
            st = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            run()
        e1.record(st)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        flops = 2.0 * m_tokens * n * k
        out["shapes"][f"{n}x{k}"] = {"ms": ms, "tflops": flops / ms / 1e9, "tokens_per_s": m_tokens / ms * 1e3}
        flops_total += flops
        ms_total += ms
    # causal attention of the same prefill (Llama-3-8B heads), fp32 head-major tensors resident on the device
    H, Hkv, d = 32, 8, 128
    gen = torch.Generator(device=dev).manual_seed(5)
    q = torch.randn(H, m_tokens, d, device=dev, generator=gen)
    kk = torch.randn(Hkv, m_tokens, d, device=dev, generator=gen)
    vv = torch.randn(Hkv, m_tokens, d, device=dev, generator=gen)
    oo = torch.empty_like(q)
    lib.ckb200_stream.restype = C.c_void_p
    st = torch.cuda.ExternalStream(lib.ckb200_stream()) if stream_ptr is None else torch.cuda.current_stream()

    def attn():
        rc = lib.ckb200_dev_attention_prefill(C.c_void_p(q.data_ptr()), C.c_void_p(kk.data_ptr()), C.c_void_p(vv.data_ptr()), C.c_void_p(oo.data_ptr()),
                                              H, Hkv, m_tokens, d, d, m_tokens, 1, stream_ptr)
        if rc != 0:
            raise RuntimeError(lib.ckb200_last_error_message().decode())

    torch.cuda.synchronize()
    for _ in range(3):
        attn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for _ in range(iters):
        attn()
    e1.record(st)
    torch.cuda.synchronize()
    attn_ms = e0.elapsed_time(e1) / iters
    attn_flops = 4.0 * (m_tokens * (m_tokens + 1) / 2) * d * H
    out["causal_attention"] = {"shape": f"H={H} Hkv={Hkv} d={d} T={m_tokens}", "ms": attn_ms, "tflops_fp32": attn_flops / attn_ms / 1e9,
                               "note": "tensor cores at fp32 accuracy: every operand split into two fp16 pieces, three mma.sync per product (tflops_fp32 counts each product once)"}
    # the prefill GEMMs the reference's thread-pool seam dispatches (version/v7/src/ck_parallel_prefill.h:44-48), from the reference's
    # own weight layouts: Q6_K (rows re-laid per call, then the tcgen05 kernel) and Q8_0 (int8 MMAs, bit-identical to the scalar loop)
    seam = {}
    for fmt, entry, (n, k) in (("q6_k", lib.ckb200_dev_gemm_nt_q6_k_q8_k, (4096, 4096)), ("q8_0", lib.ckb200_dev_gemm_nt_q8_0_q8_0, (4096, 4096))):
        w = torch.from_numpy(synth.make_weights(fmt, n, k, seed=4)).to(dev)
        a = torch.from_numpy(synth.make_x(k, seed=4, rows=m_tokens)).to(dev)
        aq = torch.empty(m_tokens * synth.row_bytes("q8_k" if fmt == "q6_k" else "q8_0", k) + 64, dtype=torch.uint8, device=dev)
        quant = lib.ckb200_dev_quantize_q8_k if fmt == "q6_k" else lib.ckb200_dev_quantize_q8_0
        assert quant(C.c_void_p(a.data_ptr()), C.c_void_p(aq.data_ptr()), m_tokens, k, stream_ptr) == 0
        c = torch.empty(m_tokens, n, dtype=torch.float32, device=dev)

        def run2(entry=entry, aq=aq, w=w, c=c, n=n, k=k):
            if entry(C.c_void_p(aq.data_ptr()), C.c_void_p(w.data_ptr()), None, C.c_void_p(c.data_ptr()), m_tokens, n, k, stream_ptr) != 0:
                raise RuntimeError(lib.ckb200_last_error_message().decode())

        for _ in range(3):
            run2()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            run2()
        e1.record(st)
        torch.cuda.synchronize()
        ms2 = e0.elapsed_time(e1) / iters
        seam[f"gemm_nt_{fmt}_q8_{'k' if fmt == 'q6_k' else '0'} {n}x{k}"] = {"ms": ms2, "tflops": 2.0 * m_tokens * n * k / ms2 / 1e9}
    out["reference_layout_gemms"] = seam
    out["tflops"] = flops_total / ms_total / 1e9
    out["roofline"] = {"bound": "tensor", "achieved": out["tflops"], "peak": tensor_peak, "unit": "TFLOP/s", "frac": out["tflops"] / tensor_peak,
                       "note": "2*M*N*K of the f16 MMA; peak = measured cuBLAS bf16 burst"}
    if lib.ckb200_synchronize() != 0:
        raise RuntimeError(lib.ckb200_last_error_message().decode())
    return out


LLAMA3_8B = dict(embed_dim=4096, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336, num_layers=32, vocab_size=128256,
                 max_seq_len=1024, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=0, fmt_o=0, fmt_gate_up=0, fmt_down=0, fmt_lm_head=0)


def prefill_step_bench(lib, tokens=512, iters=5):
    """The whole Llama-3-8B-shaped stack (32 layers, Q4_K weights, Q8_K activations, causal attention) over a 512-token prompt through
    ckb200_model_prefill: prompt ids in from the host, the last token's logits back, per iteration from an empty cache."""
    so = pkg.model_api
    so.bind_model_api(lib)
    handle = lib.ckb200_model_create(C.byref(so.make_cfg(LLAMA3_8B, batch=1)))
    if not handle:
        msg = lib.ckb200_last_error_message().decode()
        lib.ckb200_clear_error()
        return {"error": msg}
    try:
        assert lib.ckb200_model_fill_synthetic(handle, 1) == 0
        prompt = np.random.default_rng(0).integers(0, LLAMA3_8B["vocab_size"], size=tokens).astype(np.int32)
        logits = np.zeros((1, LLAMA3_8B["vocab_size"]), np.float32)
        lib.ckb200_model_reset.argtypes = [C.c_void_p]
        times = []
        launches = 0
        for i in range(iters + 1):
            assert lib.ckb200_model_reset(handle) == 0
            n0 = lib.ckb200_launch_count()
            t0 = time.perf_counter()
            assert lib.ckb200_model_prefill(handle, vptr(prompt), tokens, vptr(logits)) == 0, lib.ckb200_last_error_message()
            if i:
                times.append(time.perf_counter() - t0)
            launches = lib.ckb200_launch_count() - n0
        ms = statistics.median(times) * 1e3
        flops = 2.0 * tokens * sum(n * k for n, k in ((4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (28672, 4096), (4096, 14336))) * LLAMA3_8B["num_layers"]
        return {"workload": f"Llama-3-8B-shaped prefill, {tokens}-token prompt, 32 layers, Q4_K x Q8_K, causal attention, host ids in / last logits out",
                "ms": ms, "prompt_tokens_per_s": tokens / ms * 1e3, "projection_tflops": flops / ms / 1e9, "launches": int(launches),
                "finite": bool(np.isfinite(logits).all())}
    finally:
        lib.ckb200_model_free(handle)


def run_prefill_only(args):
    """Plain launches of the prefill GEMM: the command behind the tensor-core profile."""
    import torch

    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    print(json.dumps(prefill_bench(lib, args.prefill_only, args.launches, None, torch, measured_tensor_peak())))


def run_prefill_stack_only(args):
    """Two whole-stack prefill passes (Llama-3-8B shape): the command behind the prefill launch list."""
    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    lib.ckb200_launch_count.restype = C.c_longlong
    print(json.dumps(prefill_step_bench(lib, args.prefill_stack_only, iters=1)))


def run_single(args):
    """A few plain (un-captured) launches of one GEMV on rotating weight copies: the small case for ncu captures.
    FMT: q4_k, q6_k (ring kernel on the reference's rows), q6_k_planar, q8_0, q8_0_planar, q5_0, q5_0_planar."""
    import torch

    name, shape = args.single.split(":")
    planar = name.endswith("_planar")
    fmt = name[:-7] if planar else name
    m, k = (int(v) for v in shape.split("x"))
    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    dev = torch.device("cuda", 0)
    gemv = {"q4_k": lib.ckb200_dev_gemv_q4_k_q8_k, "q6_k": lib.ckb200_dev_gemv_q6_k_q8_k, "q8_0": lib.ckb200_dev_gemv_q8_0_q8_0,
            "q6_k_planar": lib.ckb200_dev_gemv_q6_k_planar_q8_k, "q8_0_planar": lib.ckb200_dev_gemv_q8_0_planar_q8_0,
            "q5_0": lib.ckb200_dev_gemv_q5_0_q8_0, "q5_0_planar": lib.ckb200_dev_gemv_q5_0_planar_q8_0}[name]
    quant = lib.ckb200_dev_quantize_q8_0 if fmt in ("q8_0", "q5_0") else lib.ckb200_dev_quantize_q8_k
    w_host = synth.make_weights(fmt, m, k, seed=1)
    src = torch.from_numpy(w_host).to(dev)
    nbytes = w_host.nbytes
    if planar:
        size_fn, conv_fn = {"q6_k": (lib.ckb200_q6_k_planar_bytes, lib.ckb200_dev_q6_k_to_planar),
                            "q8_0": (lib.ckb200_q8_0_planar_bytes, lib.ckb200_dev_q8_0_to_planar),
                            "q5_0": (lib.ckb200_q5_0_planar_bytes, lib.ckb200_dev_q5_0_to_planar)}[fmt]
        size_fn.restype = C.c_size_t
        nbytes = size_fn(m, k)
        dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        assert conv_fn(C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), m, k, None) == 0
        assert lib.ckb200_synchronize() == 0
        src = dst
    copies = max(2, min(8, -(-600_000_000 // nbytes)))          # > L2 in total, well under 1 GB on the device
    slot = (nbytes + 255) & ~255
    wbuf = torch.empty(copies * slot + 256, dtype=torch.uint8, device=dev)
    for c in range(copies):
        wbuf[c * slot:c * slot + nbytes].copy_(src)
    x = torch.from_numpy(synth.make_x(k, seed=1)).to(dev)
    xq = torch.empty(synth.row_bytes("q8_0" if fmt in ("q8_0", "q5_0") else "q8_k", k) + 64, dtype=torch.uint8, device=dev)
    y = torch.empty(copies, m, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    assert quant(C.c_void_p(x.data_ptr()), C.c_void_p(xq.data_ptr()), 1, k, None) == 0
    for i in range(args.launches):
        c = i % copies
        assert gemv(C.c_void_p(y[c].data_ptr()), C.c_void_p(wbuf.data_ptr() + c * slot), C.c_void_p(xq.data_ptr()), m, k, None) == 0
    assert lib.ckb200_synchronize() == 0
    print(json.dumps({"single": args.single, "launches": args.launches, "copies": copies, "bytes_per_launch": synth.gemv_bytes(fmt, m, k)}))


def attention_bench(lib, torch, peak, iters=40):
    """Decode attention of the 70B shape (64 Q / 8 KV heads, d 128, context 4096) over an fp32 and an IEEE fp16 KV cache, batch 1 and
    32, each launch on another layer's cache (the caches of a case total several L2 sizes).  Times cover attention and split merge."""
    lib.ckb200_attention_decode_scratch_bytes.restype = C.c_size_t
    lib.ckb200_stream.restype = C.c_void_p
    dev = torch.device("cuda", torch.cuda.current_device())
    st = torch.cuda.ExternalStream(lib.ckb200_stream())
    H, Hkv, d, T = 64, 8, 128, 4096
    out = []
    for batch, nl in ((1, 12), (32, 2)):
        for kind, dt, eb, fn in (("fp32", torch.float32, 4, lib.ckb200_dev_attention_decode_ws), ("fp16", torch.float16, 2, lib.ckb200_dev_attention_decode_f16cache_ws)):
            q = torch.randn(batch, H, d, device=dev)
            o = torch.empty_like(q)
            kc = torch.randn(nl, batch, Hkv, T, d, device=dev, dtype=dt)
            vc = torch.randn(nl, batch, Hkv, T, d, device=dev, dtype=dt)
            splits = lib.ckb200_attention_decode_splits_kv(batch, Hkv, T, eb)
            scratch = torch.empty(max(256, lib.ckb200_attention_decode_scratch_bytes(batch, H, d, splits)) // 4, device=dev)

            def run(i):
                l = i % nl
                rc = fn(C.c_void_p(q.data_ptr()), C.c_void_p(kc[l].data_ptr()), C.c_void_p(vc[l].data_ptr()), C.c_void_p(o.data_ptr()), batch,
                        C.c_longlong(Hkv * T * d), H, Hkv, T, T, d, d, splits, C.c_void_p(scratch.data_ptr()), None, None)
                if rc != 0:
                    raise RuntimeError(lib.ckb200_last_error_message().decode())

            torch.cuda.synchronize()
            for i in range(3):
                run(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for i in range(iters):
                run(i)
            e1.record(st)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            nbytes = batch * (2 * Hkv * T * d * eb + 2 * H * d * 4)
            out.append({"kv_cache": kind, "batch": batch, "us": ms * 1e3, "kv_bytes": nbytes, "gbs": nbytes / ms / 1e6, "frac_of_measured_peak": nbytes / ms / 1e6 / peak,
                        "splits": splits})
            del kc, vc
    # the llama template's attention (fp32 cache read through fp16 rounding, accumulator rounded after every key): an ordered walk, latency-bound
    q = torch.randn(1, H, d, device=dev)
    o = torch.empty_like(q)
    kc = torch.randn(12, Hkv, T, d, device=dev)
    vc = torch.randn(12, Hkv, T, d, device=dev)

    def run_f16kv(i):
        l = i % 12
        rc = lib.ckb200_dev_attention_decode_f16kv(C.c_void_p(q.data_ptr()), C.c_void_p(kc[l].data_ptr()), C.c_void_p(vc[l].data_ptr()), C.c_void_p(o.data_ptr()),
                                                   H, Hkv, T, T, d, d, None, None)
        if rc != 0:
            raise RuntimeError(lib.ckb200_last_error_message().decode())

    torch.cuda.synchronize()
    for i in range(3):
        run_f16kv(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for i in range(iters):
        run_f16kv(i)
    e1.record(st)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    nbytes = 2 * Hkv * T * d * 4 + 2 * H * d * 4
    out.append({"kv_cache": "fp32 read as fp16, fp16-rounded accumulator (attention_forward_decode_head_major_gqa_flash_f16kv)", "batch": 1, "us": ms * 1e3,
                "kv_bytes": nbytes, "gbs": nbytes / ms / 1e6, "frac_of_measured_peak": nbytes / ms / 1e6 / peak, "splits": 1,
                "note": "keys are walked in order (the rounding sequence is part of the result): about 15 cycles per key"})
    if lib.ckb200_synchronize() != 0:
        raise RuntimeError(lib.ckb200_last_error_message().decode())
    return out


def run_attention_only(args):
    """Plain launches of decode attention on the 70B shape (64 Q / 8 KV heads, d 128) over rotating KV caches."""
    import torch

    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    lib.ckb200_attention_decode_scratch_bytes.restype = C.c_size_t
    dev = torch.device("cuda", 0)
    H, Hkv, d, T, cap, nl = 64, 8, 128, args.attention_only, args.attention_only + 256, 8
    q = torch.randn(1, H, d, device=dev)
    out = torch.empty_like(q)
    kc = torch.randn(nl, Hkv, cap, d, device=dev)
    vc = torch.randn(nl, Hkv, cap, d, device=dev)
    splits = lib.ckb200_attention_decode_splits(1, Hkv, T)
    scratch = torch.empty(max(256, lib.ckb200_attention_decode_scratch_bytes(1, H, d, splits)) // 4, device=dev)
    torch.cuda.synchronize()
    for i in range(args.launches):
        l = i % nl
        assert lib.ckb200_dev_attention_decode_ws(C.c_void_p(q.data_ptr()), C.c_void_p(kc[l].data_ptr()), C.c_void_p(vc[l].data_ptr()), C.c_void_p(out.data_ptr()),
                                                  1, C.c_longlong(Hkv * cap * d), H, Hkv, T, cap, d, d, splits, C.c_void_p(scratch.data_ptr()), None, None) == 0
    for i in range(args.launches):          # and the fp16-rounded form on the same caches
        l = i % nl
        assert lib.ckb200_dev_attention_decode_f16kv(C.c_void_p(q.data_ptr()), C.c_void_p(kc[l].data_ptr()), C.c_void_p(vc[l].data_ptr()), C.c_void_p(out.data_ptr()),
                                                     H, Hkv, T, cap, d, d, None, None) == 0
    assert lib.ckb200_synchronize() == 0
    print(json.dumps({"attention_only": T, "launches": args.launches, "splits": splits, "kv_bytes_per_launch": 2 * Hkv * T * d * 4}))
    if args.batch > 1:
        # the same shape for --batch sequences over IEEE fp16 caches (the tensor-core kernel), timed with events
        B = args.batch
        del kc, vc
        q = torch.randn(B, H, d, device=dev)
        out = torch.empty_like(q)
        kc16 = torch.randn(2, B, Hkv, cap, d, device=dev, dtype=torch.float16)
        vc16 = torch.randn(2, B, Hkv, cap, d, device=dev, dtype=torch.float16)
        splits = lib.ckb200_attention_decode_splits_kv(B, Hkv, T, 2)
        scratch = torch.empty(max(256, lib.ckb200_attention_decode_scratch_bytes(B, H, d, 64)) // 4, device=dev)
        lstream = torch.cuda.ExternalStream(lib.ckb200_stream())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()

        def launch16(i):
            l = i % 2
            assert lib.ckb200_dev_attention_decode_f16cache_ws(C.c_void_p(q.data_ptr()), C.c_void_p(kc16[l].data_ptr()), C.c_void_p(vc16[l].data_ptr()),
                                                               C.c_void_p(out.data_ptr()), B, C.c_longlong(Hkv * cap * d), H, Hkv, T, cap, d, d, splits,
                                                               C.c_void_p(scratch.data_ptr()), None, None) == 0

        for i in range(2):
            launch16(i)
        e0.record(lstream)
        for i in range(args.launches):
            launch16(i)
        e1.record(lstream)
        assert lib.ckb200_synchronize() == 0
        us = e0.elapsed_time(e1) / args.launches * 1e3
        kv_bytes = 2 * B * Hkv * T * d * 2
        print(json.dumps({"attention_only": T, "batch": B, "kv_cache": "fp16", "launches": args.launches, "splits": splits, "us_per_launch": us,
                          "kv_bytes_per_launch": kv_bytes, "tb_s": kv_bytes / us / 1e6}))
        # and over fp32 caches (keys and values split into fp16 pieces in the kernel)
        del kc16, vc16
        kc32 = torch.randn(2, B, Hkv, cap, d, device=dev)
        vc32 = torch.randn(2, B, Hkv, cap, d, device=dev)
        splits = lib.ckb200_attention_decode_splits_kv(B, Hkv, T, 4)
        torch.cuda.synchronize()

        def launch32(i):
            l = i % 2
            assert lib.ckb200_dev_attention_decode_ws(C.c_void_p(q.data_ptr()), C.c_void_p(kc32[l].data_ptr()), C.c_void_p(vc32[l].data_ptr()),
                                                      C.c_void_p(out.data_ptr()), B, C.c_longlong(Hkv * cap * d), H, Hkv, T, cap, d, d, splits,
                                                      C.c_void_p(scratch.data_ptr()), None, None) == 0

        for i in range(2):
            launch32(i)
        e0.record(lstream)
        for i in range(args.launches):
            launch32(i)
        e1.record(lstream)
        assert lib.ckb200_synchronize() == 0
        us = e0.elapsed_time(e1) / args.launches * 1e3
        print(json.dumps({"attention_only": T, "batch": B, "kv_cache": "fp32", "launches": args.launches, "splits": splits, "us_per_launch": us,
                          "kv_bytes_per_launch": 2 * kv_bytes, "tb_s": 2 * kv_bytes / us / 1e6}))


def run_small_gemm_only(args):
    """Plain launches of gemm_nt_q4_k_q8_k (or, with --small-gemm-fmt q6_k, of the planar Q6_K product) for a handful of tokens (M,N,K):
    the small case behind profiles/gemm_q4k_mma_*.md and gemm_q6k_mma_*.md, with event timing."""
    import torch

    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    M, N, K = (int(v) for v in args.small_gemm_only.split(","))
    dev = torch.device("cuda", 0)
    nb = K // 256
    q6 = args.small_gemm_fmt == "q6_k"
    lib.ckb200_q6_k_planar_bytes.restype = C.c_size_t
    wbytes = lib.ckb200_q6_k_planar_bytes(N, K) if q6 else N * nb * 144
    copies = max(1, min(8, int(300e6 // wbytes)))                      # rotate over more than L2 of weights where that stays small
    W = torch.empty(copies * wbytes, dtype=torch.uint8, device=dev)
    if q6:                                                             # random Q6_K rows, re-laid row-planar as resident weights are
        raw = torch.empty(N * nb * 210, dtype=torch.uint8, device=dev)
        assert lib.ckb200_dev_fill_blocks(C.c_void_p(raw.data_ptr()), C.c_longlong(N * nb), 1, C.c_ulonglong(5), None) == 0
        for c in range(copies):
            assert lib.ckb200_dev_q6_k_to_planar(C.c_void_p(W.data_ptr() + c * wbytes), C.c_void_p(raw.data_ptr()), N, K, None) == 0
        del raw
    else:
        assert lib.ckb200_dev_fill_blocks(C.c_void_p(W.data_ptr()), C.c_longlong(copies * N * nb), 0, C.c_ulonglong(5), None) == 0
    x = torch.randn(M, K, device=dev)
    xq = torch.empty(M * nb * 292, dtype=torch.uint8, device=dev)
    assert lib.ckb200_dev_quantize_q8_k(C.c_void_p(x.data_ptr()), C.c_void_p(xq.data_ptr()), M, K, None) == 0
    out = torch.zeros(M, N, device=dev)
    lstream = torch.cuda.ExternalStream(lib.ckb200_stream())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    gemm = lib.ckb200_dev_gemm_nt_q6_k_planar_q8_k if q6 else lib.ckb200_dev_gemm_nt_q4_k_q8_k

    def launch(i):
        w = W.data_ptr() + (i % copies) * wbytes
        assert gemm(C.c_void_p(xq.data_ptr()), C.c_void_p(w), None, C.c_void_p(out.data_ptr()), M, N, K, None) == 0

    for i in range(3):
        launch(i)
    e0.record(lstream)
    for i in range(args.launches):
        launch(i)
    e1.record(lstream)
    assert lib.ckb200_synchronize() == 0
    us = e0.elapsed_time(e1) / args.launches * 1e3
    print(json.dumps({"small_gemm_only": [M, N, K], "fmt": args.small_gemm_fmt, "launches": args.launches, "us_per_launch": us, "weight_bytes": wbytes,
                      "weights_tb_s": wbytes / us / 1e6}))


def run_decode_only(args):
    """Eager (un-captured) decode steps of a model shape: the command behind the decode launch lists in profiles/."""
    so = pkg.model_api
    lib = pkg.load_lib()
    assert lib.ckb200_init(0) == 0
    so.bind_model_api(lib)
    cfg, ctx = (QWEN2_05B, 1024) if args.decode_only == "qwen2-0.5b" else (LLAMA3_70B, 4096)
    lib.ckb200_tune_set(b"model_graph", 0)
    st = so.make_cfg(cfg, batch=args.batch)
    h = lib.ckb200_model_create(C.byref(st))
    assert h, lib.ckb200_last_error_message()
    assert lib.ckb200_model_fill_synthetic(h, 1) == 0 and lib.ckb200_model_fill_kv_synthetic(h, ctx, 2) == 0
    ids = np.full(args.batch, 11, np.int32)
    lib.ckb200_launch_count.restype = C.c_longlong
    n0 = lib.ckb200_launch_count()
    for _ in range(args.steps):
        assert lib.ckb200_model_decode(h, vptr(ids), None) == 0
    assert lib.ckb200_synchronize() == 0
    print(json.dumps({"decode_only": args.decode_only, "batch": args.batch, "steps": args.steps, "launches_per_step": (lib.ckb200_launch_count() - n0) // args.steps}))
    lib.ckb200_model_free(h)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--detail", action="store_true", help="also time the Q5_0 sweeps and every shape on its own")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-step tokens/s section")
    ap.add_argument("--streams", type=int, default=8, help="streams the independent GEMV launches of a sweep step are dealt to")
    ap.add_argument("--single", default=None, metavar="FMT:MxK", help="profiling aid: plain launches of one GEMV, e.g. q4_k:14336x4096, q6_k_planar:14336x4096")
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--prefill-only", type=int, default=None, metavar="M", help="profiling aid: the prefill GEMM section alone at M tokens")
    ap.add_argument("--prefill-stack-only", type=int, default=None, metavar="T", help="profiling aid: whole-stack prefill of a T-token prompt, twice")
    ap.add_argument("--small-gemm-only", default=None, metavar="M,N,K", help="profiling aid: gemm_nt_q4_k_q8_k (or planar Q6_K) launches for a few tokens")
    ap.add_argument("--small-gemm-fmt", default="q4_k", choices=["q4_k", "q6_k"])
    ap.add_argument("--attention-only", type=int, default=None, metavar="T", help="profiling aid: decode attention launches, 70B head shape, context T")
    ap.add_argument("--batch", type=int, default=1, help="sequences per step of --decode-only")
    ap.add_argument("--decode-only", default=None, choices=["qwen2-0.5b", "llama3-70b"], help="profiling aid: eager decode steps of one model shape")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE", help="set a kernel-variant switch of the library (ckb200_tune_set) before running")
    args = ap.parse_args()
    if args.tune:
        lib = pkg.load_lib()
        for kv in args.tune:
            key, _, val = kv.partition("=")
            lib.ckb200_tune_set(key.encode(), int(val))
    if args.single:
        return run_single(args)
    if args.decode_only:
        return run_decode_only(args)
    if args.attention_only:
        return run_attention_only(args)
    if args.small_gemm_only:
        return run_small_gemm_only(args)
    if args.prefill_only:
        return run_prefill_only(args)
    if args.prefill_stack_only:
        return run_prefill_stack_only(args)
    args.warmup = max(args.warmup, 3) if args.impl == "cuda" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
