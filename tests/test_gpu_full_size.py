"""Parity at the full sizes of the benchmark configurations: one decode step of the whole Qwen2-0.5B-shaped model (24 layers,
vocabulary 151 936, context 1024), one layer of the Llama-3-70B shape (hidden 8192, FFN 28 672, context 4096), the
tensor-core GEMM on a real prefill projection (512 x 4096 x 4096), and graph replay of a batched step after the library's
scratch pool has been regrown by another call."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases
import step_oracle as so

pytestmark = pytest.mark.gpu
synth = cases.synth

QWEN2_05B = dict(embed_dim=896, num_heads=14, num_kv_heads=2, head_dim=64, intermediate_size=4864, num_layers=24, vocab_size=151936,
                 max_seq_len=1088, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
LLAMA70B_LAYER = dict(embed_dim=8192, num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=28672, num_layers=1, vocab_size=2048,
                      max_seq_len=4160, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("cfg,ctx", [(QWEN2_05B, 1024), (LLAMA70B_LAYER, 4096)], ids=["qwen2-0.5b-24-layers", "llama3-70b-one-layer"])
def test_full_size_decode_step(ck, orc, cfg, ctx):
    so.bind_model_api(ck)
    cpu = so.CpuModel(cfg, seed=21)
    cpu.prefill_kv(ctx, seed=22)
    st = so.make_cfg(cfg, batch=1)
    handle = ck.ckb200_model_create(C.byref(st))
    assert handle, ck.ckb200_last_error_message()
    try:
        so.upload_whole_model(ck, handle, cpu, 1)
        assert ck.ckb200_model_set_pos(handle, ctx) == 0
        for step, tok in enumerate([12345 % cfg["vocab_size"], 777]):
            want = cpu.decode(orc, tok, ctx + step)
            ids = np.array([tok], dtype=np.int32)
            logits = np.full((1, cfg["vocab_size"]), np.nan, dtype=np.float32)
            assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
            cos = cosine(logits[0], want)
            err = float(np.max(np.abs(logits[0] - want))) / float(np.max(np.abs(want)))
            assert cos >= 0.9999, (step, cos)            # the contract for whole steps
            # max-abs bound relative to the largest logit: across 24 layers a Q8_K code that sits on a rounding boundary may fall
            # the other way (the fp32 sums feeding it are added in another order), which moves single logits by a fraction of a percent
            assert err < 2e-2, (step, err)
    finally:
        ck.ckb200_model_free(handle)


@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_tensor_core_gemm_on_prefill_projection_shapes(ck, orc, n, k):
    """512-token prefill projections of the Llama-3-8B shape through gemm_nt_q4_k_q8_k; the scalar oracle checks all 512
    tokens on every 16th weight row plus the first and last 128-row tiles."""
    m = 512
    w = synth.make_weights("q4_k", n, k, seed=n + k)
    a = synth.make_x(k, seed=n, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    assert np.array_equal(cases.quantize_act(ck, "", "q4_k", a, rows=m), aq)
    bias = np.random.default_rng(k).standard_normal(n).astype(np.float32)
    got = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
    assert np.isfinite(got).all()
    rows = sorted(set(range(0, n, 16)) | set(range(128)) | set(range(n - 128, n)))
    rb = synth.row_bytes("q4_k", k)
    wsub = np.ascontiguousarray(w.reshape(n, rb)[rows]).reshape(-1)
    want = cases.gemm_nt(orc, "oracle_", "q4_k", aq, wsub, np.ascontiguousarray(bias[rows]), m, len(rows), k)
    sub = got[:, rows]
    scale = float(np.max(np.abs(want)))
    err = np.abs(sub - want)
    worst = np.unravel_index(int(np.argmax(err)), err.shape)
    assert float(err.max()) <= 1e-5 * scale, f"max abs err {err.max():.3e} (scale {scale:.3e}) at token {worst[0]}, sampled row {rows[worst[1]]}; {(err > 1e-5 * scale).sum()} elements over"
    rel = err / np.maximum(np.abs(want), 1e-2 * scale)
    assert float(rel.max()) <= 1e-3


def test_batched_step_graph_survives_scratch_regrowth(ck, orc):
    """A batch-16 step records tensor-core GEMM launches in its graph; a large prefill GEMM through the host API afterwards makes
    the library's scratch pool free and regrow its buffers.  The replayed step must not read freed memory: same logits as before."""
    cfg = dict(embed_dim=512, num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1024, num_layers=2, vocab_size=777,
               max_seq_len=64, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
    so.bind_model_api(ck)
    cpu = so.CpuModel(cfg, seed=31)
    cpu.prefill_kv(20, seed=32)
    batch = 16
    st = so.make_cfg(cfg, batch=batch)
    handle = ck.ckb200_model_create(C.byref(st))
    assert handle, ck.ckb200_last_error_message()
    try:
        so.upload_whole_model(ck, handle, cpu, batch)
        ids = np.full(batch, 9, dtype=np.int32)
        first = np.zeros((batch, cfg["vocab_size"]), np.float32)
        assert ck.ckb200_model_set_pos(handle, 20) == 0
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(first)) == 0
        # a prefill-sized product through the pool: far larger activation tiles and partial sums than the step's
        m, n, k = 1024, 512, 8192
        w = synth.make_weights("q4_k", n, k, seed=5)
        aq = cases.quantize_act(orc, "oracle_", "q4_k", synth.make_x(k, seed=6, rows=m), rows=m)
        big = cases.gemm_nt(ck, "", "q4_k", aq, w, None, m, n, k)
        assert np.isfinite(big).all()
        again = np.zeros_like(first)
        assert ck.ckb200_model_set_pos(handle, 20) == 0
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(again)) == 0
        assert np.array_equal(first, again)
        want = cpu.decode(orc, 9, 20)
        assert cosine(again[0], want) >= 0.9999
    finally:
        ck.ckb200_model_free(handle)


def test_decode_past_the_context_is_refused(ck):
    so.bind_model_api(ck)
    cfg = dict(embed_dim=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512, num_layers=1, vocab_size=300,
               max_seq_len=8, rms_eps=1e-6, rope_theta=1.0e4, fmt_q=0, fmt_k=0, fmt_v=0, fmt_o=0, fmt_gate_up=0, fmt_down=0, fmt_lm_head=0)
    st = so.make_cfg(cfg, batch=1)
    handle = ck.ckb200_model_create(C.byref(st))
    assert handle
    try:
        assert ck.ckb200_model_fill_synthetic(handle, 1) == 0
        assert ck.ckb200_model_set_pos(handle, 7) == 0
        ids = np.array([3], dtype=np.int32)
        logits = np.zeros((1, 300), np.float32)
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0       # position 7: the last slot
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 6       # CKB_ERR_LIMIT: the context is full
        assert ck.ckb200_last_error() == 6
        ck.ckb200_clear_error()
        assert ck.ckb200_model_decode_repeat(handle, 1) == 6
        ck.ckb200_clear_error()
        assert ck.ckb200_model_set_pos(handle, 2) == 0
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0
    finally:
        ck.ckb200_model_free(handle)
        ck.ckb200_clear_error()
