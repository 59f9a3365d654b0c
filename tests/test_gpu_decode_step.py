"""Full decode steps on the device-resident executor against the CPU step built from the oracle's
kernels: logits cosine >= 0.9999 (the contract for whole steps) and a tight max-abs bound."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases
import step_oracle as so

pytestmark = pytest.mark.gpu

MINI_QWEN = dict(embed_dim=384, num_heads=6, num_kv_heads=2, head_dim=64, intermediate_size=768, num_layers=3, vocab_size=1000,
                 max_seq_len=96, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
MINI_LLAMA = dict(embed_dim=512, num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1024, num_layers=2, vocab_size=777,
                  max_seq_len=64, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)


# hidden size 384 is not a multiple of 256: the projections that read it are Q5_0 (32-element blocks, Q8_0 activations), as in
# GGUF Q4_K_M files of models like Qwen2-0.5B; the down projection (K = 768) stays a K-quant
MINI_Q5_0 = dict(embed_dim=384, num_heads=6, num_kv_heads=2, head_dim=64, intermediate_size=768, num_layers=3, vocab_size=500,
                 max_seq_len=96, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=3, fmt_k=3, fmt_v=3, fmt_o=3, fmt_gate_up=3, fmt_down=1, fmt_lm_head=1)


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("cfg,batch,use_graph", [(MINI_QWEN, 1, 1), (MINI_QWEN, 1, 0), (MINI_LLAMA, 2, 1), (MINI_LLAMA, 16, 1), (MINI_LLAMA, 5, 1),
                                                 (MINI_LLAMA, 33, 1), (MINI_Q5_0, 1, 1), (MINI_Q5_0, 1, 0)])   # from 4 sequences: tensor-core GEMMs
def test_decode_steps_match_cpu_step(ck, orc, cfg, batch, use_graph):
    so.bind_model_api(ck)
    ck.ckb200_tune_set(b"model_graph", use_graph)
    cpu = so.CpuModel(cfg, seed=7)
    start = 40
    cpu.prefill_kv(start, seed=8)
    st = so.make_cfg(cfg, batch=batch)
    handle = ck.ckb200_model_create(C.byref(st))
    assert handle, ck.ckb200_last_error_message()
    try:
        so.upload_whole_model(ck, handle, cpu, batch)
        assert ck.ckb200_model_set_pos(handle, start) == 0
        V = cfg["vocab_size"]
        tokens = [5, 17, 123]
        for step, tok in enumerate(tokens):
            want = cpu.decode(orc, tok, start + step)
            ids = np.full(batch, tok, dtype=np.int32)
            logits = np.full((batch, V), np.nan, dtype=np.float32)
            assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
            for b in range(batch):
                cos = cosine(logits[b], want)
                err = float(np.max(np.abs(logits[b] - want))) / float(np.max(np.abs(want)))
                assert cos >= 0.9999, (step, b, cos)
                assert err < 5e-3, (step, b, err)
            assert ck.ckb200_model_get_pos(handle) == start + step + 1
    finally:
        ck.ckb200_model_free(handle)
        ck.ckb200_tune_set(b"model_graph", 1)


@pytest.mark.parametrize("cfg,batch", [(MINI_QWEN, 1), (MINI_LLAMA, 2)])
def test_decode_steps_with_fp16_cache(ck, orc, cfg, batch):
    """tune model_kv_f16 = 1 at creation: k and v are rounded to IEEE halves on the store (kv_cache_store_f16) and attention widens
    them again (the reference's _f16cache decode attention); the CPU step keeps its caches the same way."""
    so.bind_model_api(ck)
    cpu = so.CpuModel(cfg, seed=17, kv_f16=True)
    start = 33
    cpu.prefill_kv(start, seed=18)
    st = so.make_cfg(cfg, batch=batch)
    ck.ckb200_tune_set(b"model_kv_f16", 1)
    try:
        handle = ck.ckb200_model_create(C.byref(st))
    finally:
        ck.ckb200_tune_set(b"model_kv_f16", 0)
    assert handle, ck.ckb200_last_error_message()
    try:
        assert ck.ckb200_model_kv_element_bytes(handle) == 2
        so.upload_whole_model(ck, handle, cpu, batch)
        assert ck.ckb200_model_set_pos(handle, start) == 0
        V, Hkv, d, S = cfg["vocab_size"], cfg["num_kv_heads"], cfg["head_dim"], cfg["max_seq_len"]
        for step, tok in enumerate([9, 41, 300]):
            want = cpu.decode(orc, tok, start + step)
            ids = np.full(batch, tok, dtype=np.int32)
            logits = np.full((batch, V), np.nan, dtype=np.float32)
            assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
            for b in range(batch):
                assert cosine(logits[b], want) >= 0.9999, (step, b)
                assert float(np.max(np.abs(logits[b] - want))) / float(np.max(np.abs(want))) < 5e-3, (step, b)
        # the stored halves of layer 0 (whose inputs do not depend on earlier attention) are the CPU step's, up to the last place of a half
        got = np.zeros((batch, Hkv, S, d), np.uint16)
        assert ck.ckb200_copy_to_host(cases.vptr(got), C.c_void_p(ck.ckb200_model_kv_device(handle, 0, 1)), got.nbytes) == 0
        a, w = got[0].view(np.float16).astype(np.float32), cpu.vc16[0].view(np.float16).astype(np.float32)
        np.testing.assert_array_equal(a[:, :start], w[:, :start])
        np.testing.assert_allclose(a[:, start:start + 3], w[:, start:start + 3], rtol=2e-3, atol=1e-4)
        assert not a[:, start + 3:].any()
        # prompts on such a model go through the step path (the batched prefill writes fp32 caches)
        assert ck.ckb200_model_reset(handle) == 0
    finally:
        ck.ckb200_model_free(handle)


def test_fp16_cache_refuses_unsupported_head_size(ck):
    so.bind_model_api(ck)
    cfg = dict(MINI_QWEN, head_dim=32, num_heads=12, num_kv_heads=4)
    ck.ckb200_tune_set(b"model_kv_f16", 1)
    try:
        assert not ck.ckb200_model_create(C.byref(so.make_cfg(cfg, batch=1)))
        assert b"fp16 cache" in ck.ckb200_last_error_message()
    finally:
        ck.ckb200_tune_set(b"model_kv_f16", 0)
        ck.ckb200_clear_error()


def test_synthetic_fill_and_repeat(ck):
    """Device-side synthetic weights: the step runs, logits are finite, the position advances per replay."""
    so.bind_model_api(ck)
    st = so.make_cfg(MINI_QWEN, batch=1)
    handle = ck.ckb200_model_create(C.byref(st))
    assert handle
    try:
        assert ck.ckb200_model_fill_synthetic(handle, 3) == 0
        assert ck.ckb200_model_fill_kv_synthetic(handle, 20, 4) == 0
        ids = np.array([11], dtype=np.int32)
        logits = np.zeros((1, MINI_QWEN["vocab_size"]), np.float32)
        assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0
        assert np.isfinite(logits).all() and float(np.abs(logits).max()) > 0
        assert ck.ckb200_model_decode_repeat(handle, 5) == 0
        assert ck.ckb200_synchronize() == 0
        assert ck.ckb200_model_get_pos(handle) == 26
    finally:
        ck.ckb200_model_free(handle)


@pytest.mark.parametrize("cfg", [MINI_QWEN, MINI_LLAMA], ids=["mini-qwen", "mini-llama"])
@pytest.mark.parametrize("pdl", [1, 0])
def test_fused_step_matches_the_launch_per_op_step(ck, orc, cfg, pdl):
    """One sequence on one GPU runs as five fused launches per layer (prologue: residual add + RMSNorm + Q8_K or plain Q8_K;
    epilogue: RoPE + cache store or SwiGLU); the launch-per-op step (tune model_fused_step 0) is the same arithmetic, so the two
    agree far inside the contract, and both match the CPU step.  With and without programmatic dependent launch."""
    so.bind_model_api(ck)
    cpu = so.CpuModel(cfg, seed=11)
    start = 33
    cpu.prefill_kv(start, seed=12)
    V = cfg["vocab_size"]
    tokens = [3, 250, 77, 8]
    want = [cpu.decode(orc, tok, start + i) for i, tok in enumerate(tokens)]
    got = {}
    launches = {}
    ck.ckb200_launch_count.restype = C.c_longlong
    try:
        ck.ckb200_tune_set(b"pdl", pdl)
        for fused in (1, 0):
            ck.ckb200_tune_set(b"model_fused_step", fused)
            cpu2 = so.CpuModel(cfg, seed=11)
            cpu2.prefill_kv(start, seed=12)
            handle = ck.ckb200_model_create(C.byref(so.make_cfg(cfg, batch=1)))
            assert handle, ck.ckb200_last_error_message()
            try:
                so.upload_whole_model(ck, handle, cpu2, 1)
                assert ck.ckb200_model_set_pos(handle, start) == 0
                outs = []
                for i, tok in enumerate(tokens):
                    ids = np.array([tok], dtype=np.int32)
                    logits = np.full((1, V), np.nan, dtype=np.float32)
                    n0 = ck.ckb200_launch_count()
                    assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
                    if i == 0:
                        launches[fused] = (ck.ckb200_launch_count() - n0) // 2      # the first call issues the step twice (warm-up, capture)
                    outs.append(logits[0].copy())
                    assert ck.ckb200_model_get_pos(handle) == start + i + 1
                got[fused] = outs
            finally:
                ck.ckb200_model_free(handle)
    finally:
        ck.ckb200_tune_set(b"model_fused_step", 1)
        ck.ckb200_tune_set(b"pdl", 1)
    assert 2 * launches[1] < launches[0], launches          # (both counts include the one-off weight re-layout launches)
    for i in range(len(tokens)):
        for fused in (1, 0):
            assert cosine(got[fused][i], want[i]) >= 0.9999, (fused, i)
        scale = float(np.max(np.abs(want[i])))
        assert float(np.max(np.abs(got[1][i] - got[0][i]))) <= 2e-3 * scale, i
        assert cosine(got[1][i], got[0][i]) >= 0.99999, i
