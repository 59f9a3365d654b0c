"""The batched prefill step against the CPU step: a prompt run as ONE pass (tensor-core GEMMs over all tokens, RoPE and KV fill
over all tokens, causal prefill attention) must leave the same logits and the same KV cache as the prompt fed token by token
through the CPU oracle's decode step, and decoding must continue seamlessly from the cache it filled."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases
import step_oracle as so

pytestmark = pytest.mark.gpu

PF_QWEN = dict(embed_dim=384, num_heads=6, num_kv_heads=2, head_dim=64, intermediate_size=768, num_layers=3, vocab_size=1000,
               max_seq_len=96, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
PF_LLAMA = dict(embed_dim=512, num_heads=8, num_kv_heads=2, head_dim=128, intermediate_size=1024, num_layers=2, vocab_size=777,
                max_seq_len=160, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("cfg,T", [(PF_QWEN, 40), (PF_LLAMA, 130), (PF_QWEN, 16)], ids=["qwen-40", "llama-130", "qwen-16"])
def test_prefill_step_matches_token_by_token_cpu(ck, orc, cfg, T):
    so.bind_model_api(ck)
    cpu = so.CpuModel(cfg, seed=41)
    rng = np.random.default_rng(T)
    prompt = rng.integers(0, cfg["vocab_size"], size=T).astype(np.int32)
    want = None
    for i, tok in enumerate(prompt):
        want = cpu.decode(orc, int(tok), i)
    handle = ck.ckb200_model_create(C.byref(so.make_cfg(cfg, batch=1)))
    assert handle, ck.ckb200_last_error_message()
    try:
        so.upload_whole_model(ck, handle, cpu.__class__(cfg, seed=41), 1)       # same weights, empty cache
        ck.ckb200_launch_count.restype = C.c_longlong
        n0 = ck.ckb200_launch_count()
        logits = np.full((1, cfg["vocab_size"]), np.nan, dtype=np.float32)
        assert ck.ckb200_model_prefill(handle, cases.vptr(prompt), T, cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
        launches = ck.ckb200_launch_count() - n0
        assert launches < 40 * cfg["num_layers"] + 40, f"{launches} launches: the prompt ran token by token"
        assert ck.ckb200_model_get_pos(handle) == T
        assert cosine(logits[0], want) >= 0.9999
        assert float(np.max(np.abs(logits[0] - want))) <= 2e-2 * float(np.max(np.abs(want)))
        # the cache it filled: every layer, rows 0 .. T-1
        Hkv, S, d = cfg["num_kv_heads"], cfg["max_seq_len"], cfg["head_dim"]
        for layer in range(cfg["num_layers"]):
            for is_v, ref in ((0, cpu.kc), (1, cpu.vc)):
                got = np.zeros((Hkv, S, d), np.float32)
                assert ck.ckb200_copy_to_host(cases.vptr(got), C.c_void_p(ck.ckb200_model_kv_device(handle, layer, is_v)), got.nbytes) == 0
                # Layer 0 differs by fp32 summation order only.  Deeper layers see the attention output of the layer below, and with
                # random weights the scores are so large that the softmax is nearly one-hot: where two keys almost tie, the order of
                # the fp32 sums decides their weights, so single tokens move by a few percent while the tensor as a whole agrees.
                scale = float(np.max(np.abs(ref[layer][:, :T])))
                if layer == 0:
                    assert float(np.max(np.abs(got[:, :T] - ref[layer][:, :T]))) <= 1e-4 * scale, is_v
                assert cosine(got[:, :T].reshape(-1), ref[layer][:, :T].reshape(-1)) >= 0.9999, (layer, is_v)
                assert not got[:, T:].any()
        # and decoding goes on from there
        for step, tok in enumerate((5, 77)):
            want = cpu.decode(orc, tok, T + step)
            ids = np.array([tok], dtype=np.int32)
            assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0
            assert cosine(logits[0], want) >= 0.9999, step
    finally:
        ck.ckb200_model_free(handle)


def test_short_prompts_and_later_chunks_fall_back_to_decode_steps(ck, orc):
    so.bind_model_api(ck)
    cfg = PF_QWEN
    cpu = so.CpuModel(cfg, seed=43)
    prompt = np.arange(3, 3 + 9, dtype=np.int32)
    want = None
    for i, tok in enumerate(prompt):
        want = cpu.decode(orc, int(tok), i)
    handle = ck.ckb200_model_create(C.byref(so.make_cfg(cfg, batch=1)))
    assert handle
    try:
        so.upload_whole_model(ck, handle, so.CpuModel(cfg, seed=43), 1)
        logits = np.zeros((1, cfg["vocab_size"]), np.float32)
        assert ck.ckb200_model_prefill(handle, cases.vptr(prompt), len(prompt), cases.vptr(logits)) == 0     # 9 tokens: decode steps
        assert ck.ckb200_model_get_pos(handle) == len(prompt)
        assert cosine(logits[0], want) >= 0.9999
        more = np.arange(100, 120, dtype=np.int32)                                                           # position 9: decode steps too
        for i, tok in enumerate(more):
            want = cpu.decode(orc, int(tok), len(prompt) + i)
        assert ck.ckb200_model_prefill(handle, cases.vptr(more), len(more), cases.vptr(logits)) == 0
        assert ck.ckb200_model_get_pos(handle) == len(prompt) + len(more)
        assert cosine(logits[0], want) >= 0.9999
        too_many = np.zeros(cfg["max_seq_len"], dtype=np.int32)
        assert ck.ckb200_model_prefill(handle, cases.vptr(too_many), len(too_many), None) == 6                # CKB_ERR_LIMIT
        ck.ckb200_clear_error()
    finally:
        ck.ckb200_model_free(handle)
        ck.ckb200_clear_error()
