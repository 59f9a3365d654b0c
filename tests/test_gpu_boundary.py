"""GPU parity of the later reference-named entry points: fp32-activation GEMMs, the contract forms that quantise inside,
the general RoPE table and the pairwise rotation, add_inplace_f32 / logits_copy_to_position and the flat ck_test_* API -
against the committed reference outputs, the CPU oracle and (when built) the reference's own wrappers."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases
from test_oracle import parity_api_cases

pytestmark = pytest.mark.gpu
synth = cases.synth


def close(a, b, tol):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)))) <= tol * max(1e-30, float(np.max(np.abs(b))))


def test_boundary_cases_against_reference_outputs(ck, golden_boundary, orc):
    got = cases.boundary_outputs(ck, "")
    want_orc = cases.boundary_outputs(orc, "oracle_")
    for name in golden_boundary.files:
        want = golden_boundary[name]
        if name in ("add_inplace", "logits_copy"):
            assert np.array_equal(got[name], want), name                        # one rounding per element: identical bits
        elif name.startswith("rope_pair"):
            assert float(np.max(np.abs(got[name] - want))) <= 2e-5, name        # rotated with this library's own table (below)
        elif name.startswith("rope_"):
            assert float(np.max(np.abs(got[name] - want))) <= 2e-6, name        # table values in [-1, 1]; libm vs device cos/sin
        elif name.startswith("attn_f16kv_"):
            # same rounding sequence, but a score that differs in the last bit can flip one fp16 rounding of the accumulator (2^-11 relative)
            assert close(got[name], want, 2e-3), name
            assert close(got[name], want_orc[name], 2e-3), name
        else:
            assert close(got[name], want, 1e-5), name
            assert close(got[name], want_orc[name], 1e-5), name


@pytest.mark.parametrize("fmt,m,n,k", [("q4_k", 5, 130, 1024), ("q6_k", 4, 33, 2048), ("q8_0", 7, 50, 896)])
def test_fp32_activation_gemm_both_orientations(ck, orc, fmt, m, n, k):
    w = synth.make_weights(fmt, n, k, seed=n + k)
    a = synth.make_x(k, seed=n, rows=m).reshape(m, k)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt_f32(orc, "oracle_", f"gemm_nt_{fmt}", a, w, bias, m, n, k)
    assert close(cases.gemm_nt_f32(ck, "", f"gemm_nt_{fmt}", a, w, bias, m, n, k), want, 1e-5)
    want_t = cases.gemm_f32(orc, "oracle_", f"gemm_{fmt}", w, a, n, m, k)
    assert close(cases.gemm_f32(ck, "", f"gemm_{fmt}", w, a, n, m, k), want_t, 1e-5)
    if fmt == "q6_k":
        for sym in ("gemm_nt_q6_k_ref", "gemm_nt_q6_k_sse"):
            ref_sym = "gemm_nt_q6_k" if sym.endswith("_ref") else sym
            assert close(cases.gemm_nt_f32(ck, "", sym, a, w, bias, m, n, k), cases.gemm_nt_f32(orc, "oracle_", ref_sym, a, w, bias, m, n, k), 1e-5), sym


@pytest.mark.parametrize("m,n,k", [(1, 64, 896), (5, 33, 4096), (2, 7, 32 * 1030)])
def test_contract_forms_quantise_inside(ck, orc, m, n, k):
    """fp32 in: Q8_0 quantisation (bit-exact) then the integer kernel; rows of more than 1024 blocks take the fp32 GEMV as in the reference."""
    w = synth.make_weights("q8_0", n, k, seed=k + n)
    a = synth.make_x(k, seed=m, rows=m).reshape(m, k)
    bias = np.random.default_rng(k).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt_f32(orc, "oracle_", "gemm_nt_q8_0_q8_0_contract", a, w, bias, m, n, k)
    assert close(cases.gemm_nt_f32(ck, "", "gemm_nt_q8_0_q8_0_contract", a, w, bias, m, n, k), want, 1e-5)
    assert close(cases.gemv_contract(ck, "", w, a[0].copy(), n, k), cases.gemv_contract(orc, "oracle_", w, a[0].copy(), n, k), 1e-5)


@pytest.mark.parametrize("heads,kvh,tokens,hd,ad,rot,pos", [(32, 8, 1, 128, 128, 0, 4095), (14, 2, 17, 64, 64, 64, 3), (8, 8, 5, 80, 96, 40, 11)])
def test_pairwise_rope_bit_exact(ck, orc, heads, kvh, tokens, hd, ad, rot, pos):
    rng = np.random.default_rng(heads + tokens)
    cos, sin = cases.rope_cache_general(orc, "oracle_", pos + tokens, hd, 5.0e5, rot, None, 1.0)
    cos_g, sin_g = cases.rope_cache_general(ck, "", pos + tokens, hd, 5.0e5, rot, None, 1.0)
    assert float(np.max(np.abs(cos - cos_g))) <= 2e-6 and float(np.max(np.abs(sin - sin_g))) <= 2e-6
    q = rng.standard_normal((heads, tokens, ad)).astype(np.float32)
    k = rng.standard_normal((kvh, tokens, ad)).astype(np.float32)
    q2, k2 = q.copy(), k.copy()
    cases.rope_qk_pairwise(ck, "", q, k, cos, sin, pos, hd, rot)
    cases.rope_qk_pairwise(orc, "oracle_", q2, k2, cos, sin, pos, hd, rot)
    assert np.array_equal(q, q2) and np.array_equal(k, k2)


def test_parity_api_wrappers(ck, orc):
    """The flat ck_test_* API through the CUDA library against the same compositions of oracle functions."""
    got = parity_api_cases(ck, orc, "oracle_")
    w4, w6 = synth.make_weights("q4_k", 6, 512, 91), synth.make_weights("q6_k", 6, 512, 92)
    w8, w5 = synth.make_weights("q8_0", 6, 256, 93), synth.make_weights("q5_0", 6, 256, 94)
    x512, x256 = synth.make_x(512, 91), synth.make_x(256, 93)
    xq = cases.quantize_q8_k(orc, "oracle_", x512)
    assert np.array_equal(got["quantize_q8_k"], xq)
    assert np.array_equal(got["dequant_q4_k"], cases.dequant_row(orc, "oracle_", "q4_k", w4, 512))
    assert np.array_equal(got["dequant_q6_k"], cases.dequant_row(orc, "oracle_", "q6_k", w6, 512))
    aq = cases.quantize_q8_k(orc, "oracle_", synth.make_x(512, 95, rows=3), rows=3)
    for fmt, w in (("q4_k", w4), ("q6_k", w6)):
        assert close(got[f"gemv_{fmt}"], cases.gemv(orc, "oracle_", fmt, w, xq, 1, 512), 1e-5), fmt
        assert close(got[f"gemm_{fmt}"], cases.gemm_nt(orc, "oracle_", fmt, aq, w, None, 3, 6, 512), 1e-5), fmt
    xq0 = cases.quantize_q8_0(orc, "oracle_", x256)
    aq0 = cases.quantize_q8_0(orc, "oracle_", synth.make_x(256, 96, rows=2), rows=2)
    for fmt, w in (("q8_0", w8), ("q5_0", w5)):
        want = cases.gemv(orc, "oracle_", fmt, w, xq0, 6, 256)
        assert close(got[f"ck_test_gemv_{fmt}"], want, 1e-5) and close(got[f"ck_test_gemv_{fmt}_q8_0"], want, 1e-5), fmt
        assert close(got[f"vec_dot_{fmt}"], want[:1], 1e-5), fmt
        assert close(got[f"gemm_{fmt}"], cases.gemm_nt(orc, "oracle_", fmt, aq0, w, None, 2, 6, 256), 1e-5), fmt
    rng = np.random.default_rng(91)
    xn = rng.standard_normal((2, 320)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(320)).astype(np.float32)
    assert close(got["rmsnorm"], cases.rmsnorm(orc, "oracle_", xn, g, 320, 1e-5), 1e-5)
    qr, kr = rng.standard_normal((3, 4 * 64)).astype(np.float32), rng.standard_normal((3, 2 * 64)).astype(np.float32)
    cos, sin = cases.rope_cache(orc, "oracle_", 8, 64, 1.0e4)
    qh = np.ascontiguousarray(qr.reshape(3, 4, 64).transpose(1, 0, 2))
    kh = np.ascontiguousarray(kr.reshape(3, 2, 64).transpose(1, 0, 2))
    cases.rope_qk(orc, "oracle_", qh, kh, cos, sin, pos=5, tokens=3)
    assert float(np.max(np.abs(got["rope_q"].reshape(3, 4, 64).transpose(1, 0, 2) - qh))) <= 1e-5
    assert float(np.max(np.abs(got["rope_k"].reshape(3, 2, 64).transpose(1, 0, 2) - kh))) <= 1e-5
    gu = (2 * rng.standard_normal((2, 2 * 96))).astype(np.float32)
    assert close(got["swiglu"], cases.swiglu(orc, "oracle_", gu, 96), 2e-4)
    qi, ki = rng.standard_normal((3, 4 * 64)).astype(np.float32), rng.standard_normal((3, 2 * 64)).astype(np.float32)
    cosg, sing = cases.rope_cache_general(orc, "oracle_", 8, 64, 1.0e4, 64, None, 1.0)
    qh = np.ascontiguousarray(qi.reshape(3, 4, 64).transpose(1, 0, 2))
    kh = np.ascontiguousarray(ki.reshape(3, 2, 64).transpose(1, 0, 2))
    cases.rope_qk_pairwise(orc, "oracle_", qh, kh, cosg, sing, pos=5, hd=64, rotary_dim=64)
    assert float(np.max(np.abs(got["rope_interleaved_q"].reshape(3, 4, 64).transpose(1, 0, 2) - qh))) <= 2e-5
    assert float(np.max(np.abs(got["rope_interleaved_k"].reshape(3, 2, 64).transpose(1, 0, 2) - kh))) <= 2e-5
    w40 = synth.make_weights("q4_0", 4, 128, 97)
    d40 = np.zeros(512, np.float32)
    orc.oracle_dequant_q4_0_row(cases.vptr(w40), cases.fptr(d40), C.c_size_t(512))
    assert np.array_equal(got["dequant_q4_0"], d40)
    aq, ak, av = cases.prefill_attention_inputs(98, 4, 2, 64, 64, 9, 9)
    assert close(got["attention_causal"], cases.attention_prefill(orc, "oracle_", aq, ak, av, 64), 1e-4)


def test_parity_api_wrappers_against_the_references_own(ck, orc, ref_parity, ref):
    a, b = parity_api_cases(ck, orc, "oracle_"), parity_api_cases(ref_parity, ref, "")
    for name in b:
        if name in ("quantize_q8_k", "dequant_q4_k", "dequant_q6_k"):
            assert np.array_equal(a[name], b[name]), name
        else:
            assert close(a[name], b[name], {"swiglu": 2e-4, "attention_causal": 1e-4, "rope_interleaved_q": 3e-5, "rope_interleaved_k": 3e-5}.get(name, 1e-5)), name


def test_bounded_wait_runs_out_and_is_reported(ck):
    """An exchange whose peers never write: the kernel gives up after the (shortened) limit and returns, the next synchronising
    call reports CKB_ERR_DEVICE_WAIT, later calls do not wait while the error stands, and clearing it restores service."""
    import time

    import torch

    dev = torch.device("cuda", 0)
    handle = (C.c_ubyte * 64)()
    ck.ckb200_tp_p2p_shutdown()
    assert ck.ckb200_tp_p2p_create(0, 2, C.c_size_t(4096), handle) == 0
    try:
        assert ck.ckb200_tp_p2p_connect_self() == 0
        ck.ckb200_tune_set(b"wait_limit_ms", 5)
        buf = torch.arange(1024, dtype=torch.float32, device=dev)
        before = buf.clone()
        torch.cuda.synchronize()
        ck.ckb_tp_p2p_allreduce.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        t0 = time.perf_counter()
        assert ck.ckb_tp_p2p_allreduce(C.c_void_p(buf.data_ptr()), 1024, None) == 0
        rc = ck.ckb200_synchronize()
        waited = time.perf_counter() - t0
        assert rc == 5, rc                                   # CKB_ERR_DEVICE_WAIT
        assert ck.ckb200_last_error() == 5
        assert waited < 2.0, waited                          # 5 ms of polling, not the ten-second default
        assert torch.equal(buf, before)                      # a timed-out call leaves the vector unreduced
        ck.ckb200_clear_error()
        # the host-pointer calls fold the same word in: a second timed-out exchange surfaces through the next one of them
        assert ck.ckb_tp_p2p_allreduce(C.c_void_p(buf.data_ptr()), 1024, None) == 0
        x = synth.make_x(256, 1)
        cases.quantize_q8_k(ck, "", x)
        assert ck.ckb200_last_error() == 5
        ck.ckb200_clear_error()
        assert ck.ckb200_synchronize() == 0                  # the device word was cleared when it was read
    finally:
        ck.ckb200_tune_set(b"wait_limit_ms", 10000)
        ck.ckb200_tp_p2p_shutdown()
        ck.ckb200_clear_error()


@pytest.mark.parametrize("heads,kv_heads,d,tokens,cap", [(32, 8, 128, 1500, 2048), (14, 2, 64, 1024, 1024), (6, 3, 64, 33, 40), (2, 1, 128, 4096, 4096),
                                                        (4, 2, 256, 300, 320), (3, 1, 80, 77, 77)])   # wider than 128: every thread walks; 80: odd row width
def test_f16kv_decode_attention_walks_the_keys_in_order(ck, orc, heads, kv_heads, d, tokens, cap):
    """attention_forward_decode_head_major_gqa_flash_f16kv: the accumulator is rounded to fp16 after every key, so only a kernel that keeps the
    reference's key order stays within fp16 rounding flips of it (a split-K kernel drifts by about 1 % at these lengths)."""
    q, kc, vc = cases.attention_inputs(tokens + heads, heads, kv_heads, d, tokens, cap)
    want = cases.attention_decode_f16kv(orc, "oracle_", q, kc, vc, tokens)
    got = cases.attention_decode_f16kv(ck, "", q, kc, vc, tokens)
    assert close(got, want, 2e-3)
    exact = cases.attention_decode(orc, "oracle_", q, kc, vc, tokens)
    assert not close(want, exact, 1e-4) or tokens < 64          # the fp16 form is a different function, not a relabelled fp32 kernel


@pytest.mark.parametrize("v_scale,tol", [(2.0e-5, 2e-2), (3.0e-8, 0.3), (8.0e3, 2e-3)])
def test_f16kv_decode_attention_outside_the_normal_fp16_range(ck, orc, v_scale, tol):
    """Values so small that the accumulator lives among fp16's subnormals (steps of 2^-24: the looser bounds) or vanishes, and so large
    that about 8 % of the outputs overflow to infinity: the kernel's arithmetic shortcut for the rounding does not hold there and it has to
    notice.  An accumulator that passes within a rounding step of the overflow threshold may land on either side (the scores differ in
    the last place), so a few outputs may disagree on finiteness; the rest must agree as closely as in the normal range."""
    heads, kv_heads, d, tokens = 8, 2, 128, 700
    q, kc, vc = cases.attention_inputs(5, heads, kv_heads, d, tokens, tokens)
    vc = (vc * np.float32(v_scale)).astype(np.float32)
    want = cases.attention_decode_f16kv(orc, "oracle_", q, kc, vc, tokens)
    got = cases.attention_decode_f16kv(ck, "", q, kc, vc, tokens)
    assert not np.isnan(want).any() and not np.isnan(got).any()
    both = np.isfinite(got) & np.isfinite(want)
    assert float(np.mean(np.isfinite(got) != np.isfinite(want))) <= 0.01
    if v_scale > 1:
        assert 0.02 < float(np.mean(np.isinf(got))) < 0.2
        assert np.array_equal(got[np.isinf(got) & np.isinf(want)], want[np.isinf(got) & np.isinf(want)])       # the sign of the infinity
    assert close(np.where(both, got, 0), np.where(both, want, 0), tol)


@pytest.mark.parametrize("fmt,m,k", [("q4_k", 301, 1024), ("q8_0", 77, 160), ("q6_k", 64, 512)])
def test_host_call_with_pinned_buffers_matches_pageable(ck, orc, fmt, m, k):
    """A result row in memory from ckb200_host_alloc is written across the bus by a kernel in the call's stream instead of the copy
    engine (at offset 4 it is not 16-byte aligned: the byte path of that kernel): same GEMV kernels, so the same bits as with ordinary
    host buffers, and nothing written around the row."""
    ck.ckb200_host_alloc.restype = C.c_void_p
    w = cases.synth.make_weights(fmt, m, k, seed=31)
    xq = cases.quantize_act(orc, "oracle_", fmt, cases.synth.make_x(k, seed=32))
    want = cases.gemv(ck, "", fmt, w, xq, m, k)
    assert close(want, cases.gemv(orc, "oracle_", fmt, w, xq, m, k), 1e-5)
    hx = ck.ckb200_host_alloc(C.c_size_t(xq.nbytes + 64))
    hy = ck.ckb200_host_alloc(C.c_size_t(4 * m + 64))
    assert hx and hy
    try:
        for x_off, y_off in ((0, 0), (4, 4)):
            C.memmove(hx + x_off, xq.ctypes.data, xq.nbytes)
            C.memset(hy, 0xFF, 4 * m + 64)
            cases.fn(ck, "", cases.GEMV_SYMBOL[fmt])(C.c_void_p(hy + y_off), cases.vptr(w), C.c_void_p(hx + x_off), C.c_int(m), C.c_int(k))
            got = np.frombuffer((C.c_char * (4 * m + 64)).from_address(hy), dtype=np.uint8).copy()
            assert np.array_equal(got[y_off:y_off + 4 * m].view(np.float32), want)
            assert (got[:y_off] == 0xFF).all() and (got[y_off + 4 * m:] == 0xFF).all()          # nothing written around the row
    finally:
        ck.ckb200_host_free(C.c_void_p(hx))
        ck.ckb200_host_free(C.c_void_p(hy))


def test_f16kv_prefill_attention(ck, orc):
    q, k, v = cases.prefill_attention_inputs(91, 8, 2, 128, 128, 200, 256)
    want = cases.attention_prefill_f16kv(orc, "oracle_", q, k, v, 128)
    got = cases.attention_prefill_f16kv(ck, "", q, k, v, 128)
    assert close(got, want, 2e-3)
