"""Seeded cases for the further weight formats (Q5_K, Q4_0, Q4_1, Q5_1 with Q8_1 activations): one dict of outputs per library, so the same
cases run through the reference build, the oracle and the CUDA library."""
from __future__ import annotations

import ctypes as C

import numpy as np

import cases

synth = cases.synth
fn, fptr, vptr = cases.fn, cases.fptr, cases.vptr


def _gemv_f32(lib, prefix, name, w, x, m, k):
    y = np.full(m, np.nan, np.float32)
    fn(lib, prefix, name)(fptr(y), vptr(w), fptr(x), C.c_int(m), C.c_int(k))
    return y


def _gemm_nt_f32(lib, prefix, name, a, w, bias, m, n, k):
    c = np.full((m, n), np.nan, np.float32)
    fn(lib, prefix, name)(fptr(a), vptr(w), fptr(bias) if bias is not None else None, fptr(c), C.c_int(m), C.c_int(n), C.c_int(k))
    return c


def _gemv_q(lib, prefix, name, w, xq, m, k):
    y = np.full(m, np.nan, np.float32)
    fn(lib, prefix, name)(fptr(y), vptr(w), vptr(xq), C.c_int(m), C.c_int(k))
    return y


def _gemm_nt_q(lib, prefix, name, aq, w, bias, m, n, k):
    c = np.full((m, n), np.nan, np.float32)
    fn(lib, prefix, name)(vptr(aq), vptr(w), fptr(bias) if bias is not None else None, fptr(c), C.c_int(m), C.c_int(n), C.c_int(k))
    return c


def _dequant(lib, prefix, name, w, n):
    out = np.full(n, np.nan, np.float32)
    fn(lib, prefix, name)(vptr(w), fptr(out), C.c_size_t(n))
    return out


def quantize_q8_1(orc, x, k):
    """Q8_1 rows from the oracle (the reference keeps its Q8_1 quantiser static)."""
    rows = x.size // k
    out = np.zeros(rows * (k // 32) * 36, np.uint8)
    for r in range(rows):
        orc.oracle_quantize_row_q8_1(fptr(x.reshape(rows, k)[r]), C.c_void_p(out.ctypes.data + r * (k // 32) * 36), C.c_int(k))
    return out


def outputs(lib, prefix: str, orc) -> dict[str, np.ndarray]:
    """prefix "" = the reference's symbols (reference build or CUDA library), "oracle_" = the restatement."""
    out = {}
    # Q5_K x Q8_K and its fp32-in adapters
    m, n, k = 3, 37, 1024
    w = synth.make_weights("q5_k", n, k, seed=101)
    a = synth.make_x(k, seed=101, rows=m).reshape(m, k)
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    bias = np.random.default_rng(101).standard_normal(n).astype(np.float32)
    out["gemv_q5_k_q8_k"] = _gemv_q(lib, prefix, "gemv_q5_k_q8_k", w, aq[: (k // 256) * 292], n, k)
    out["gemm_nt_q5_k_q8_k"] = _gemm_nt_q(lib, prefix, "gemm_nt_q5_k_q8_k", aq, w, bias, m, n, k)
    out["gemv_q5_k"] = _gemv_f32(lib, prefix, "gemv_q5_k", w, a[0], n, k)
    out["gemm_nt_q5_k"] = _gemm_nt_f32(lib, prefix, "gemm_nt_q5_k", a, w, bias, m, n, k)
    # Q5_1 x Q8_1
    m, n, k = 2, 29, 896
    w = synth.make_weights("q5_1", n, k, seed=102)
    a = synth.make_x(k, seed=102, rows=m).reshape(m, k)
    aq = quantize_q8_1(orc, a, k)
    out["gemv_q5_1_q8_1_ref"] = _gemv_q(lib, prefix, "gemv_q5_1_q8_1_ref", w, aq[: (k // 32) * 36], n, k)
    out["gemm_nt_q5_1_q8_1_ref"] = _gemm_nt_q(lib, prefix, "gemm_nt_q5_1_q8_1_ref", aq, w, bias[:n], m, n, k)
    out["gemv_q5_1_q8_1"] = _gemv_f32(lib, prefix, "gemv_q5_1_q8_1", w, a[0], n, k)
    out["gemm_nt_q5_1_q8_1"] = _gemm_nt_f32(lib, prefix, "gemm_nt_q5_1_q8_1", a, w, bias[:n], m, n, k)
    # 32-element formats with fp32 activations: row dequantisers and the scalar GEMVs
    for fmt, seed in (("q4_0", 103), ("q4_1", 104), ("q5_1", 105)):
        n, k = 19, 480
        w = synth.make_weights(fmt, n, k, seed=seed)
        x = synth.make_x(k, seed=seed)
        out[f"dequant_{fmt}_row"] = _dequant(lib, prefix, f"dequant_{fmt}_row", w, n * k)
        out[f"gemv_{fmt}_ref"] = _gemv_f32(lib, prefix, f"gemv_{fmt}_ref", w, x, n, k)
    return out


# what the oracle reproduces bit for bit: integer block sums combined in the reference's fp32 order, and one-rounding-chain dequantisers
BIT_EXACT = ("gemv_q5_k_q8_k", "gemm_nt_q5_k_q8_k", "gemv_q5_1_q8_1_ref", "gemm_nt_q5_1_q8_1_ref", "gemv_q5_1_q8_1", "gemm_nt_q5_1_q8_1", "dequant_",
             "gemv_q4_0_ref", "gemv_q4_1_ref", "gemv_q5_1_ref")
