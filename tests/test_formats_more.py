"""Q5_K, Q5_1 x Q8_1 and the 32-element formats Q4_0 / Q4_1 / Q5_1: the oracle against the reference build (CPU), the CUDA library against
the oracle (GPU).  Cases in tests/legacy_cases.py."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases
import legacy_cases as lc

synth = cases.synth


def close(a, b, tol):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)))) <= tol * max(1e-30, float(np.max(np.abs(b))))


def test_oracle_equals_the_reference_build(orc, ref):
    """Every restated function, bit for bit: integer block sums and the reference's fp32 operation order."""
    want, got = lc.outputs(ref, "", orc), lc.outputs(orc, "oracle_", orc)
    assert sorted(want) == sorted(got)
    for name in want:
        assert np.isfinite(want[name]).all(), name
        assert np.array_equal(want[name], got[name]), name


def test_q5_k_long_rows_take_the_fp32_path(orc, ref):
    """More than 128 superblocks per row: gemv_q5_k reads the block in its fall-back order (a different function of the same bytes)."""
    n, k = 3, 256 * 130
    w = synth.make_weights("q5_k", n, k, seed=5)
    x = synth.make_x(k, seed=5)
    a, b = lc._gemv_f32(ref, "", "gemv_q5_k", w, x, n, k), lc._gemv_f32(orc, "oracle_", "gemv_q5_k", w, x, n, k)
    assert np.array_equal(a, b)


@pytest.mark.gpu
def test_cuda_library_matches_the_oracle(ck, orc):
    want, got = lc.outputs(orc, "oracle_", orc), lc.outputs(ck, "", orc)
    for name in want:
        if name.startswith(("gemv_q5_k_q8_k", "gemm_nt_q5_k_q8_k", "gemv_q5_1_q8_1", "gemm_nt_q5_1_q8_1", "gemv_q5_k", "gemm_nt_q5_k", "dequant_")):
            assert np.array_equal(got[name], want[name]), name          # integer sums, fp32 steps in block order; dequantisers one chain per element
        else:
            assert close(got[name], want[name], 1e-5), name             # fp32-activation GEMVs: lanes sum in another order


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 130, 2048), (5, 33, 768), (2, 300, 256 * 130)])
def test_q5_k_shapes(ck, orc, m, n, k):
    w = synth.make_weights("q5_k", n, k, seed=n + k)
    a = synth.make_x(k, seed=m, rows=m).reshape(m, k)
    bias = np.random.default_rng(k).standard_normal(n).astype(np.float32)
    want = lc._gemm_nt_f32(orc, "oracle_", "gemm_nt_q5_k", a, w, bias, m, n, k)
    got = lc._gemm_nt_f32(ck, "", "gemm_nt_q5_k", a, w, bias, m, n, k)
    if k // 256 <= 128:
        assert np.array_equal(got, want)            # quantised path: bit-exact (the device Q8_K quantiser is bit-exact as well)
    else:
        assert close(got, want, 1e-5)               # fp32 fall-back


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 257, 4096), (7, 40, 896), (3, 9, 32 * 256)])
def test_q5_1_q8_1_shapes(ck, orc, m, n, k):
    w = synth.make_weights("q5_1", n, k, seed=n + k)
    a = synth.make_x(k, seed=m, rows=m).reshape(m, k)
    bias = np.random.default_rng(k).standard_normal(n).astype(np.float32)
    aq = lc.quantize_q8_1(orc, a, k)
    dev = np.zeros_like(aq)
    ck.ckb200_dev_quantize_q8_1.argtypes = [C.c_void_p] * 2 + [C.c_int] * 2 + [C.c_void_p]
    want = lc._gemm_nt_f32(orc, "oracle_", "gemm_nt_q5_1_q8_1", a, w, bias, m, n, k)
    assert np.array_equal(lc._gemm_nt_f32(ck, "", "gemm_nt_q5_1_q8_1", a, w, bias, m, n, k), want)
    assert np.array_equal(lc._gemm_nt_q(ck, "", "gemm_nt_q5_1_q8_1_ref", aq, w, bias, m, n, k), lc._gemm_nt_q(orc, "oracle_", "gemm_nt_q5_1_q8_1_ref", aq, w, bias, m, n, k))
    del dev


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["q4_0", "q4_1", "q5_1"])
def test_block32_fp32_forms(ck, orc, fmt):
    m, n, k = 4, 70, 1024
    w = synth.make_weights(fmt, n, k, seed=17)
    a = synth.make_x(k, seed=17, rows=m).reshape(m, k)
    bias = np.random.default_rng(17).standard_normal(n).astype(np.float32)
    want_rows = np.stack([lc._gemv_f32(orc, "oracle_", f"gemv_{fmt}_ref", w, a[t], n, k) for t in range(m)])
    assert close(lc._gemm_nt_f32(ck, "", f"gemm_nt_{fmt}", a, w, bias, m, n, k), want_rows + bias, 1e-5)
    y = np.full((m, n), np.nan, np.float32)
    cases.fn(ck, "", f"gemm_{fmt}")(cases.fptr(y), cases.vptr(w), cases.fptr(a), C.c_int(n), C.c_int(m), C.c_int(k))
    assert close(y, want_rows, 1e-5)
    dot = cases.fn(ck, "", f"dot_{fmt}", restype=C.c_float)(cases.vptr(w), cases.fptr(a[0]), C.c_int(k))
    assert abs(dot - want_rows[0, 0]) <= 1e-5 * float(np.max(np.abs(want_rows)))
    assert close(lc._gemv_f32(ck, "", f"gemv_{fmt}", w, a[1], n, k), want_rows[1], 1e-5)
