"""The CPU oracle is pinned against the reference: (1) against committed golden vectors that
tests/golden/make_golden.py produced from the reference's own kernels, (2) live against
oracle/_ref when it has been built here, on more and larger seeded cases."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases

synth = cases.synth


def _close(a, b, rtol_scale):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)))) <= rtol_scale * max(1e-30, float(np.max(np.abs(a))))


@pytest.fixture(scope="module")
def oracle_outputs(orc):
    return cases.golden_outputs(orc, "oracle_")


def test_golden_file_is_complete(golden, oracle_outputs):
    missing = [k for k in oracle_outputs if k not in golden.files and k != "residual"]
    assert not missing, missing
    assert len(golden.files) >= 40


def test_oracle_bit_exact_stages(golden, oracle_outputs):
    """Integer / byte stages and every function whose fp32 order the oracle keeps: identical bytes."""
    checked = 0
    for name in golden.files:
        if name in oracle_outputs and name.startswith(cases.BIT_EXACT):
            assert np.array_equal(golden[name], oracle_outputs[name]), name
            checked += 1
    assert checked >= 25


def test_oracle_float_stages_within_tolerance(golden, oracle_outputs):
    """Where the reference's dispatched path is vectorised (different fp32 order, FMA, fast exp)
    the oracle agrees to well inside the 1e-3 contract."""
    for name in golden.files:
        if name not in oracle_outputs or name.startswith(cases.BIT_EXACT):
            continue
        tol = 2e-4 if name == "swiglu" else 1e-5     # the reference's AVX-512 SwiGLU uses a polynomial exp
        assert _close(golden[name], oracle_outputs[name], tol), name


def test_dispatched_reference_paths_agree_with_scalar(golden):
    """The reference's own ISA paths differ from its scalar path only by fp32 rounding."""
    for name in golden.files:
        if name.startswith("gemv_dispatch_"):
            assert _close(golden[name.replace("dispatch", "ref")], golden[name], 1e-5), name


def test_q8k_edge_cases_decoded(golden):
    """Spot-check the meaning of the edge-case vectors, not only their bytes."""
    blocks = golden["q8k_edge"].reshape(5, 292)
    d = blocks[:, :4].copy().view(np.float32).reshape(5)
    qs = blocks[:, 4:260].copy().view(np.int8)
    bsums = blocks[:, 260:].copy().view(np.int16)
    assert d[0] == 0 and not qs[0].any() and not bsums[0].any()          # zero block
    assert qs[1, 10] == -127 and qs[1, 200] == 127 and d[1] < 0          # +3 first: scale sign from it
    assert qs[2, 7] == -127 and qs[2, 8] == 127 and d[2] > 0             # -5 first
    assert qs[3, 0] == -127 and qs[3, 1] == 0 and qs[3, 2] == -2         # -0.5 -> 0, -1.5 -> -2 (ties to even)
    assert np.array_equal(bsums, qs.reshape(5, 16, 16).sum(axis=2).astype(np.int16))


def test_fp16_conversions_all_values(orc):
    """Every half value round-trips; float->half agrees with numpy's IEEE conversion on a dense sample."""
    orc.oracle_fp16_to_fp32.restype = C.c_float
    orc.oracle_fp32_to_fp16.restype = C.c_uint16
    h = np.arange(65536, dtype=np.uint16)
    f = np.array([orc.oracle_fp16_to_fp32(C.c_uint16(int(v))) for v in h[::7]], dtype=np.float32)
    expect = h[::7].view(np.float16).astype(np.float32)
    ok = (f == expect) | (np.isnan(f) & np.isnan(expect))
    assert ok.all()
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -25, 2.0 ** -24, 6.1e-5], np.float32)])
    got = np.array([orc.oracle_fp32_to_fp16(C.c_float(float(v))) for v in xs], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_subblock_sums_recompose_gemv(orc):
    """The exported int32 sub-block sums are the integer stage of the GEMV: recombining them with the
    unpacked scales in float64 reproduces the oracle's fp32 output to rounding."""
    m, k = 6, 1024
    for fmt in ("q4_k", "q6_k"):
        w = synth.make_weights(fmt, m, k, seed=77)
        xq = cases.quantize_q8_k(orc, "oracle_", synth.make_x(k, seed=77))
        y = cases.gemv(orc, "oracle_", fmt, w, xq, m, k)
        nb = k // 256
        xb = xq.reshape(nb, 292)
        xd = xb[:, :4].copy().view(np.float32).reshape(nb).astype(np.float64)
        bs = xb[:, 260:].copy().view(np.int16).reshape(nb, 16).astype(np.int64)
        for r in range(m):
            row = w.reshape(m, -1)[r]
            if fmt == "q4_k":
                sums = np.zeros(nb * 8, dtype=np.int32)
                orc.oracle_q4_k_q8_k_subblock_sums(cases.vptr(row), cases.vptr(xq), C.c_int(k), sums.ctypes.data_as(cases.c_int32_p))
                blk = row.reshape(nb, 144)
                acc = 0.0
                for b in range(nb):
                    d = float(blk[b, 0:2].copy().view(np.float16)[0]) * xd[b]
                    dm = float(blk[b, 2:4].copy().view(np.float16)[0]) * xd[b]
                    sc = np.zeros(8, np.uint8)
                    mn = np.zeros(8, np.uint8)
                    s12 = np.ascontiguousarray(blk[b, 4:16])
                    orc.oracle_unpack_q4_k_scales(cases.vptr(s12), cases.vptr(sc), cases.vptr(mn))
                    for j in range(8):
                        acc += d * sc[j] * int(sums[8 * b + j]) - dm * mn[j] * int(bs[b, 2 * j] + bs[b, 2 * j + 1])
            else:
                sums = np.zeros(nb * 16, dtype=np.int32)
                orc.oracle_q6_k_q8_k_subblock_sums(cases.vptr(row), cases.vptr(xq), C.c_int(k), sums.ctypes.data_as(cases.c_int32_p))
                blk = row.reshape(nb, 210)
                acc = 0.0
                for b in range(nb):
                    d = float(blk[b, 208:210].copy().view(np.float16)[0]) * xd[b]
                    sc = blk[b, 192:208].copy().view(np.int8).astype(np.int64)
                    acc += d * float((sc * sums[16 * b:16 * b + 16].astype(np.int64)).sum())
            assert abs(acc - float(y[r])) <= 2e-5 * max(1.0, abs(acc)), (fmt, r, acc, y[r])


# ---------------------------------------------------------------- live against the reference

LIVE_GEMV = [("q4_k", 37, 4096, None), ("q4_k", 64, 1024, 896), ("q6_k", 33, 4096, None), ("q6_k", 21, 4864, None),
             ("q8_0", 50, 896, None), ("q8_0", 19, 4864, None)]


@pytest.mark.parametrize("fmt,m,k,kv", LIVE_GEMV)
def test_oracle_vs_reference_gemv(ref, orc, fmt, m, k, kv):
    w = synth.make_weights(fmt, m, k, seed=m)
    x = synth.make_x(k, seed=m, k_valid=kv)
    xq_r = cases.quantize_act(ref, "", fmt, x)
    xq_o = cases.quantize_act(orc, "oracle_", fmt, x)
    assert np.array_equal(xq_r, xq_o)
    scalar = {"q4_k": "gemv_q4_k_q8_k_ref", "q6_k": "gemv_q6_k_q8_k_ref", "q8_0": None}[fmt]
    y_o = cases.gemv(orc, "oracle_", fmt, w, xq_o, m, k)
    if scalar:
        assert np.array_equal(cases.gemv(ref, "", fmt, w, xq_r, m, k, scalar), y_o)
    y_d = cases.gemv(ref, "", fmt, w, xq_r, m, k)          # the path a user of the reference gets
    assert _close(y_d, y_o, 1e-5)


def test_oracle_vs_reference_quantiser_many_rows(ref, orc):
    x = synth.make_x(4864, seed=9, rows=16) * np.float32(3.7)
    assert np.array_equal(cases.quantize_q8_k(ref, "", x, rows=16), cases.quantize_q8_k(orc, "oracle_", x, rows=16))
    x = synth.make_x(896, seed=10, rows=16) * np.float32(0.01)
    assert np.array_equal(cases.quantize_q8_0(ref, "", x, rows=16), cases.quantize_q8_0(orc, "oracle_", x, rows=16))


@pytest.mark.parametrize("heads,kvh,d,tokens,cap", [(14, 2, 64, 1025, 1100), (16, 2, 128, 333, 512), (8, 4, 64, 64, 64)])
def test_oracle_vs_reference_attention(ref, orc, heads, kvh, d, tokens, cap):
    q, kc, vc = cases.attention_inputs(tokens, heads, kvh, d, tokens, cap)
    a = cases.attention_decode(ref, "", q, kc, vc, tokens)
    b = cases.attention_decode(orc, "oracle_", q, kc, vc, tokens)
    assert float(np.max(np.abs(a - b))) < 1e-5          # the reference's own decode-vs-full tolerance


@pytest.mark.parametrize("heads,kvh,ad,hd,tokens,stride,causal", [(8, 4, 64, 64, 37, 37, True), (14, 2, 64, 64, 70, 96, True), (4, 4, 64, 40, 9, 16, True),
                                                                (8, 2, 128, 128, 33, 40, False)])
def test_oracle_vs_reference_prefill_attention(ref, orc, heads, kvh, ad, hd, tokens, stride, causal):
    """The restated per-query online softmax against the reference's own build (its SIMD path sums in another order)."""
    q, k, v = cases.prefill_attention_inputs(tokens, heads, kvh, ad, hd, tokens, stride)
    a = cases.attention_prefill(ref, "", q, k, v, hd, causal)
    b = cases.attention_prefill(orc, "oracle_", q, k, v, hd, causal)
    assert float(np.max(np.abs(a - b))) < 1e-5
    assert np.all(b[:, :, hd:] == 0)


@pytest.mark.parametrize("heads,kvh,d,tokens,cap", [(14, 2, 64, 300, 320), (16, 2, 128, 333, 512), (8, 4, 64, 5000, 5000)])
def test_oracle_vs_reference_f16_kv_cache(ref, orc, heads, kvh, d, tokens, cap):
    """fp16 cache: the store is bit-exact (round to nearest even), decode attention agrees within the reference's own
    tolerance between its paths (the last case is large enough for the reference's two-pass branch)."""
    rng = np.random.default_rng(tokens)
    kc_r = np.zeros((kvh, cap, d), np.uint16); vc_r = np.zeros_like(kc_r)
    kc_o = np.zeros_like(kc_r); vc_o = np.zeros_like(kc_r)
    for pos in (0, 1, cap - 1):
        k = (rng.standard_normal((kvh, d)) * rng.choice([1e-6, 1.0, 300.0], size=(kvh, d))).astype(np.float32)
        v = rng.standard_normal((kvh, d)).astype(np.float32)
        cases.kv_cache_store_f16(ref, "", kc_r, vc_r, k, v, pos)
        cases.kv_cache_store_f16(orc, "oracle_", kc_o, vc_o, k, v, pos)
    assert np.array_equal(kc_r, kc_o) and np.array_equal(vc_r, vc_o)
    q, kc, vc = cases.attention_inputs(tokens, heads, kvh, d, tokens, cap)
    kc16, vc16 = kc.astype(np.float16).view(np.uint16), vc.astype(np.float16).view(np.uint16)
    a = cases.attention_decode_f16cache(ref, "", q, kc16, vc16, tokens)
    b = cases.attention_decode_f16cache(orc, "oracle_", q, kc16, vc16, tokens)
    assert float(np.max(np.abs(a - b))) < 1e-5


@pytest.mark.parametrize("window", [0, 1, 7, 32, 1000])
def test_oracle_vs_reference_sliding_window(ref, orc, window):
    """Sliding-window prefill and decode attention against the reference build (a window of 0 means no limit)."""
    q, k, v = cases.prefill_attention_inputs(window + 3, 8, 4, 64, 64, 70, 80)
    a = cases.attention_prefill_sliding(ref, "", q, k, v, 64, window)
    b = cases.attention_prefill_sliding(orc, "oracle_", q, k, v, 64, window)
    assert float(np.max(np.abs(a - b))) < 1e-5
    qd, kc, vc = cases.attention_inputs(window + 5, 14, 2, 64, 333, 400)
    a = cases.attention_decode_sliding(ref, "", qd, kc, vc, 333, window)
    b = cases.attention_decode_sliding(orc, "oracle_", qd, kc, vc, 333, window)
    assert float(np.max(np.abs(a - b))) < 1e-5


@pytest.mark.parametrize("m,k", [(3, 32), (5, 896), (7, 4096), (64, 4864)])
def test_oracle_vs_reference_q5_0(ref, orc, m, k):
    """Q5_0 x Q8_0: the scalar restatement against the reference's dispatched GEMV (SIMD paths sum the same exact int32
    block sums; fp32 order may differ) and bit for bit against its scalar vec_dot."""
    w = synth.make_weights("q5_0", m, k, seed=m)
    xq = cases.quantize_q8_0(ref, "", synth.make_x(k, seed=m))
    a = cases.gemv(ref, "", "q5_0", w, xq, m, k)
    b = cases.gemv(orc, "oracle_", "q5_0", w, xq, m, k)
    assert _close(a, b, 1e-5)
    s_ref, s_orc = np.zeros(1, np.float32), np.zeros(1, np.float32)
    ref.vec_dot_q5_0_q8_0_ref(C.c_int(k), cases.fptr(s_ref), cases.vptr(w), cases.vptr(xq))
    orc.oracle_vec_dot_q5_0_q8_0(C.c_int(k), cases.fptr(s_orc), cases.vptr(w), cases.vptr(xq))
    assert s_ref[0] == s_orc[0]


def test_oracle_vs_reference_q5_0_dequant_and_fp32_gemv(ref, orc):
    m, k = 9, 896
    w = synth.make_weights("q5_0", m, k, seed=11)
    assert np.array_equal(cases.dequant_row(ref, "", "q5_0", w, m * k), cases.dequant_row(orc, "oracle_", "q5_0", w, m * k))
    x = synth.make_x(k, seed=12)
    a = cases.gemv_f32(ref, "", "q5_0", w, x, m, k, "gemv_q5_0_ref")
    b = cases.gemv_f32(orc, "oracle_", "q5_0", w, x, m, k, "gemv_q5_0")
    assert np.array_equal(a, b)


# ---------------------------------------------------------------- later entry points: fp32-activation GEMMs, contract forms, pairwise RoPE, copies

def test_boundary_oracle_against_golden(golden_boundary, orc):
    got = cases.boundary_outputs(orc, "oracle_")
    assert sorted(got) == sorted(golden_boundary.files)
    for name in golden_boundary.files:
        if name.startswith(cases.BOUNDARY_BIT_EXACT):
            assert np.array_equal(golden_boundary[name], got[name]), name
        else:
            # the reference dispatches these to vector code (another fp32 order); the rope tables go through libm's long double
            assert _close(golden_boundary[name], got[name], 2e-6 if name.startswith("rope_") else 1e-5), name


def test_boundary_oracle_vs_reference_live(ref, orc):
    a, b = cases.boundary_outputs(ref, ""), cases.boundary_outputs(orc, "oracle_")
    for name in a:
        if name.startswith(cases.BOUNDARY_BIT_EXACT):
            assert np.array_equal(a[name], b[name]), name
        else:
            assert _close(a[name], b[name], 1e-5), name


def test_contract_long_rows_take_the_fp32_path(ref, orc):
    """More than 1024 blocks per row: the reference's contract GEMV falls back to gemv_q8_0; so does the oracle."""
    m, k = 3, 32 * 1030
    w = synth.make_weights("q8_0", m, k, 81)
    x = synth.make_x(k, 81)
    assert _close(cases.gemv_contract(ref, "", w, x, m, k), cases.gemv_contract(orc, "oracle_", w, x, m, k), 1e-5)


def parity_api_cases(lib, quant_lib, quant_prefix):
    """Drives the flat ck_test_* API of `lib` (the reference's wrappers or the CUDA library's)."""
    out = {}
    rng = np.random.default_rng(91)
    w4, w6 = synth.make_weights("q4_k", 6, 512, 91), synth.make_weights("q6_k", 6, 512, 92)
    w8, w5 = synth.make_weights("q8_0", 6, 256, 93), synth.make_weights("q5_0", 6, 256, 94)
    x512, x256 = synth.make_x(512, 91), synth.make_x(256, 93)
    for name, w in (("q4_k", w4), ("q6_k", w6)):
        d = np.zeros(512, np.float32)
        getattr(lib, f"ck_test_dequant_{name}")(cases.vptr(w), cases.fptr(d), 512)
        out[f"dequant_{name}"] = d
        y = np.zeros(1, np.float32)
        getattr(lib, f"ck_test_gemv_{name}")(cases.vptr(w), cases.fptr(x512), cases.fptr(y), 512)
        out[f"gemv_{name}"] = y
        a = synth.make_x(512, 95, rows=3)
        c = np.zeros((3, 6), np.float32)
        getattr(lib, f"ck_test_gemm_{name}")(cases.vptr(w), cases.fptr(a), cases.fptr(c), 6, 512, 3)
        out[f"gemm_{name}"] = c
    q = np.zeros(2 * 292, np.uint8)
    lib.ck_test_quantize_q8_k(cases.fptr(x512), cases.vptr(q), 512)
    out["quantize_q8_k"] = q
    for name, w in (("q8_0", w8), ("q5_0", w5)):
        for sym in (f"ck_test_gemv_{name}", f"ck_test_gemv_{name}_q8_0"):
            y = np.zeros(6, np.float32)
            getattr(lib, sym)(cases.vptr(w), cases.fptr(x256), cases.fptr(y), 6, 256)
            out[sym] = y
        xq = cases.quantize_q8_0(quant_lib, quant_prefix, x256)
        y = np.zeros(1, np.float32)
        getattr(lib, f"ck_test_vec_dot_{name}_q8_0")(cases.vptr(w), cases.vptr(xq), cases.fptr(y), 256)
        out[f"vec_dot_{name}"] = y
        a = synth.make_x(256, 96, rows=2)
        c = np.zeros((2, 6), np.float32)
        getattr(lib, f"ck_test_gemm_{name}")(cases.vptr(w), cases.fptr(a), cases.fptr(c), 6, 256, 2)
        out[f"gemm_{name}"] = c
    xn = rng.standard_normal((2, 320)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(320)).astype(np.float32)
    yn = np.zeros_like(xn)
    lib.ck_test_rmsnorm(cases.fptr(xn), cases.fptr(g), cases.fptr(yn), 2, 320, C.c_float(1e-5))
    out["rmsnorm"] = yn
    qr, kr = rng.standard_normal((3, 4 * 64)).astype(np.float32), rng.standard_normal((3, 2 * 64)).astype(np.float32)
    lib.ck_test_rope(cases.fptr(qr), cases.fptr(kr), 3, 4, 2, 64, 5, C.c_float(1.0e4))
    out["rope_q"], out["rope_k"] = qr, kr
    gu = (2 * rng.standard_normal((2, 2 * 96))).astype(np.float32)
    so = np.zeros((2, 96), np.float32)
    lib.ck_test_swiglu(cases.fptr(gu), cases.fptr(so), 2, 96)
    out["swiglu"] = so
    qi, ki = rng.standard_normal((3, 4 * 64)).astype(np.float32), rng.standard_normal((3, 2 * 64)).astype(np.float32)
    lib.ck_test_rope_interleaved(cases.fptr(qi), cases.fptr(ki), 3, 4, 2, 64, 5, C.c_float(1.0e4))
    out["rope_interleaved_q"], out["rope_interleaved_k"] = qi, ki
    w40 = synth.make_weights("q4_0", 4, 128, 97)
    d40 = np.zeros(512, np.float32)
    lib.ck_test_dequant_q4_0(cases.vptr(w40), cases.fptr(d40), 512)
    out["dequant_q4_0"] = d40
    aq, ak, av = cases.prefill_attention_inputs(98, 4, 2, 64, 64, 9, 9)
    ao = np.zeros_like(aq)
    lib.ck_test_attention_causal(cases.fptr(aq), cases.fptr(ak), cases.fptr(av), cases.fptr(ao), 4, 2, 9, 9, 64)
    out["attention_causal"] = ao
    return out


def test_parity_api_reference_wrappers_match_oracle_compositions(ref_parity, ref, orc):
    """The reference's ck_test_* wrappers are thin compositions (quantise, then the quantised kernel); the same compositions of
    oracle functions give the same numbers, which is what the CUDA library's wrappers are held to on the GPU."""
    got = parity_api_cases(ref_parity, ref, "")
    w4, w6 = synth.make_weights("q4_k", 6, 512, 91), synth.make_weights("q6_k", 6, 512, 92)
    x512 = synth.make_x(512, 91)
    xq = cases.quantize_q8_k(orc, "oracle_", x512)
    assert np.array_equal(got["quantize_q8_k"], xq)
    assert np.array_equal(got["dequant_q4_k"], cases.dequant_row(orc, "oracle_", "q4_k", w4, 512))
    assert _close(got["gemv_q4_k"], cases.gemv(orc, "oracle_", "q4_k", w4, xq, 1, 512), 1e-5)
    assert _close(got["gemv_q6_k"], cases.gemv(orc, "oracle_", "q6_k", w6, xq, 1, 512), 1e-5)
    aq = cases.quantize_q8_k(orc, "oracle_", synth.make_x(512, 95, rows=3), rows=3)
    assert _close(got["gemm_q4_k"], cases.gemm_nt(orc, "oracle_", "q4_k", aq, w4, None, 3, 6, 512), 1e-5)
    assert _close(got["gemm_q6_k"], cases.gemm_nt(orc, "oracle_", "q6_k", aq, w6, None, 3, 6, 512), 1e-5)
