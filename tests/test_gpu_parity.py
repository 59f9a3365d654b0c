"""Parity of the CUDA path with the reference, through the C ABI, on a B200.

Bars (the contract of this path): Q8_K / Q8_0 activation quantisation and all integer stages
bit-exact; fp32 outputs within 1e-3 max relative error of the same-path CPU result (checked
much tighter against the output scale); decode attention within 1e-4 absolute.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
synth = cases.synth

REL_TOL = 1e-3          # max elementwise relative error, fp32 outputs (north-star tolerance)
SCALE_TOL = 1e-5        # max abs error relative to the largest output (what fp32 reordering costs)
ATTN_ABS_TOL = 1e-4


def assert_fp32_close(got, want, what=""):
    got64, want64 = got.astype(np.float64), want.astype(np.float64)
    err = np.abs(got64 - want64)
    scale = float(np.max(np.abs(want64))) or 1.0
    assert float(err.max()) <= SCALE_TOL * scale, f"{what}: max abs err {err.max():.3e} vs scale {scale:.3e}"
    rel = err / np.maximum(np.abs(want64), 1e-2 * scale)     # elementwise, guarded where |y| is tiny
    assert float(rel.max()) <= REL_TOL, f"{what}: max rel err {rel.max():.3e}"


# ---------------------------------------------------------------- golden vectors (reference outputs)

def test_golden_cases_through_host_abi(ck, golden):
    out = cases.golden_outputs(ck, "")
    for name in golden.files:
        if name.startswith("gemv_dispatch_"):
            continue
        assert name in out, name
        g, o = golden[name], out[name]
        if name.startswith(("q8k_", "q80_", "dequant_", "kv_store", "embed_")):
            assert np.array_equal(g, o), f"{name}: not bit-exact"
        elif name.startswith(("attn_", "prefill_attn_")):
            assert float(np.max(np.abs(g - o))) <= ATTN_ABS_TOL, name
        elif name in ("rope_cos", "rope_sin", "rope_q", "rope_k", "rmsnorm"):
            assert float(np.max(np.abs(g - o))) <= 2e-6 * max(1.0, float(np.max(np.abs(g)))), name
        elif name == "swiglu":
            assert float(np.max(np.abs(g - o))) <= 2e-4 * float(np.max(np.abs(g))), name   # reference uses a fast exp
        else:
            assert_fp32_close(o, g, name)


# ---------------------------------------------------------------- quantisers, bit-exact

@pytest.mark.parametrize("rows,k", [(1, 256), (1, 4096), (3, 4864), (32, 8192), (512, 4096)])
def test_quantize_q8_k_bit_exact(ck, orc, rows, k):
    x = synth.make_x(k, seed=rows + k, rows=rows) * np.float32(2.5)
    if rows > 2:
        x[1, 256:512] = 0.0                                   # an all-zero block inside a batch
    assert np.array_equal(cases.quantize_q8_k(ck, "", x, rows), cases.quantize_q8_k(orc, "oracle_", x, rows))


def test_quantize_q8_k_edge_cases_bit_exact(ck, orc):
    x = cases.q8k_edge_input()
    assert np.array_equal(cases.quantize_q8_k(ck, "", x), cases.quantize_q8_k(orc, "oracle_", x))


@pytest.mark.parametrize("rows,k", [(1, 32), (1, 896), (7, 4864), (64, 4096)])
def test_quantize_q8_0_bit_exact(ck, orc, rows, k):
    x = synth.make_x(k, seed=rows * 3 + k, rows=rows) * np.float32(0.3)
    assert np.array_equal(cases.quantize_q8_0(ck, "", x, rows), cases.quantize_q8_0(orc, "oracle_", x, rows))


# ---------------------------------------------------------------- GEMV: every kernel variant, ragged shapes

VARIANTS = {"q4_k": [1, 2, 10, 11, 12, 13, 14, 15, 16, 17, 20, 21, 22, 23, 30, 31, 32, 33], "q6_k": [1, 2], "q8_0": [1, 2]}
RAGGED = {
    "q4_k": [(1, 256), (3, 512), (7, 1024), (33, 4096), (130, 4864), (5, 14336), (257, 2048), (3, 36864), (300, 6144)],
    "q6_k": [(1, 256), (3, 512), (7, 1024), (33, 4096), (130, 4864), (5, 14336), (2, 28672)],
    "q8_0": [(1, 32), (3, 96), (7, 896), (33, 4096), (130, 4864), (5, 14336), (2, 28672)],
}


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_gemv_all_variants_ragged_shapes(ck, orc, fmt):
    key = ("gemv_" + fmt).encode()
    try:
        for m, k in RAGGED[fmt]:
            w = synth.make_weights(fmt, m, k, seed=m + k)
            xq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(k, seed=m + k))
            want = cases.gemv(orc, "oracle_", fmt, w, xq, m, k)
            for v in VARIANTS[fmt]:
                ck.ckb200_tune_set(key, v)
                got = cases.gemv(ck, "", fmt, w, xq, m, k)
                assert ck.ckb200_synchronize() == 0
                assert_fp32_close(got, want, f"{fmt} variant {v} {m}x{k}")
    finally:
        ck.ckb200_tune_set(key, 0)


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_gemv_ring_with_small_stages_splits_rows_into_chunks(ck, orc, fmt):
    """A tiny stage forces long rows through several bulk copies (partial sums carried across chunks)."""
    key = ("gemv_" + fmt).encode()
    try:
        ck.ckb200_tune_set(key, 1)
        ck.ckb200_tune_set(b"ring_stage_bytes", 1024)
        for m, k in [(9, 4096), (4, 14336), (300, 1024 if fmt != "q8_0" else 896)]:
            w = synth.make_weights(fmt, m, k, seed=k)
            xq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(k, seed=k))
            got = cases.gemv(ck, "", fmt, w, xq, m, k)
            assert ck.ckb200_synchronize() == 0
            assert_fp32_close(got, cases.gemv(orc, "oracle_", fmt, w, xq, m, k), f"{fmt} {m}x{k}")
    finally:
        ck.ckb200_tune_set(key, 0)
        ck.ckb200_tune_set(b"ring_stage_bytes", 0)


SWEEP = [(fmt, m, k) for fmt in ("q4_k", "q6_k", "q8_0") for (m, k) in synth.SWEEP_SHAPES]


@pytest.mark.parametrize("fmt,m,k_raw", SWEEP)
def test_gemv_benchmark_sweep_full_size(ck, orc, fmt, m, k_raw):
    """The benchmark shapes at full size, seed 0, against the CPU oracle (K=896 padded to 1024 for the K-quants)."""
    k = synth.k_for(fmt, k_raw)
    w = synth.make_weights(fmt, m, k, seed=0)
    x = synth.make_x(k, seed=0, k_valid=k_raw if k != k_raw else None)
    xq = cases.quantize_act(ck, "", fmt, x)
    assert np.array_equal(xq, cases.quantize_act(orc, "oracle_", fmt, x))
    got = cases.gemv(ck, "", fmt, w, xq, m, k)
    assert ck.ckb200_synchronize() == 0
    assert_fp32_close(got, cases.gemv(orc, "oracle_", fmt, w, xq, m, k), f"{fmt} {m}x{k}")


def test_gemv_row_split_variants_cover_all_rows(ck, orc):
    """gemv_*_parallel(ith, nth) computes rows [dr*ith, dr*(ith+1)); the union over ith is the whole result."""
    m, k, nth = 101, 1024, 7
    for fmt, name in (("q4_k", "gemv_q4_k_q8_k_parallel_simd"), ("q6_k", "gemv_q6_k_q8_k_parallel"), ("q8_0", "gemv_q8_0_q8_0_parallel_simd")):
        kk = k if fmt != "q8_0" else 896
        w = synth.make_weights(fmt, m, kk, seed=3)
        xq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(kk, seed=3))
        y = np.full(m, np.nan, dtype=np.float32)
        f = getattr(ck, name)
        f.restype = None
        for ith in range(nth):
            f(cases.fptr(y), cases.vptr(w), cases.vptr(xq), C.c_int(m), C.c_int(kk), C.c_int(ith), C.c_int(nth))
        assert_fp32_close(y, cases.gemv(orc, "oracle_", fmt, w, xq, m, kk), name)


def test_registered_weights_are_used_from_hbm(ck, orc):
    m, k = 64, 2048
    w = synth.make_weights("q4_k", m, k, seed=8)
    xq = cases.quantize_q8_k(orc, "oracle_", synth.make_x(k, seed=8))
    want = cases.gemv(orc, "oracle_", "q4_k", w, xq, m, k)
    assert ck.ckb200_register_weights(cases.vptr(w), C.c_size_t(w.nbytes)) == 0
    try:
        ck.ckb200_device_ptr.restype = C.c_void_p
        assert ck.ckb200_device_ptr(cases.vptr(w)) is not None
        inner = C.c_void_p(w.ctypes.data + 5 * (k // 256) * 144)
        assert ck.ckb200_device_ptr(inner) is not None
        # the device copy is what is read: scribbling on the host buffer must not change the result
        backup = w.copy()
        w[:] = 0
        got = cases.gemv(ck, "", "q4_k", w, xq, m, k)
        w[:] = backup
        assert_fp32_close(got, want, "registered")
    finally:
        assert ck.ckb200_unregister_weights(cases.vptr(w)) == 0
    assert ck.ckb200_device_ptr(cases.vptr(w)) is None


def test_silent_return_on_null_and_shape_error_is_reported(ck):
    y = np.full(4, np.nan, dtype=np.float32)
    w = synth.make_weights("q4_k", 4, 256, 1)
    ck.gemv_q4_k_q8_k(cases.fptr(y), cases.vptr(w), C.c_void_p(), C.c_int(4), C.c_int(256))     # NULL: silent, like the reference
    assert np.isnan(y).all() and ck.ckb200_last_error() == 0
    xq = np.zeros(292, dtype=np.uint8)
    ck.gemv_q4_k_q8_k(cases.fptr(y), cases.vptr(w), cases.vptr(xq), C.c_int(4), C.c_int(200))   # K % 256 != 0
    assert ck.ckb200_last_error() == 2
    ck.ckb200_clear_error()


# ---------------------------------------------------------------- fp32-activation path, GEMM, dequant

@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_fp32_activation_gemv(ck, orc, fmt):
    m, k = 17, 1024 if fmt != "q8_0" else 896
    w = synth.make_weights(fmt, m, k, seed=4)
    x = synth.make_x(k, seed=4)
    got = cases.gemv_f32(ck, "", fmt, w, x, m, k)
    deq = np.stack([cases.dequant_row(orc, "oracle_", fmt, w.reshape(m, -1)[r].copy(), k) for r in range(m)]).astype(np.float64)
    want = (deq @ x.astype(np.float64)).astype(np.float32)
    assert_fp32_close(got, want, fmt)


@pytest.mark.parametrize("fmt,m,n,k", [("q4_k", 5, 33, 1024), ("q6_k", 4, 20, 512), ("q8_0", 6, 17, 896), ("q4_k", 64, 96, 2048)])
def test_gemm_nt_matches_loop_of_gemv(ck, orc, fmt, m, n, k):
    w = synth.make_weights(fmt, n, k, seed=n)
    a = synth.make_x(k, seed=n, rows=m)
    aq = cases.quantize_act(orc, "oracle_", fmt, a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    got = cases.gemm_nt(ck, "", fmt, aq, w, bias, m, n, k)
    want = cases.gemm_nt(orc, "oracle_", fmt, aq, w, bias, m, n, k)
    assert_fp32_close(got, want, fmt)


@pytest.mark.parametrize("m,n,k,with_bias", [(64, 128, 256, False), (128, 256, 1024, True), (200, 200, 512, True), (512, 384, 4096, False),
                                               (65, 129, 768, True), (300, 1000, 2048, False),
                                               (16, 128, 256, False), (32, 300, 4096, True), (40, 256, 2048, True), (33, 520, 8192, True)])
def test_gemm_nt_q4_k_tensor_core(ck, orc, m, n, k, with_bias):
    """M >= 16 takes the tcgen05 kernel (32-token tiles up to 64 tokens, 128-token tiles above): full tiles, ragged token
    and row edges, one and many superblocks, K split over several CTAs where the grid would not fill the SMs."""
    w = synth.make_weights("q4_k", n, k, seed=m + n)
    a = synth.make_x(k, seed=m, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32) if with_bias else None
    want = cases.gemm_nt(orc, "oracle_", "q4_k", aq, w, bias, m, n, k)
    got = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
    assert_fp32_close(got, want, "q4_k tensor-core path")
    try:
        ck.ckb200_tune_set(b"gemm_tc", 0)
        by_rows = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
    finally:
        ck.ckb200_tune_set(b"gemm_tc", 1)
    assert_fp32_close(by_rows, want, "q4_k per-token path")


@pytest.mark.parametrize("tma", [1, 0])
@pytest.mark.parametrize("shape,rw", [(1, 2), (2, 2), (4, 2), (1, 1), (4, 1)])
@pytest.mark.parametrize("m,n,k", [(16, 128, 256), (1, 40, 512), (8, 129, 1024), (9, 64, 2048), (17, 300, 1280), (32, 1000, 4096), (33, 77, 768), (64, 260, 2560)])
def test_gemm_nt_q4_k_integer_mma_small_batches(ck, orc, tma, shape, rw, m, n, k):
    """Up to 64 tokens gemm_nt_q4_k_q8_k runs on the integer-MMA kernel that streams the weights through registers: all four token-tile
    counts (8, 16, 32, 64 slots) with ragged token and row counts, the three CTA shapes (8 row warps, 4 x 2 K slices, 2 x 4 K slices;
    superblock counts that do not divide by the slices, a slice without work for k = 256), one and two 16-row tiles per warp, and both
    ways of staging the activations (16-byte windows when K is a multiple of 1024, 4-byte copies otherwise); with tma = 1 the shapes
    whose K is a multiple of 1024 take the form fed by tiled bulk copies (rows past N and token slots past M are zero-filled by the
    copy).  The integer sums are exact, the slices are added in a fixed order: two runs agree bit for bit."""
    w = synth.make_weights("q4_k", n, k, seed=m + n)
    a = synth.make_x(k, seed=m, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32) if m % 2 else None
    want = cases.gemm_nt(orc, "oracle_", "q4_k", aq, w, bias, m, n, k)
    try:
        ck.ckb200_tune_set(b"gemm_q4k_mma_min", 1)
        ck.ckb200_tune_set(b"gemm_q4k_mma_shape", shape)
        ck.ckb200_tune_set(b"gemm_q4k_mma_rw", rw)
        ck.ckb200_tune_set(b"gemm_q4k_mma_tma", tma)
        ck.ckb200_launch_count.restype = C.c_longlong
        n0 = ck.ckb200_launch_count()
        got = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
        assert ck.ckb200_launch_count() - n0 == 1                # one kernel, no per-token loop
        again = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
    finally:
        ck.ckb200_tune_set(b"gemm_q4k_mma_min", 2)
        ck.ckb200_tune_set(b"gemm_q4k_mma_shape", 0)
        ck.ckb200_tune_set(b"gemm_q4k_mma_rw", 0)
        ck.ckb200_tune_set(b"gemm_q4k_mma_tma", 1)
    assert_fp32_close(got, want, "q4_k integer-MMA path")
    assert np.array_equal(got, again)


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
@pytest.mark.parametrize("m,small_max,slices", [(24, 64, 3), (24, 0, 3), (70, 64, 4), (64, 64, 1), (64, 64, 10)])
def test_gemm_tensor_core_split_k(ck, orc, fmt, m, small_max, slices):
    """Both tile widths with a forced number of K slices (uneven last slice: 10 superblocks in 3 or 4 slices; one
    superblock per slice), against the oracle; the slices are summed in a fixed order, so two runs agree bit for bit."""
    import torch

    dev = torch.device("cuda", 0)
    n, k = 260, 2560
    w = synth.make_weights(fmt, n, k, seed=m)
    a = synth.make_x(k, seed=m + 1, rows=m)
    aq = cases.quantize_act(orc, "oracle_", fmt, a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt(orc, "oracle_", fmt, aq, w, bias, m, n, k)
    raw, taq, tb = torch.from_numpy(w).to(dev), torch.from_numpy(aq).to(dev), torch.from_numpy(bias).to(dev)
    if fmt == "q6_k":
        ck.ckb200_q6_k_planar_bytes.restype = C.c_size_t
        wdev = torch.empty(ck.ckb200_q6_k_planar_bytes(n, k), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        assert ck.ckb200_dev_q6_k_to_planar(C.c_void_p(wdev.data_ptr()), C.c_void_p(raw.data_ptr()), n, k, None) == 0
        fn = ck.ckb200_dev_gemm_nt_q6_k_planar_q8_k
    else:
        wdev, fn = raw, ck.ckb200_dev_gemm_nt_q4_k_q8_k
    outs = []
    try:
        ck.ckb200_tune_set(b"gemm_q4k_mma", 0)             # this test is about the tcgen05 kernel's K split
        ck.ckb200_tune_set(b"gemm_tc_small_max", small_max)
        ck.ckb200_tune_set(b"gemm_tc_slices", slices)
        for _ in range(2):
            c = torch.full((m, n), float("nan"), device=dev)
            torch.cuda.synchronize()
            assert fn(C.c_void_p(taq.data_ptr()), C.c_void_p(wdev.data_ptr()), C.c_void_p(tb.data_ptr()), C.c_void_p(c.data_ptr()), m, n, k, None) == 0
            assert ck.ckb200_synchronize() == 0
            outs.append(c.cpu().numpy())
    finally:
        ck.ckb200_tune_set(b"gemm_q4k_mma", 1)
        ck.ckb200_tune_set(b"gemm_tc_small_max", 64)
        ck.ckb200_tune_set(b"gemm_tc_slices", 0)
    assert_fp32_close(outs[0], want, f"{fmt} split-K gemm")
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("m", [17, 40])
def test_gemm_nt_q4_k_integer_mma_tail_launch(ck, orc, m):
    """From 17 tokens up the rows behind whole waves of CTAs go to a second launch in smaller CTAs: 150 CTAs of 32 rows on 148 SMs
    leave 64 rows for it.  Same results within fp32 rounding as one launch; bit-identical between runs."""
    import torch

    n, k = 4800, 1024
    w = synth.make_weights("q4_k", n, k, seed=m)
    a = synth.make_x(k, seed=m + 1, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    bias = np.random.default_rng(m).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt(orc, "oracle_", "q4_k", aq, w, bias, m, n, k)
    ck.ckb200_launch_count.restype = C.c_longlong
    try:
        ck.ckb200_tune_set(b"gemm_q4k_mma_shape", 4)
        ck.ckb200_tune_set(b"gemm_q4k_mma_rw", 1)
        n0 = ck.ckb200_launch_count()
        got = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
        launches = ck.ckb200_launch_count() - n0
        again = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
        ck.ckb200_tune_set(b"gemm_q4k_mma_tail", 0)
        single = cases.gemm_nt(ck, "", "q4_k", aq, w, bias, m, n, k)
    finally:
        ck.ckb200_tune_set(b"gemm_q4k_mma_shape", 0)
        ck.ckb200_tune_set(b"gemm_q4k_mma_rw", 0)
        ck.ckb200_tune_set(b"gemm_q4k_mma_tail", 1)
    assert_fp32_close(got, want, "q4_k integer-MMA tail launch")
    assert_fp32_close(single, want, "q4_k integer-MMA single launch")
    assert np.array_equal(got, again)
    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        assert launches == 2, launches
        assert np.array_equal(got[:, :4736], single[:, :4736])      # the rows of the whole waves come from the same CTAs either way


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
def test_gemm_nt_tensor_core_tail_launch(ck, orc, fmt):
    """A tile grid of whole waves plus a few tiles (150 tiles on 148 SMs) sends the last row tile to a second launch with K split:
    same results within fp32 rounding, two launches more than with the switch off, two runs bit-identical."""
    m, n, k = 130, 9600, 2048
    w = synth.make_weights(fmt, n, k, seed=5)
    a = synth.make_x(k, seed=6, rows=m)
    aq = cases.quantize_act(orc, "oracle_", fmt, a, rows=m)
    bias = np.random.default_rng(7).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt(orc, "oracle_", fmt, aq, w, bias, m, n, k)
    ck.ckb200_launch_count.restype = C.c_longlong
    n0 = ck.ckb200_launch_count()
    got = cases.gemm_nt(ck, "", fmt, aq, w, bias, m, n, k)
    with_tail = ck.ckb200_launch_count() - n0
    again = cases.gemm_nt(ck, "", fmt, aq, w, bias, m, n, k)
    try:
        ck.ckb200_tune_set(b"gemm_tc_tail", 0)
        n0 = ck.ckb200_launch_count()
        plain = cases.gemm_nt(ck, "", fmt, aq, w, bias, m, n, k)
        without = ck.ckb200_launch_count() - n0
    finally:
        ck.ckb200_tune_set(b"gemm_tc_tail", 1)
    assert_fp32_close(got, want, f"{fmt} tail launch")
    assert_fp32_close(plain, want, f"{fmt} single launch")
    assert np.array_equal(got, again)
    import torch

    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        assert with_tail == without + 2, (with_tail, without)


@pytest.mark.parametrize("m", [64, 128])
def test_gemm_nt_q4_k_tensor_core_extreme_values(ck, orc, m):
    """Largest scales, nibbles and activations: the integer sums reach the top of the fp32-exact range (both tile widths)."""
    n, k = 128, 512
    w = synth.make_weights("q4_k", n, k, seed=9).reshape(n, k // 256, 144).copy()
    w[:, :, 4:16] = 0xFF          # every 6-bit scale and min = 63
    w[:, :, 16:] = 0xFF           # every nibble = 15
    a = np.where(np.arange(k) % 3 == 0, -1.0, 1.0).astype(np.float32)[None, :].repeat(m, 0) * np.linspace(0.5, 2.0, m, dtype=np.float32)[:, None]
    aq = cases.quantize_act(orc, "oracle_", "q4_k", a, rows=m)
    got = cases.gemm_nt(ck, "", "q4_k", aq, w.reshape(-1), None, m, n, k)
    want = cases.gemm_nt(orc, "oracle_", "q4_k", aq, w.reshape(-1), None, m, n, k)
    assert_fp32_close(got, want, "q4_k")


# ---------------------------------------------------------------- decode attention + KV cache

ATTN_CASES = [  # heads, kv_heads, d(aligned), head_dim, tokens, capacity
    (14, 2, 64, 64, 1025, 2048),       # Qwen2-0.5B-shaped decode step
    (64, 8, 128, 128, 4096, 4096),     # Llama-3-70B-shaped
    (8, 4, 64, 64, 64, 64),            # the reference's own test case (unittest/test_kv_cache_attention.py:228-321)
    (8, 4, 64, 40, 63, 80),            # padded head: head_dim 40 in 64 aligned slots
    (4, 4, 64, 64, 1, 16),             # a single key
    (6, 2, 128, 128, 5, 8),
    (12, 4, 96, 96, 100, 128),         # head size outside the fast path
    (32, 2, 64, 64, 77, 128),          # group of 16 Q heads per KV head: generic path
]


@pytest.mark.parametrize("tensor_cores", [0, 1])
@pytest.mark.parametrize("heads,kvh,ad,hd,tokens,cap", ATTN_CASES)
def test_attention_decode(ck, orc, tensor_cores, heads, kvh, ad, hd, tokens, cap):
    """tensor_cores = 1 also sends a single sequence to the kernel that batches of sequences get (keys, values, query and probabilities
    split into fp16 pieces on the tensor cores; shapes outside it fall through to the same kernels as with 0).  Cache rows past the
    context hold infinities and NaNs."""
    q, kc, vc = cases.attention_inputs(tokens + heads, heads, kvh, ad, tokens, cap)
    if hd < ad:
        q[:, hd:] = 0
        kc[:, :, hd:] = 0
        vc[:, :, hd:] = 0
    kc[:, tokens:] = np.inf
    vc[:, tokens:] = np.nan
    ck.ckb200_tune_set(b"attn_f32_mma", tensor_cores)
    ck.ckb200_tune_set(b"attn_f16_mma_min_batch", 1 if tensor_cores else 2)

    def run(lib, prefix):
        out = np.full((heads, ad), np.nan, dtype=np.float32)
        cases.fn(lib, prefix, "attention_forward_decode_head_major_gqa_flash")(
            cases.fptr(q), cases.fptr(kc), cases.fptr(vc), cases.fptr(out), C.c_int(heads), C.c_int(kvh), C.c_int(tokens),
            C.c_int(cap), C.c_int(hd), C.c_int(ad))
        return out

    want = run(orc, "oracle_")
    try:
        for splits in (0, 1, 3, 16):
            ck.ckb200_tune_set(b"attn_splits", splits)
            got = run(ck, "")
            ck.ckb200_tune_set(b"attn_splits", 0)
            assert float(np.max(np.abs(got - want))) <= ATTN_ABS_TOL, (splits, float(np.max(np.abs(got - want))))
    finally:
        ck.ckb200_tune_set(b"attn_splits", 0)
        ck.ckb200_tune_set(b"attn_f32_mma", 1)
        ck.ckb200_tune_set(b"attn_f16_mma_min_batch", 2)


@pytest.mark.parametrize("tensor_cores", [0, 1])
@pytest.mark.parametrize("heads,kvh,d,tokens,cap", [(14, 2, 64, 1025, 2048), (64, 8, 128, 4096, 4096), (8, 4, 64, 64, 64), (4, 4, 64, 1, 16),
                                                    (6, 2, 128, 5, 8), (16, 2, 128, 333, 512), (8, 1, 128, 130, 131)])
def test_attention_decode_f16_cache(ck, orc, tensor_cores, heads, kvh, d, tokens, cap):
    """Decode attention over an IEEE fp16 KV cache (half the bytes), every split count, against the oracle: the tile kernel that widens
    the cache to fp32, and the tensor-core kernel (query and probabilities split into two fp16 pieces) that batches of sequences get;
    cache rows past the context hold infinities and NaNs, which must not reach the result."""
    q, kc, vc = cases.attention_inputs(tokens + heads, heads, kvh, d, tokens, cap)
    kc16, vc16 = kc.astype(np.float16).view(np.uint16), vc.astype(np.float16).view(np.uint16)
    kc16[:, tokens:] = 0x7C00                                   # +inf
    vc16[:, tokens:] = 0x7E00                                   # NaN
    want = cases.attention_decode_f16cache(orc, "oracle_", q, kc16, vc16, tokens)
    assert np.isfinite(want).all()
    try:
        ck.ckb200_tune_set(b"attn_f16_mma", tensor_cores)
        ck.ckb200_tune_set(b"attn_f16_mma_min_batch", 1)
        for splits in (0, 1, 3, 16):
            ck.ckb200_tune_set(b"attn_splits", splits)
            got = cases.attention_decode_f16cache(ck, "", q, kc16, vc16, tokens)
            ck.ckb200_tune_set(b"attn_splits", 0)
            assert float(np.max(np.abs(got - want))) <= ATTN_ABS_TOL, (splits, float(np.max(np.abs(got - want))))
    finally:
        ck.ckb200_tune_set(b"attn_splits", 0)
        ck.ckb200_tune_set(b"attn_f16_mma", 1)
        ck.ckb200_tune_set(b"attn_f16_mma_min_batch", 2)


def test_kv_cache_store_f16_bit_exact_then_attend(ck, orc):
    """fp32 -> fp16 store is bit-exact with the oracle (ties, subnormals, large values), token by token, and attention over the
    cache built that way matches."""
    heads, kvh, d, cap, steps = 8, 4, 64, 32, 10
    rng = np.random.default_rng(7)
    kc_g = np.zeros((kvh, cap, d), np.uint16); vc_g = np.zeros_like(kc_g)
    kc_c, vc_c = kc_g.copy(), vc_g.copy()
    for t in range(steps):
        k = (rng.standard_normal((kvh, d)) * rng.choice([1e-7, 1e-3, 1.0, 2049.0], size=(kvh, d))).astype(np.float32)
        v = rng.standard_normal((kvh, d)).astype(np.float32)
        k[0, :4] = [1.0009765625, 1.00048828125, 65519.9, 6.0e-8]          # halfway cases, the overflow edge, a subnormal
        q = rng.standard_normal((heads, d)).astype(np.float32)
        cases.kv_cache_store_f16(ck, "", kc_g, vc_g, k, v, t)
        cases.kv_cache_store_f16(orc, "oracle_", kc_c, vc_c, k, v, t)
        assert np.array_equal(kc_g, kc_c) and np.array_equal(vc_g, vc_c)
    ks = np.clip(kc_g.view(np.float16).astype(np.float32), -8, 8).astype(np.float16).view(np.uint16)   # keep the scores in range
    a = cases.attention_decode_f16cache(ck, "", q, ks, vc_g, steps)
    b = cases.attention_decode_f16cache(orc, "oracle_", q, ks, vc_c, steps)
    assert float(np.max(np.abs(a - b))) <= ATTN_ABS_TOL


@pytest.mark.parametrize("m,k", [(1, 32), (3, 96), (7, 896), (33, 4096), (130, 4864), (5, 14336), (4100, 896), (151936, 896)])
def test_gemv_q5_0_q8_0(ck, orc, m, k):
    """Q5_0 weights (22-byte blocks, what GGUF Q4_K_M mixes use for K = 896 tensors) x Q8_0 activations, ring and direct kernels."""
    w = synth.make_weights("q5_0", m, k, seed=m % 97)
    xq = cases.quantize_q8_0(orc, "oracle_", synth.make_x(k, seed=k))
    want = cases.gemv(orc, "oracle_", "q5_0", w, xq, m, k)
    for variant in (0, 1, 2):
        ck.ckb200_tune_set(b"gemv_q5_0", variant)
        got = cases.gemv(ck, "", "q5_0", w, xq, m, k)
        ck.ckb200_tune_set(b"gemv_q5_0", 0)
        assert_fp32_close(got, want, f"q5_0 variant {variant}")


def test_dequant_and_fp32_gemv_q5_0(ck, orc):
    m, k = 37, 896
    w = synth.make_weights("q5_0", m, k, seed=21)
    assert np.array_equal(cases.dequant_row(ck, "", "q5_0", w, m * k), cases.dequant_row(orc, "oracle_", "q5_0", w, m * k))
    x = synth.make_x(k, seed=22)
    assert_fp32_close(cases.gemv_f32(ck, "", "q5_0", w, x, m, k), cases.gemv_f32(orc, "oracle_", "q5_0", w, x, m, k, "gemv_q5_0"), "gemv_q5_0 fp32")


def test_gemm_nt_and_vec_dot_q5_0(ck, orc):
    m, n, k = 5, 17, 896
    w = synth.make_weights("q5_0", n, k, seed=3)
    a = synth.make_x(k, seed=4, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q5_0", a, rows=m)
    bias = np.random.default_rng(5).standard_normal(n).astype(np.float32)
    assert_fp32_close(cases.gemm_nt(ck, "", "q5_0", aq, w, bias, m, n, k), cases.gemm_nt(orc, "oracle_", "q5_0", aq, w, bias, m, n, k), "gemm_nt_q5_0")
    s_g, s_o = np.zeros(1, np.float32), np.zeros(1, np.float32)
    ck.vec_dot_q5_0_q8_0(C.c_int(k), cases.fptr(s_g), cases.vptr(w), cases.vptr(aq))
    orc.oracle_vec_dot_q5_0_q8_0(C.c_int(k), cases.fptr(s_o), cases.vptr(w), cases.vptr(aq))
    assert abs(float(s_g[0]) - float(s_o[0])) <= 1e-3 * max(1e-3, abs(float(s_o[0])))


PREFILL_ATTN_CASES = [  # heads, kv_heads, ad, head_dim, tokens, kv stride, causal
    (32, 8, 128, 128, 512, 512, True),     # Llama-3-8B-shaped prefill
    (14, 2, 64, 64, 100, 128, True),       # Qwen2-0.5B heads: 7 query heads per kv head, strided cache
    (8, 4, 64, 40, 33, 48, True),          # padded head, odd token count (the last pair has one row)
    (4, 4, 64, 64, 1, 1, True),            # a single token
    (6, 2, 128, 128, 65, 65, True),        # three heads per kv head
    (16, 2, 128, 128, 50, 64, False),      # full (non-causal) form, 8 heads per kv head
    (3, 3, 64, 64, 130, 130, True),        # one head per kv head: 64-token blocks
]


@pytest.mark.parametrize("tensor_cores", [1, 0])
@pytest.mark.parametrize("heads,kvh,ad,hd,tokens,stride,causal", PREFILL_ATTN_CASES + [(8, 2, 128, 128, 333, 400, True), (8, 1, 64, 64, 200, 200, False)])
def test_attention_prefill(ck, orc, tensor_cores, heads, kvh, ad, hd, tokens, stride, causal):
    """Causal / full prefill attention through the reference-named entry points against the oracle: fp32 within
    ATTN_ABS_TOL absolute on outputs of order one; pad columns of the output are zero.  Both kernels: the tensor-core one (every
    operand split into two fp16 pieces) and the CUDA-core one it replaced."""
    q, k, v = cases.prefill_attention_inputs(tokens + heads, heads, kvh, ad, hd, tokens, stride)
    want = cases.attention_prefill(orc, "oracle_", q, k, v, hd, causal)
    ck.ckb200_tune_set(b"attn_prefill_mma", tensor_cores)
    try:
        got = cases.attention_prefill(ck, "", q, k, v, hd, causal)
    finally:
        ck.ckb200_tune_set(b"attn_prefill_mma", 1)
    assert float(np.max(np.abs(got - want))) <= ATTN_ABS_TOL, float(np.max(np.abs(got - want)))
    assert np.all(got[:, :, hd:] == 0)


@pytest.mark.parametrize("heads,kvh,ad,hd,tokens,stride,window", [(32, 8, 128, 128, 300, 300, 64), (14, 2, 64, 64, 100, 128, 1), (8, 4, 64, 40, 70, 70, 33),
                                                                   (8, 2, 128, 128, 90, 96, 17), (4, 4, 64, 64, 50, 50, 0), (6, 2, 64, 64, 40, 40, 1000)])
def test_attention_prefill_sliding_window(ck, orc, heads, kvh, ad, hd, tokens, stride, window):
    """Sliding-window prefill: windows of one key, windows that end inside a key tile, windows wider than the prompt, and no window."""
    q, k, v = cases.prefill_attention_inputs(tokens + window, heads, kvh, ad, hd, tokens, stride)
    want = cases.attention_prefill_sliding(orc, "oracle_", q, k, v, hd, window)
    got = cases.attention_prefill_sliding(ck, "", q, k, v, hd, window)
    assert float(np.max(np.abs(got - want))) <= ATTN_ABS_TOL, float(np.max(np.abs(got - want)))


@pytest.mark.parametrize("heads,kvh,d,tokens,cap,window", [(14, 2, 64, 1025, 2048, 512), (64, 8, 128, 4096, 4096, 1000), (8, 4, 64, 64, 64, 1),
                                                           (8, 4, 64, 20, 32, 0), (6, 2, 128, 77, 80, 500)])
def test_attention_decode_sliding_window(ck, orc, heads, kvh, d, tokens, cap, window):
    q, kc, vc = cases.attention_inputs(tokens + window, heads, kvh, d, tokens, cap)
    want = cases.attention_decode_sliding(orc, "oracle_", q, kc, vc, tokens, window)
    got = cases.attention_decode_sliding(ck, "", q, kc, vc, tokens, window)
    assert float(np.max(np.abs(got - want))) <= ATTN_ABS_TOL, float(np.max(np.abs(got - want)))


def test_attention_prefill_refuses_unsupported_shapes(ck):
    """Head sizes and group sizes outside the kernel are refused loudly, the output stays untouched."""
    q, k, v = cases.prefill_attention_inputs(1, 12, 4, 96, 96, 8, 8)
    out = cases.attention_prefill(ck, "", q, k, v, 96)
    assert np.all(np.isnan(out))
    assert ck.ckb200_last_error() != 0
    ck.ckb200_clear_error()


def test_kv_cache_store_then_attend_token_by_token(ck, orc):
    """The reference's own KV-cache test pattern: write token t, attend over 0..t, for every t."""
    heads, kvh, d, cap, steps = 8, 4, 64, 32, 12
    rng = np.random.default_rng(5)
    kc_g = np.zeros((kvh, cap, d), np.float32)
    vc_g = np.zeros_like(kc_g)
    kc_c, vc_c = kc_g.copy(), vc_g.copy()
    for t in range(steps):
        k = rng.standard_normal((kvh, d)).astype(np.float32)
        v = rng.standard_normal((kvh, d)).astype(np.float32)
        q = rng.standard_normal((heads, d)).astype(np.float32)
        cases.kv_cache_store(ck, "", kc_g, vc_g, k, v, t)
        cases.kv_cache_store(orc, "oracle_", kc_c, vc_c, k, v, t)
        assert np.array_equal(kc_g, kc_c) and np.array_equal(vc_g, vc_c)
        a = cases.attention_decode(ck, "", q, kc_g, vc_g, t + 1)
        b = cases.attention_decode(orc, "oracle_", q, kc_c, vc_c, t + 1)
        assert float(np.max(np.abs(a - b))) <= 1e-5


@pytest.mark.parametrize("batch,heads,kvh,d,tokens,cap,splits", [(1, 14, 2, 64, 1025, 2048, 0), (1, 64, 8, 128, 4096, 4096, 0), (2, 8, 4, 64, 130, 256, 3),
                                                              (1, 8, 8, 128, 70, 128, 1), (3, 16, 2, 128, 333, 512, 5)])
def test_attention_decode_fused_merge_and_quantise(ck, orc, batch, heads, kvh, d, tokens, cap, splits):
    """Attention + split merge + Q8_K quantisation in one launch: the rows match the oracle's attention, and the
    Q8_K blocks are bit-exact with the oracle's quantiser applied to those rows.  Called twice: the arrival
    counters must be back at zero after every call."""
    import torch

    dev = torch.device("cuda", 0)
    width = heads * d
    cols = -(-width // 256) * 256                       # the row sits in a zero-padded buffer, as in the step executor
    if batch > 1:
        assert cols == width
    rng = np.random.default_rng(tokens)
    q = rng.standard_normal((batch, heads, d)).astype(np.float32)
    kc = rng.standard_normal((batch, kvh, cap, d)).astype(np.float32)
    vc = rng.standard_normal((batch, kvh, cap, d)).astype(np.float32)
    want = np.stack([cases.attention_decode(orc, "oracle_", q[b], kc[b], vc[b], tokens) for b in range(batch)]).reshape(batch, width)

    ck.ckb200_attention_decode_scratch_bytes.restype = C.c_size_t
    ck.ckb200_attention_decode_counter_bytes.restype = C.c_size_t
    ck.ckb200_stream.restype = C.c_void_p
    nsplit = splits or ck.ckb200_attention_decode_splits(batch, kvh, tokens)
    tq, tk, tv = (torch.from_numpy(a).to(dev) for a in (q, kc, vc))
    out = torch.zeros(batch, cols, device=dev)
    scratch = torch.empty(max(256, ck.ckb200_attention_decode_scratch_bytes(batch, heads, d, nsplit)) // 4, device=dev)
    counters = torch.zeros(ck.ckb200_attention_decode_counter_bytes(batch, kvh) // 4 + 4, dtype=torch.int32, device=dev)
    q8 = torch.zeros(batch * (cols // 256) * 292, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    for _ in range(2):
        out[:, :width] = float("nan")
        q8.zero_()
        torch.cuda.synchronize()
        rc = ck.ckb200_dev_attention_decode_fused(
            C.c_void_p(tq.data_ptr()), C.c_void_p(tk.data_ptr()), C.c_void_p(tv.data_ptr()), C.c_void_p(out.data_ptr()), cols, batch,
            C.c_longlong(kvh * cap * d), heads, kvh, tokens, cap, d, d, nsplit, C.c_void_p(scratch.data_ptr()), C.c_void_p(counters.data_ptr()),
            None, C.c_void_p(q8.data_ptr()), cols, None)
        assert rc == 0 and ck.ckb200_synchronize() == 0
        got = out.cpu().numpy()
        assert float(np.max(np.abs(got[:, :width] - want))) <= ATTN_ABS_TOL
        assert not counters.cpu().numpy().any()
        for b in range(batch):
            assert np.array_equal(q8.cpu().numpy().reshape(batch, -1)[b], cases.quantize_q8_k(orc, "oracle_", got[b]))


@pytest.mark.parametrize("m,k", [(1, 256), (3, 512), (7, 1024), (33, 4096), (130, 4864), (5, 14336), (2, 28672), (300, 6144), (4100, 1024)])
def test_gemv_q6_k_planar_layout(ck, orc, m, k):
    """Weights re-laid row-planar on the device give the oracle's result; both row counts per lane group."""
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights("q6_k", m, k, seed=m + k)
    xq = cases.quantize_act(orc, "oracle_", "q6_k", synth.make_x(k, seed=m + k))
    want = cases.gemv(orc, "oracle_", "q6_k", w, xq, m, k)
    ck.ckb200_q6_k_planar_bytes.restype = C.c_size_t
    raw = torch.from_numpy(w).to(dev)
    planar = torch.full((ck.ckb200_q6_k_planar_bytes(m, k),), 0xAA, dtype=torch.uint8, device=dev)
    txq = torch.from_numpy(xq).to(dev)
    y = torch.full((m,), float("nan"), device=dev)
    torch.cuda.synchronize()
    assert ck.ckb200_dev_q6_k_to_planar(C.c_void_p(planar.data_ptr()), C.c_void_p(raw.data_ptr()), m, k, None) == 0
    try:
        for rows_per_group in (0, 1, 2):
            ck.ckb200_tune_set(b"gemv_q6p_rows", rows_per_group)
            y.fill_(float("nan"))
            torch.cuda.synchronize()
            assert ck.ckb200_dev_gemv_q6_k_planar_q8_k(C.c_void_p(y.data_ptr()), C.c_void_p(planar.data_ptr()), C.c_void_p(txq.data_ptr()), m, k, None) == 0
            assert ck.ckb200_synchronize() == 0
            assert_fp32_close(y.cpu().numpy(), want, f"q6_k planar {m}x{k} rows/group={rows_per_group}")
    finally:
        ck.ckb200_tune_set(b"gemv_q6p_rows", 0)


@pytest.mark.parametrize("m,n,k,big_scales", [(16, 128, 256, False), (32, 256, 1024, False), (64, 200, 512, True), (130, 384, 2048, False), (512, 256, 4096, True),
                                                 (48, 300, 8192, False)])
def test_gemm_nt_q6_k_planar_tensor_core(ck, orc, m, n, k, big_scales):
    """Q6_K prefill / batched-decode GEMM on tcgen05 over planar weights; with |scale| up to 127 some products
    leave the exactly representable fp16 range and are rounded (<= 2^-12 relative on that element)."""
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights("q6_k", n, k, seed=m + n).reshape(n, k // 256, 210).copy()
    if big_scales:
        w[:, :, 192:208] = np.random.default_rng(3).integers(-128, 128, size=(n, k // 256, 16)).astype(np.int8).view(np.uint8)
    w = w.reshape(-1)
    a = synth.make_x(k, seed=m, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q6_k", a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt(orc, "oracle_", "q6_k", aq, w, bias, m, n, k)
    ck.ckb200_q6_k_planar_bytes.restype = C.c_size_t
    raw, taq, tb = torch.from_numpy(w).to(dev), torch.from_numpy(aq).to(dev), torch.from_numpy(bias).to(dev)
    planar = torch.empty(ck.ckb200_q6_k_planar_bytes(n, k), dtype=torch.uint8, device=dev)
    c = torch.full((m, n), float("nan"), device=dev)
    torch.cuda.synchronize()
    assert ck.ckb200_dev_q6_k_to_planar(C.c_void_p(planar.data_ptr()), C.c_void_p(raw.data_ptr()), n, k, None) == 0
    assert ck.ckb200_dev_gemm_nt_q6_k_planar_q8_k(C.c_void_p(taq.data_ptr()), C.c_void_p(planar.data_ptr()), C.c_void_p(tb.data_ptr()),
                                                  C.c_void_p(c.data_ptr()), m, n, k, None) == 0
    assert ck.ckb200_synchronize() == 0
    got = c.cpu().numpy()
    if big_scales:
        err = np.abs(got.astype(np.float64) - want) / float(np.max(np.abs(want)))
        assert float(err.max()) <= 2e-4, float(err.max())
    else:
        assert_fp32_close(got, want, "q6_k planar gemm")


@pytest.mark.parametrize("shape,rw,occ", [(1, 2, 1), (2, 2, 1), (4, 2, 1), (1, 1, 1), (4, 1, 1), (1, 0, 2), (2, 0, 2), (4, 0, 2)])
@pytest.mark.parametrize("m,n,k", [(4, 40, 1024), (8, 129, 1024), (9, 64, 2048), (16, 300, 4096), (32, 1000, 3072), (33, 77, 1024), (64, 260, 5120)])
def test_gemm_nt_q6_k_integer_mma_small_batches(ck, orc, shape, rw, occ, m, n, k):
    """4 to 64 tokens over planar Q6_K weights run on the integer-MMA kernel (K a multiple of 1024): all four token-tile counts with
    ragged token and row counts, the three CTA shapes, one and two 16-row tiles per warp, one CTA per SM and (up to 16 tokens) the
    two-CTA form, scales over the whole int8 range (exact for every scale, unlike the fp16 operand of the tcgen05 kernel).  Two runs
    agree bit for bit."""
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights("q6_k", n, k, seed=m + n).reshape(n, k // 256, 210).copy()
    w[:, :, 192:208] = np.random.default_rng(m).integers(-128, 128, size=(n, k // 256, 16)).astype(np.int8).view(np.uint8)
    w = w.reshape(-1)
    a = synth.make_x(k, seed=m, rows=m)
    aq = cases.quantize_act(orc, "oracle_", "q6_k", a, rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32) if m % 2 else None
    want = cases.gemm_nt(orc, "oracle_", "q6_k", aq, w, bias, m, n, k)
    ck.ckb200_q6_k_planar_bytes.restype = C.c_size_t
    ck.ckb200_launch_count.restype = C.c_longlong
    raw, taq = torch.from_numpy(w).to(dev), torch.from_numpy(aq).to(dev)
    tb = torch.from_numpy(bias).to(dev) if bias is not None else None
    planar = torch.empty(ck.ckb200_q6_k_planar_bytes(n, k), dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    assert ck.ckb200_dev_q6_k_to_planar(C.c_void_p(planar.data_ptr()), C.c_void_p(raw.data_ptr()), n, k, None) == 0
    outs = []
    try:
        ck.ckb200_tune_set(b"gemm_q6k_mma_shape", shape)
        ck.ckb200_tune_set(b"gemm_q6k_mma_rw", rw)
        ck.ckb200_tune_set(b"gemm_q6k_mma_occ", occ)
        for _ in range(2):
            c = torch.full((m, n), float("nan"), device=dev)
            torch.cuda.synchronize()
            n0 = ck.ckb200_launch_count()
            assert ck.ckb200_dev_gemm_nt_q6_k_planar_q8_k(C.c_void_p(taq.data_ptr()), C.c_void_p(planar.data_ptr()), C.c_void_p(tb.data_ptr() if tb is not None else None),
                                                          C.c_void_p(c.data_ptr()), m, n, k, None) == 0
            assert ck.ckb200_launch_count() - n0 == 1            # one kernel: not the tcgen05 path (tiles + kernel), not a loop of GEMVs
            assert ck.ckb200_synchronize() == 0
            outs.append(c.cpu().numpy())
    finally:
        ck.ckb200_tune_set(b"gemm_q6k_mma_shape", 0)
        ck.ckb200_tune_set(b"gemm_q6k_mma_rw", 0)
        ck.ckb200_tune_set(b"gemm_q6k_mma_occ", 0)
    assert_fp32_close(outs[0], want, "q6_k integer-MMA path")
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("m,k", [(1, 32), (3, 96), (7, 896), (33, 4096), (130, 4864), (5, 14336), (2, 28672), (4100, 896)])
def test_gemv_q8_0_planar_layout(ck, orc, m, k):
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights("q8_0", m, k, seed=m + k)
    xq = cases.quantize_act(orc, "oracle_", "q8_0", synth.make_x(k, seed=m + k))
    want = cases.gemv(orc, "oracle_", "q8_0", w, xq, m, k)
    ck.ckb200_q8_0_planar_bytes.restype = C.c_size_t
    raw, txq = torch.from_numpy(w).to(dev), torch.from_numpy(xq).to(dev)
    planar = torch.full((ck.ckb200_q8_0_planar_bytes(m, k),), 0xAA, dtype=torch.uint8, device=dev)
    y = torch.full((m,), float("nan"), device=dev)
    torch.cuda.synchronize()
    assert ck.ckb200_dev_q8_0_to_planar(C.c_void_p(planar.data_ptr()), C.c_void_p(raw.data_ptr()), m, k, None) == 0
    assert ck.ckb200_dev_gemv_q8_0_planar_q8_0(C.c_void_p(y.data_ptr()), C.c_void_p(planar.data_ptr()), C.c_void_p(txq.data_ptr()), m, k, None) == 0
    assert ck.ckb200_synchronize() == 0
    assert_fp32_close(y.cpu().numpy(), want, f"q8_0 planar {m}x{k}")


@pytest.mark.parametrize("m,k", [(1, 32), (3, 96), (7, 896), (33, 4096), (130, 4864), (5, 14336), (2, 28672), (4100, 896)])
def test_gemv_q5_0_planar_layout(ck, orc, m, k):
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights("q5_0", m, k, seed=m + k)
    xq = cases.quantize_act(orc, "oracle_", "q5_0", synth.make_x(k, seed=m + k))
    want = cases.gemv(orc, "oracle_", "q5_0", w, xq, m, k)
    ck.ckb200_q5_0_planar_bytes.restype = C.c_size_t
    raw, txq = torch.from_numpy(w).to(dev), torch.from_numpy(xq).to(dev)
    planar = torch.full((ck.ckb200_q5_0_planar_bytes(m, k),), 0xAA, dtype=torch.uint8, device=dev)
    y = torch.full((m,), float("nan"), device=dev)
    torch.cuda.synchronize()
    assert ck.ckb200_dev_q5_0_to_planar(C.c_void_p(planar.data_ptr()), C.c_void_p(raw.data_ptr()), m, k, None) == 0
    assert ck.ckb200_dev_gemv_q5_0_planar_q8_0(C.c_void_p(y.data_ptr()), C.c_void_p(planar.data_ptr()), C.c_void_p(txq.data_ptr()), m, k, None) == 0
    assert ck.ckb200_synchronize() == 0
    assert_fp32_close(y.cpu().numpy(), want, f"q5_0 planar {m}x{k}")


@pytest.mark.parametrize("tokens,d_model,aligned,cols,with_delta", [(1, 896, 1024, 896, True), (3, 384, 512, 384, False), (2, 4096, 4096, 4096, True), (1, 100, 256, 128, True)])
def test_add_rmsnorm_q8_0_matches_the_three_kernel_form(ck, tokens, d_model, aligned, cols, with_delta):
    """Residual add + RMSNorm + Q8_0 quantisation in one kernel against add_inplace + rmsnorm_forward + quantize_q8_0 on the device:
    the same bytes (and the same updated residual)."""
    import torch

    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(tokens + d_model)
    x = np.zeros((tokens, aligned), np.float32); x[:, :d_model] = rng.standard_normal((tokens, d_model)).astype(np.float32)
    dl = np.zeros_like(x); dl[:, :d_model] = rng.standard_normal((tokens, d_model)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(aligned)).astype(np.float32)
    tg = torch.from_numpy(gamma).to(dev)
    x1, x2, d1 = torch.from_numpy(x).to(dev), torch.from_numpy(x).to(dev), torch.from_numpy(dl).to(dev)
    nbytes = tokens * (cols // 32) * 34
    q1 = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    q2 = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    normed = torch.zeros(tokens, aligned, device=dev)
    torch.cuda.synchronize()
    dptr = C.c_void_p(d1.data_ptr()) if with_delta else None
    assert ck.ckb200_dev_add_rmsnorm_q8_0(C.c_void_p(x1.data_ptr()), dptr, C.c_void_p(tg.data_ptr()), C.c_void_p(q1.data_ptr()), tokens, d_model, aligned, cols,
                                          C.c_float(1e-6), None) == 0
    if with_delta:
        assert ck.ckb200_dev_add_inplace(C.c_void_p(x2.data_ptr()), C.c_void_p(d1.data_ptr()), C.c_longlong(tokens * aligned), None) == 0
    assert ck.ckb200_dev_rmsnorm_forward(C.c_void_p(x2.data_ptr()), C.c_void_p(tg.data_ptr()), C.c_void_p(normed.data_ptr()), None, tokens, d_model, aligned,
                                         C.c_float(1e-6), None) == 0
    for t in range(tokens):
        assert ck.ckb200_dev_quantize_q8_0(C.c_void_p(normed.data_ptr() + 4 * t * aligned), C.c_void_p(q2.data_ptr() + t * (cols // 32) * 34), 1, cols, None) == 0
    assert ck.ckb200_synchronize() == 0
    assert torch.equal(x1, x2)
    assert torch.equal(q1, q2)


# ---------------------------------------------------------------- prefill GEMMs behind the reference's names, from the reference's own layouts

@pytest.mark.parametrize("m,n,k", [(16, 128, 256), (64, 200, 1024), (512, 384, 4096), (130, 96, 4864)])
def test_gemm_nt_q6_k_reference_layout_runs_on_tensor_cores(ck, orc, m, n, k):
    """gemm_nt_q6_k_q8_k[_parallel_dispatch] on the reference's 210-byte rows: from 16 tokens up the rows are re-laid per call
    and the tcgen05 kernel runs (two launches, not one GEMV per token)."""
    w = synth.make_weights("q6_k", n, k, seed=m + n)
    aq = cases.quantize_act(orc, "oracle_", "q6_k", synth.make_x(k, seed=m, rows=m), rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    want = cases.gemm_nt(orc, "oracle_", "q6_k", aq, w, bias, m, n, k)
    ck.ckb200_launch_count.restype = C.c_longlong
    n0 = ck.ckb200_launch_count()
    got = cases.gemm_nt(ck, "", "q6_k", aq, w, bias, m, n, k)
    assert ck.ckb200_launch_count() - n0 <= 5, "one GEMV per token is not a prefill GEMM"
    assert_fp32_close(got, want, f"q6_k gemm_nt {m}x{n}x{k}")
    c2 = np.full((m, n), np.nan, dtype=np.float32)
    cases.fn(ck, "", "gemm_nt_q6_k_q8_k_parallel_dispatch")(cases.vptr(aq), cases.vptr(w), cases.fptr(bias), cases.fptr(c2), m, n, k)
    assert np.array_equal(c2, got)


@pytest.mark.parametrize("m,n,k,with_bias", [(16, 128, 128, False), (64, 200, 896, True), (512, 384, 4096, True), (130, 1000, 4864, False), (300, 130, 1024, True)])
def test_gemm_nt_q8_0_integer_tensor_core(ck, orc, m, n, k, with_bias):
    """gemm_nt_q8_0_q8_0 from 16 tokens up: int8 MMAs, one block of 32 per instruction, scaled block by block in the reference's
    order - the same bits as the scalar loop."""
    w = synth.make_weights("q8_0", n, k, seed=m + n)
    aq = cases.quantize_act(orc, "oracle_", "q8_0", synth.make_x(k, seed=m, rows=m), rows=m)
    bias = np.random.default_rng(n).standard_normal(n).astype(np.float32) if with_bias else None
    want = cases.gemm_nt(orc, "oracle_", "q8_0", aq, w, bias, m, n, k)
    ck.ckb200_launch_count.restype = C.c_longlong
    n0 = ck.ckb200_launch_count()
    got = cases.gemm_nt(ck, "", "q8_0", aq, w, bias, m, n, k)
    launches = ck.ckb200_launch_count() - n0
    if k % 128 == 0:
        assert launches <= 4, launches
        assert np.array_equal(got, want), float(np.max(np.abs(got - want)))
    else:
        assert_fp32_close(got, want, "q8_0 gemm_nt by rows")
    c2 = np.full((m, n), np.nan, dtype=np.float32)
    b = cases.fptr(bias) if bias is not None else cases.c_float_p()
    cases.fn(ck, "", "gemm_nt_q8_0_q8_0_parallel_dispatch")(cases.vptr(aq), cases.vptr(w), b, cases.fptr(c2), m, n, k)
    assert np.array_equal(c2, got)


@pytest.mark.parametrize("fmt,m,k", [("q6_k", 300, 2048), ("q8_0", 200, 896), ("q5_0", 130, 4096)])
def test_registered_weights_in_unaligned_formats_get_a_planar_copy(ck, orc, fmt, m, k):
    """Resident Q6_K / Q8_0 / Q5_0 weights behind the host-pointer GEMV (and GEMM) are read from a row-planar copy built on first
    use; same results as on unregistered weights, and unregistering drops the copy."""
    w = synth.make_weights(fmt, m, k, seed=k)
    xq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(k, seed=1))
    want = cases.gemv(orc, "oracle_", fmt, w, xq, m, k)
    plain = cases.gemv(ck, "", fmt, w, xq, m, k)
    assert_fp32_close(plain, want, fmt)
    assert ck.ckb200_register_weights(cases.vptr(w), C.c_size_t(w.nbytes)) == 0
    try:
        for _ in range(2):                                   # first call builds the copy, second reuses it
            assert_fp32_close(cases.gemv(ck, "", fmt, w, xq, m, k), want, fmt + " registered")
        if fmt != "q5_0":
            mt = 32
            aq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(k, seed=2, rows=mt), rows=mt)
            assert_fp32_close(cases.gemm_nt(ck, "", fmt, aq, w, None, mt, m, k), cases.gemm_nt(orc, "oracle_", fmt, aq, w, None, mt, m, k), fmt + " registered gemm")
    finally:
        assert ck.ckb200_unregister_weights(cases.vptr(w)) == 0
    assert_fp32_close(cases.gemv(ck, "", fmt, w, xq, m, k), want, fmt + " after unregister")


@pytest.mark.parametrize("tokens,dim", [(1, 256), (3, 1024), (17, 4864)])
def test_swiglu_q8k_aligned_and_unaligned_inputs(ck, orc, tokens, dim):
    """swiglu_q8k (swiglu_forward + quantize_row_q8_k in one kernel) reads a 16-byte-aligned input with vector loads and any
    other with 4-byte loads: both give the same bytes, and the blocks decode to the oracle's swiglu within the Q8_K step."""
    import torch

    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(tokens * 1000 + dim)
    gu = (2.0 * rng.standard_normal((tokens, 2 * dim))).astype(np.float32)
    want = cases.swiglu(orc, "oracle_", gu, dim)
    nb = dim // 256
    outs = []
    for off in (0, 1):
        buf = torch.zeros(tokens * 2 * dim + 4, dtype=torch.float32, device=dev)
        buf[off:off + tokens * 2 * dim] = torch.from_numpy(gu.reshape(-1)).to(dev)
        q = torch.zeros(tokens * nb * 292, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        assert ck.ckb200_dev_swiglu_q8k(C.c_void_p(buf.data_ptr() + 4 * off), C.c_void_p(q.data_ptr()), tokens, dim, None) == 0
        assert ck.ckb200_synchronize() == 0
        outs.append(q.cpu().numpy())
    assert np.array_equal(outs[0], outs[1])
    blocks = outs[0].reshape(tokens, nb, 292)
    d = blocks[:, :, :4].copy().view(np.float32).reshape(tokens, nb, 1)
    qs = blocks[:, :, 4:260].view(np.int8).astype(np.float32)
    got = (d * qs).reshape(tokens, dim)
    step = np.abs(np.repeat(d.reshape(tokens, nb), 256, axis=1))            # Q8_K's d carries the sign of the block's largest element
    assert np.all(np.abs(got - want) <= 0.51 * step + 1e-4 * np.abs(want) + 1e-6)


@pytest.mark.parametrize("heads,kvh,d,tokens,cap,pos0", [(8, 2, 128, 37, 64, 0), (14, 2, 64, 20, 32, 5), (4, 4, 72, 9, 16, 0)])
def test_prefill_rope_scatter_vector_and_scalar_forms(ck, heads, kvh, d, tokens, cap, pos0):
    """prefill_rope_scatter (rotate-half RoPE of q and k, head-major q, k and v rows into the caches) takes 16-byte accesses when
    every pointer is aligned and the head size a multiple of 8, 4-byte accesses otherwise: both forms give the same bits and match
    the rotation computed here."""
    import torch

    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(heads * 100 + d)
    q = torch.randn(tokens, heads, d, generator=g)
    k = torch.randn(tokens, kvh, d, generator=g)
    v = torch.randn(tokens, kvh, d, generator=g)
    half = d // 2
    ang = torch.rand(cap, half, generator=g) * 6.0
    cos, sin = torch.cos(ang), torch.sin(ang)
    outs = []
    for off in (0, 1):                                          # off = 1: q_tm is only 4-byte aligned -> the scalar form
        qb = torch.zeros(q.numel() + 4, device=dev)
        qb[off:off + q.numel()] = q.reshape(-1).to(dev)
        kd, vd, cd, sd = k.to(dev).contiguous(), v.to(dev).contiguous(), cos.to(dev).contiguous(), sin.to(dev).contiguous()
        qh = torch.zeros(heads, tokens, d, device=dev)
        kc = torch.zeros(kvh, cap, d, device=dev)
        vc = torch.zeros(kvh, cap, d, device=dev)
        torch.cuda.synchronize()
        assert ck.ckb200_dev_prefill_rope_scatter(C.c_void_p(qb.data_ptr() + 4 * off), C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), C.c_void_p(qh.data_ptr()),
                                                  C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()), C.c_void_p(cd.data_ptr()), C.c_void_p(sd.data_ptr()),
                                                  tokens, heads, kvh, d, cap, pos0, None) == 0
        assert ck.ckb200_synchronize() == 0
        outs.append((qh.cpu(), kc.cpu(), vc.cpu()))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    c, s = cos[pos0:pos0 + tokens, None, :], sin[pos0:pos0 + tokens, None, :]

    def rot(x):
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)

    qh, kc, vc = outs[0]
    assert torch.allclose(qh, rot(q).permute(1, 0, 2), rtol=0, atol=2e-6)
    assert torch.allclose(kc[:, pos0:pos0 + tokens], rot(k).permute(1, 0, 2), rtol=0, atol=2e-6)
    assert torch.equal(vc[:, pos0:pos0 + tokens], v.permute(1, 0, 2))
    assert float(kc[:, pos0 + tokens:].abs().max()) == 0.0 if pos0 + tokens < cap else True
