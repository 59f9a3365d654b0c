"""The integer stage on the GPU, bit for bit: the per-sub-block int32 sums that the dequant-dot kernels build before
any floating point (Q4_K: eight sums of 32 products per superblock, src/kernels/gemm_kernels_q4k_q8k.c:144-167 in the
reference; Q6_K: sixteen sums of 16 products, src/kernels/gemm_kernels_q6k_q8k.c:92-111), dumped by the kernels' own
unit functions and compared with the CPU oracle's restatement of those loops."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
synth = cases.synth

# config 1 (4096 x 4096, seed 0), the ragged shapes of the GEMV tests and the other sweep shapes' row lengths
SHAPES = [(4096, 4096, 0), (1, 256, 1), (3, 512, 2), (7, 1024, 3), (33, 4096, 4), (130, 4864, 5), (5, 14336, 6), (2, 28672, 7), (300, 6144, 8), (1000, 1024, 9)]


def oracle_sums(orc, fmt, w, xq, m, k):
    per = 8 if fmt == "q4_k" else 16
    rb = synth.row_bytes(fmt, k)
    out = np.zeros((m, k // 256, per), dtype=np.int32)
    f = getattr(orc, f"oracle_{fmt}_q8_k_subblock_sums")
    f.restype = None
    for r in range(m):
        row = np.ascontiguousarray(w[r * rb:(r + 1) * rb])
        f(cases.vptr(row), cases.vptr(xq), C.c_int(k), out[r].ctypes.data_as(cases.c_int32_p))
    return out


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
@pytest.mark.parametrize("m,k,seed", SHAPES)
def test_subblock_sums_bit_exact(ck, orc, fmt, m, k, seed):
    import torch

    dev = torch.device("cuda", 0)
    w = synth.make_weights(fmt, m, k, seed)
    x = synth.make_x(k, seed)
    xq_gpu = cases.quantize_act(ck, "", fmt, x)
    xq = cases.quantize_act(orc, "oracle_", fmt, x)
    assert np.array_equal(xq_gpu, xq)                       # Q8_K activations: bit-exact, sums included
    rows = min(m, 64) if m * k > 1 << 22 else m             # the oracle loop is scalar: a slice of the big case ...
    pick = np.linspace(0, m - 1, rows).astype(np.int64) if rows < m else np.arange(m)
    want = oracle_sums(orc, fmt, np.concatenate([w[r * synth.row_bytes(fmt, k):(r + 1) * synth.row_bytes(fmt, k)] for r in pick]), xq, len(pick), k)
    tw, tx = torch.from_numpy(w).to(dev), torch.from_numpy(xq).to(dev)
    per = 8 if fmt == "q4_k" else 16
    f = getattr(ck, f"ckb200_dev_subblock_sums_{fmt}_q8_k")
    for variant in (0, 1):
        out = torch.full((m, k // 256, per), -(2 ** 31), dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        assert f(C.c_void_p(tw.data_ptr()), C.c_void_p(tx.data_ptr()), m, k, C.c_void_p(out.data_ptr()), variant, None) == 0
        assert ck.ckb200_synchronize() == 0
        got = out.cpu().numpy()
        assert np.array_equal(got[pick], want), f"{fmt} {m}x{k} variant {variant}: integer stage differs"
        if variant == 0:
            first = got
        else:
            assert np.array_equal(got, first), f"{fmt} {m}x{k}: the two kernel families disagree"   # ... and every row across families


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
def test_subblock_sums_recompose_the_gemv(ck, orc, fmt):
    """The dumped sums, combined with scales and activation sums as the reference does, give the GEMV output."""
    import torch

    dev = torch.device("cuda", 0)
    m, k = 37, 2048
    w = synth.make_weights(fmt, m, k, 77)
    xq = cases.quantize_act(orc, "oracle_", fmt, synth.make_x(k, 77))
    want = oracle_sums(orc, fmt, w, xq, m, k)
    per = 8 if fmt == "q4_k" else 16
    out = torch.zeros((m, k // 256, per), dtype=torch.int32, device=dev)
    tw, tx = torch.from_numpy(w).to(dev), torch.from_numpy(xq).to(dev)
    assert getattr(ck, f"ckb200_dev_subblock_sums_{fmt}_q8_k")(C.c_void_p(tw.data_ptr()), C.c_void_p(tx.data_ptr()), m, k, C.c_void_p(out.data_ptr()), 0, None) == 0
    assert ck.ckb200_synchronize() == 0
    assert np.array_equal(out.cpu().numpy(), want)
    y = cases.gemv(ck, "", fmt, w, xq, m, k)
    y_ref = cases.gemv(orc, "oracle_", fmt, w, xq, m, k)
    assert float(np.max(np.abs(y - y_ref))) <= 1e-5 * float(np.max(np.abs(y_ref)))
