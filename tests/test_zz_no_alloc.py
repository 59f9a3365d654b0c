"""The allocation-free decode-attention entry point.

Who needs it: a caller that may not allocate device memory while decoding - a model runtime that
planned its whole device arena at load time, a real-time loop that must stay clear of the
allocator, a process that has given all remaining memory to another pool.  The ordinary entry
point takes its split-K scratch from the library's growing pool; this one keeps the scratch in a
fixed 4 MiB array inside the library and therefore needs only inputs and outputs.

The test calls it through the C ABI twice in a row (different context lengths, so the second
call runs over the first call's leftovers in the shared array) and checks each result against
the ordinary entry point and against the CPU oracle, checks that the calls left the amount of free
device memory unchanged, then checks that an oversized request is refused with a clear error.
It is collected last so that a failure here cannot hide any other test.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(ck, torch, fn_static: bool, q, kc, vc, tokens, splits, stream):
    batch, heads, ad = q.shape
    kvh, cap = kc.shape[1], kc.shape[2]
    out = torch.full_like(q, float("nan"))
    args = [C.c_void_p(q.data_ptr()), C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_int(batch), C.c_longlong(kvh * cap * ad), C.c_int(heads), C.c_int(kvh), C.c_int(tokens), C.c_int(cap),
            C.c_int(ad), C.c_int(ad)]
    sp = C.c_void_p(stream.cuda_stream)
    if fn_static:
        rc = ck.ckb200_dev_attention_decode_static(*args, C.c_int(splits), sp)
    else:
        rc = ck.ckb200_dev_attention_decode(*args, sp)
    stream.synchronize()
    return rc, out.cpu().numpy()


def _free_device_bytes(torch):
    free, _total = torch.cuda.mem_get_info()
    return free


def test_static_scratch_attention_matches_allocating_entry_point(ck, orc):
    import torch

    import cases

    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    rng = np.random.default_rng(123)
    # two calls in a row: a long context with many splits, then a shorter one with a different geometry
    for batch, heads, kvh, ad, tokens, cap in [(2, 16, 2, 128, 3000, 3072), (1, 14, 2, 64, 700, 1024)]:
        q = torch.from_numpy(rng.standard_normal((batch, heads, ad)).astype(np.float32)).to(dev)
        kc = torch.from_numpy(rng.standard_normal((batch, kvh, cap, ad)).astype(np.float32)).to(dev)
        vc = torch.from_numpy(rng.standard_normal((batch, kvh, cap, ad)).astype(np.float32)).to(dev)
        torch.cuda.synchronize()
        splits = ck.ckb200_attention_decode_splits(batch, kvh, tokens)
        assert splits > 1, "the case must exercise the scratch"
        rc_ref, want = _run(ck, torch, False, q, kc, vc, tokens, splits, stream)
        rc, got = _run(ck, torch, True, q, kc, vc, tokens, splits, stream)      # first call on the device: looks the array up
        assert rc_ref == 0 and rc == 0
        assert np.isfinite(got).all()
        assert float(np.max(np.abs(got - want))) <= 1e-4
        free_before = _free_device_bytes(torch)
        rc, got_auto = _run(ck, torch, True, q, kc, vc, tokens, 0, stream)      # split count chosen by the entry point
        rc2, got_again = _run(ck, torch, True, q, kc, vc, tokens, splits, stream)
        assert _free_device_bytes(torch) == free_before, "the entry point must not allocate device memory"
        assert rc == 0 and float(np.max(np.abs(got_auto - want))) <= 1e-4
        assert rc2 == 0 and np.array_equal(got_again, got)
        for b in range(batch):                                                  # and directly against the CPU oracle
            cpu = cases.attention_decode(orc, "oracle_", q[b].cpu().numpy(), kc[b].cpu().numpy(), vc[b].cpu().numpy(), tokens)
            assert float(np.max(np.abs(got[b] - cpu))) <= 1e-4


def test_static_scratch_rejects_oversized_request(ck):
    import torch

    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    ck.ckb200_attention_decode_static_scratch_limit.restype = C.c_size_t
    limit = ck.ckb200_attention_decode_static_scratch_limit()
    batch, heads, kvh, ad, tokens, cap, splits = 8, 64, 8, 128, 256, 256, 64
    assert batch * heads * splits * (ad + 2) * 4 > limit
    q = torch.zeros((batch, heads, ad), device=dev)
    kc = torch.zeros((batch, kvh, cap, ad), device=dev)
    vc = torch.zeros_like(kc)
    torch.cuda.synchronize()
    rc, _ = _run(ck, torch, True, q, kc, vc, tokens, splits, stream)
    assert rc == 6                                                    # CKB_ERR_LIMIT
    assert b"exceed" in ck.ckb200_last_error_message()
    ck.ckb200_clear_error()
    rc, out = _run(ck, torch, True, q, kc, vc, tokens, 1, stream)     # one split needs no scratch and always fits
    assert rc == 0 and np.isfinite(out).all()
