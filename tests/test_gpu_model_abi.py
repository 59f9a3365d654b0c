"""The two model-level ABIs of the reference, served by the device-resident step executor:
the singleton API that ck_chat.py binds (libckb200_model_v7.so) and the handle API of
include/ck_model_api.h (libckb200_model_api.so).  A small model is written to a CKB2MDL1 file,
loaded through each ABI, and its logits are checked against the CPU step oracle."""
from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

import cases
import step_oracle as so
from test_gpu_decode_step import MINI_QWEN, cosine

pytestmark = pytest.mark.gpu


def write_model_file(path, cfg, cpu: so.CpuModel):
    st = so.make_cfg(cfg, batch=1)
    with open(path, "wb") as f:
        f.write(b"CKB2MDL1")
        f.write(struct.pack("<I", 1))
        f.write(bytes(st))
        def put(a):
            a = np.ascontiguousarray(a)
            f.write(struct.pack("<Q", a.nbytes))
            f.write(a.tobytes())
        for lay in cpu.layers:
            put(lay["LN1"])
            for n in ("WQ", "WK", "WV", "WO"):
                put(lay[n][3])
            put(lay["LN2"])
            put(lay["W1"][3])
            put(lay["W2"][3])
        put(cpu.final_gamma)
        put(cpu.lm_head[3])


@pytest.fixture(scope="module")
def model_file(tmp_path_factory):
    cpu = so.CpuModel(MINI_QWEN, seed=21)
    path = str(tmp_path_factory.mktemp("model") / "mini.ckb2mdl")
    write_model_file(path, MINI_QWEN, cpu)
    return path


def expected_logits(orc, tokens):
    cpu = so.CpuModel(MINI_QWEN, seed=21)
    out = None
    for pos, t in enumerate(tokens):
        out = cpu.decode(orc, t, pos)
    return out


def test_singleton_api_like_ck_chat(ck, orc, pkg, model_file):
    lib = C.CDLL(pkg.find_lib("libckb200_model_v7.so"))
    lib.ck_model_get_logits.restype = C.POINTER(C.c_float)
    assert lib.ck_model_init(model_file.encode()) == 0
    try:
        V = lib.ck_model_get_vocab_size()
        assert V == MINI_QWEN["vocab_size"] and lib.ck_model_get_context_window() == MINI_QWEN["max_seq_len"]
        prompt = np.array([3, 250, 77], dtype=np.int32)
        assert lib.ck_model_embed_tokens(prompt.ctypes.data_as(C.POINTER(C.c_int32)), 3) == 0
        out = np.zeros(V, np.float32)
        assert lib.ck_model_forward(cases.fptr(out)) == 0
        assert cosine(out, expected_logits(orc, [3, 250, 77])) >= 0.9999
        assert lib.ck_model_get_active_tokens() == 3
        assert lib.ck_model_decode(C.c_int32(9), None) == 0                      # ck_chat.py:1610 passes NULL and reads get_logits
        got = np.ctypeslib.as_array(lib.ck_model_get_logits(), shape=(V,)).copy()
        assert cosine(got, expected_logits(orc, [3, 250, 77, 9])) >= 0.9999
        lib.ck_model_kv_cache_reset()
        assert lib.ck_model_get_active_tokens() == 0
        assert lib.ck_model_decode(C.c_int32(3), cases.fptr(out)) == 0
        assert cosine(out, expected_logits(orc, [3])) >= 0.9999
    finally:
        lib.ck_model_free()


def test_handle_api_in_a_fresh_process(orc, pkg, model_file, tmp_path):
    """The handle library reads its model from CKB200_MODEL; run it the way test_generic_api.c does."""
    script = tmp_path / "run_handle.py"
    script.write_text(f"""
import ctypes as C, numpy as np, sys
lib = C.CDLL({pkg.find_lib("libckb200_model_api.so")!r})
lib.ck_model_create.restype = C.c_void_p
lib.ck_model_get_logits.restype = C.POINTER(C.c_float)
lib.ck_model_get_logits.argtypes = [C.c_void_p]
lib.ck_model_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
lib.ck_model_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
lib.ck_model_free.argtypes = [C.c_void_p]
lib.ck_model_precompute_rope.argtypes = [C.c_void_p]
m = lib.ck_model_create(); assert m
lib.ck_model_precompute_rope(m)
toks = np.array([3, 250, 77], dtype=np.int32)
lib.ck_model_forward(m, toks.ctypes.data, 3)
a = np.ctypeslib.as_array(lib.ck_model_get_logits(m), shape=({MINI_QWEN["vocab_size"]},)).copy()
t = np.array([9], dtype=np.int32)
lib.ck_model_decode(m, t.ctypes.data, 3)
b = np.ctypeslib.as_array(lib.ck_model_get_logits(m), shape=({MINI_QWEN["vocab_size"]},)).copy()
np.save(sys.argv[1], np.stack([a, b]))
lib.ck_model_free(m)
""")
    out = str(tmp_path / "logits.npy")
    env = dict(os.environ, CKB200_MODEL=model_file)
    subprocess.run([sys.executable, str(script), out], check=True, env=env, timeout=300)
    got = np.load(out)
    assert cosine(got[0], expected_logits(orc, [3, 250, 77])) >= 0.9999
    assert cosine(got[1], expected_logits(orc, [3, 250, 77, 9])) >= 0.9999
