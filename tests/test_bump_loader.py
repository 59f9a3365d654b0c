"""The loader of the reference's BUMPWGT5 weight files (version/v7/scripts/convert_gguf_to_bump_v7.py writes them,
version/v7/src/ckernel_model_load_v7.c reads them): digests, refusals (no GPU needed - they come before any device work) and, on a
GPU, decode steps of a model loaded from such a file against the CPU step."""
from __future__ import annotations

import ctypes as C
import hashlib

import numpy as np
import pytest

import bump_file
import cases
import step_oracle as so

LLAMA = dict(embed_dim=512, num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1024, num_layers=2, vocab_size=777,
             max_seq_len=64, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
Q5_0 = dict(embed_dim=384, num_heads=6, num_kv_heads=2, head_dim=64, intermediate_size=768, num_layers=2, vocab_size=500,
            max_seq_len=96, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=3, fmt_k=3, fmt_v=3, fmt_o=3, fmt_gate_up=3, fmt_down=1, fmt_lm_head=2)


@pytest.fixture(scope="module")
def lib(pkg):
    """The CUDA library loaded but not initialised: digests and refusals touch no device."""
    return pkg.load_lib()


def bind(ck):
    so.bind_model_api(ck)
    ck.ckb200_sha256.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]


@pytest.mark.parametrize("n", [0, 1, 55, 56, 63, 64, 65, 119, 120, 1000, 1 << 20])
def test_sha256_matches_hashlib(lib, n):
    ck = lib
    bind(ck)
    data = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
    out = np.zeros(32, np.uint8)
    ck.ckb200_sha256(cases.vptr(data) if n else None, n, cases.vptr(out))
    assert out.tobytes() == hashlib.sha256(data.tobytes()).digest()


def _write(tmp_path, cfg=LLAMA, **kw):
    cpu = so.CpuModel(cfg, seed=11)
    path, mp = tmp_path / "weights.bump", tmp_path / "weights_manifest.map"
    entries = bump_file.write_bump(path, mp, cpu, **kw)
    return cpu, path, mp, entries


def _refused(ck, path, mp, needle):
    h = ck.ckb200_model_open_bump(str(path).encode(), str(mp).encode() if mp else None, 1)
    assert not h
    assert needle in ck.ckb200_last_error_message().decode(), ck.ckb200_last_error_message()
    ck.ckb200_clear_error()


def test_corrupted_payload_is_refused(lib, tmp_path):
    ck = lib
    bind(ck)
    _, path, mp, entries = _write(tmp_path)
    raw = bytearray(path.read_bytes())
    raw[entries[3][2] + 5] ^= 0x40
    path.write_bytes(bytes(raw))
    _refused(ck, path, mp, "payload SHA-256 mismatch")


def test_corrupted_metadata_is_refused(lib, tmp_path):
    ck = lib
    bind(ck)
    _, path, mp, _ = _write(tmp_path)
    raw = bytearray(path.read_bytes())
    raw[-60] ^= 1                                   # inside the JSON blob, before the footer
    path.write_bytes(bytes(raw))
    _refused(ck, path, mp, "metadata SHA-256 mismatch")


def test_truncated_file_and_missing_map_are_refused(lib, tmp_path):
    ck = lib
    bind(ck)
    _, path, mp, _ = _write(tmp_path, meta=False)
    good = path.read_bytes()
    path.write_bytes(good[:-100])
    _refused(ck, path, mp, "SHA-256 mismatch")
    path.write_bytes(good)
    _refused(ck, path, tmp_path / "nowhere.map", "cannot open the manifest")
    (tmp_path / "other.bin").write_bytes(b"GGUF" + b"\0" * 200)
    _refused(ck, tmp_path / "other.bin", mp, "not a BUMPWGT5 file")


def test_what_the_executor_cannot_run_is_refused(lib, tmp_path):
    ck = lib
    bind(ck)
    _, path, mp, _ = _write(tmp_path, bias_value=0.25)
    _refused(ck, path, mp, "non-zero bias")
    _, path, mp, _ = _write(tmp_path)
    lines = mp.read_text().splitlines()
    mp.write_text("\n".join(l.replace("|q6_k|", "|fp16|") if l.startswith("layer.1.wv") else l for l in lines) + "\n")
    _refused(ck, path, mp, "weight format this library does not run")
    mp.write_text("\n".join(l for l in lines if not l.startswith("layer.0.w2")) + "\n")
    _refused(ck, path, mp, "layer.0.w2 is missing")
    mp.write_text("\n".join(lines[:5] + ["layer.0.wq|q4_k|0x98"]) + "\n")
    _refused(ck, path, mp, "malformed manifest line")
    mp.write_text("\n".join(l.replace("|q4_k|", "|q4_k|0x7fffffff|")[: l.index("|q4_k|") + 17] + "|1|0" if l.startswith("layer.0.wq") else l for l in lines) + "\n")
    _refused(ck, path, mp, "outside the payload")


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.gpu
@pytest.mark.parametrize("cfg,untied,via_open", [(LLAMA, False, True), (LLAMA, True, False), (Q5_0, False, False)])
def test_model_loaded_from_a_bump_file_decodes_like_the_cpu_step(ck, orc, tmp_path, cfg, untied, via_open):
    bind(ck)
    cpu, path, mp, _ = _write(tmp_path, cfg, untied_head=untied)
    if via_open:                                    # the generic open finds the map beside the file
        handle = ck.ckb200_model_open(str(path).encode(), 1)
    else:
        other = tmp_path / "elsewhere.map"
        mp.rename(other)
        handle = ck.ckb200_model_open_bump(str(path).encode(), str(other).encode(), 1)
    assert handle, ck.ckb200_last_error_message()
    try:
        got = ck.ckb200_model_config(handle).contents
        for key in ("embed_dim", "num_heads", "num_kv_heads", "head_dim", "intermediate_size", "num_layers", "vocab_size", "max_seq_len",
                    "fmt_q", "fmt_k", "fmt_v", "fmt_o", "fmt_gate_up", "fmt_down", "fmt_lm_head"):
            assert getattr(got, key) == cfg[key], key
        assert got.tie_embeddings == (0 if untied else 1)
        assert abs(got.rope_theta - cfg["rope_theta"]) < 1e-3 * cfg["rope_theta"] and abs(got.rms_eps - cfg["rms_eps"]) < 1e-9
        V = cfg["vocab_size"]
        for step, tok in enumerate([3, 41, 7, 300]):
            want = cpu.decode(orc, tok, step)
            ids = np.array([tok], np.int32)
            logits = np.full((1, V), np.nan, np.float32)
            assert ck.ckb200_model_decode(handle, cases.vptr(ids), cases.vptr(logits)) == 0, ck.ckb200_last_error_message()
            assert cosine(logits[0], want) >= 0.9999, step
            # one activation that rounds the other way in a Q8_0 block (inputs one ulp apart) moves logits by about 1 %
            assert float(np.max(np.abs(logits[0] - want))) < 2e-2 * float(np.max(np.abs(want))), step
    finally:
        ck.ckb200_model_free(handle)


@pytest.mark.gpu
def test_v7_init_with_manifest_loads_a_bump_file(ck, orc, pkg, tmp_path):
    """ck_chat.py's route: ck_model_init_with_manifest(weights.bump, weights_manifest.map), then decode."""
    v7 = C.CDLL(pkg.find_lib("libckb200_model_v7.so"))
    cpu, path, mp, _ = _write(tmp_path, LLAMA)
    v7.ck_model_init_with_manifest.argtypes = [C.c_char_p, C.c_char_p]
    assert v7.ck_model_init_with_manifest(str(path).encode(), str(mp).encode()) == 0
    try:
        V = v7.ck_model_get_vocab_size()
        assert V == LLAMA["vocab_size"] and v7.ck_model_get_context_window() == LLAMA["max_seq_len"]
        out = np.zeros(V, np.float32)
        assert v7.ck_model_decode(C.c_int32(12), cases.fptr(out)) == 0
        assert cosine(out, cpu.decode(orc, 12, 0)) >= 0.9999
    finally:
        v7.ck_model_free()
