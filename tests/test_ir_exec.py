"""The lowered-IR executor (include/ckb200_ir.h): the reference's own lowering pipeline wrote the call IR fixtures under tests/golden/ir/
(tests/golden/make_ir_fixtures.py); here they are replayed on the device and compared with a CPU interpretation of the same files over
the oracle's kernels (tests/ir_oracle.py).  CPU part: the interpreter itself against the independent step oracle and against the
reference's kernels, and the refusals that need no device."""
from __future__ import annotations

import ctypes as C
import json

import numpy as np
import pytest

import bump_file
import cases
import ir_cases
import ir_oracle
import step_oracle as so

TOKENS = [3, 41, 7, 300]


@pytest.fixture(scope="module")
def lib(pkg):
    return bind(pkg.load_lib())


def bind(ck):
    ck.ckb200_ir_open.restype = C.c_void_p
    ck.ckb200_ir_open.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
    ck.ckb200_ir_free.argtypes = [C.c_void_p]
    ck.ckb200_ir_free.restype = None
    ck.ckb200_ir_decode.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    ck.ckb200_ir_reset.argtypes = [C.c_void_p]
    for name in ("get_pos", "vocab_size", "context_length", "num_ops", "graph_nodes"):
        getattr(ck, "ckb200_ir_" + name).argtypes = [C.c_void_p]
    ck.ckb200_ir_op_symbol.argtypes = [C.c_void_p, C.c_int]
    ck.ckb200_ir_op_symbol.restype = C.c_char_p
    ck.ckb200_ir_buffer.restype = C.c_void_p
    ck.ckb200_ir_buffer.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
    ck.ckb200_copy_to_host.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    return ck


def write_model(tmp_path, name):
    arch, cfg, seed = ir_cases.CASES[name]
    cpu = so.CpuModel(cfg, seed=seed)
    bump, mp = tmp_path / "weights.bump", tmp_path / "weights_manifest.map"
    bump_file.write_bump(bump, mp, cpu)
    return cfg, cpu, bump, mp


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


# ----------------------------------------------------------------------------- CPU: the checker itself

@pytest.mark.parametrize("name", ["qwen2_kquant", "qwen2_q5_0"])
def test_interpreter_equals_the_step_oracle(orc, tmp_path, name):
    """The qwen2 template lowers to exactly the recipe tests/step_oracle.py hard-codes: same kernels, same order, so the same bits."""
    cfg, cpu, bump, mp = write_model(tmp_path, name)
    m = ir_oracle.IrCpuModel(ir_cases.fixture_path(name), bump, mp, orc)
    for step, tok in enumerate(TOKENS):
        assert np.array_equal(m.decode(tok), cpu.decode(orc, tok, step)), step


@pytest.mark.parametrize("name", list(ir_cases.CASES))
def test_interpreter_over_the_reference_kernels(orc, ref, tmp_path, name):
    """The same files interpreted with the reference's own kernels (what its generated C calls) agree with the oracle's: cosine of the logits."""
    cfg, cpu, bump, mp = write_model(tmp_path, name)
    a = ir_oracle.IrCpuModel(ir_cases.fixture_path(name), bump, mp, orc)
    b = ir_oracle.IrCpuModel(ir_cases.fixture_path(name), bump, mp, ref, prefix="")
    for tok in TOKENS:
        la, lb = a.decode(tok), b.decode(tok)
        assert cosine(la, lb) >= 0.9999
        assert float(np.max(np.abs(la - lb))) <= 2e-2 * float(np.max(np.abs(lb)))


def test_llama_template_differs_from_the_qwen2_one(orc, tmp_path):
    """Pair-rotated RoPE and the fp16-rounded attention are a different function of the same weights: the executor must follow the file."""
    _, cpu, bump, mp = write_model(tmp_path, "llama_kquant")
    a = ir_oracle.IrCpuModel(ir_cases.fixture_path("llama_kquant"), bump, mp, orc)
    b = ir_oracle.IrCpuModel(ir_cases.fixture_path("qwen2_kquant"), bump, mp, orc)
    for tok in (5, 9, 2):
        a.decode(tok), b.decode(tok)
    # with a few tokens of context the logits of random weights barely notice (which is why the GPU test below compares the caches too);
    # the cached keys of positions > 0 are rotated differently
    assert float(np.max(np.abs(a.kv - b.kv))) > 0.1 * float(np.max(np.abs(b.kv)))
    assert not np.array_equal(a.buffers["attn_scratch"], b.buffers["attn_scratch"])


def _refused(lib, call, bump, mp, needle):
    h = lib.ckb200_ir_open(str(call).encode(), str(bump).encode(), str(mp).encode())
    msg = lib.ckb200_last_error_message().decode()
    lib.ckb200_clear_error()
    assert not h and needle in msg, msg


def test_files_the_executor_cannot_replay_are_refused(lib, tmp_path):
    _, _, bump, mp = write_model(tmp_path, "qwen2_kquant")
    doc = json.load(open(ir_cases.fixture_path("qwen2_kquant")))
    bad = tmp_path / "bad.json"

    d = json.loads(json.dumps(doc)); d["operations"][5]["function"] = "gated_deltanet_autoregressive_forward"
    bad.write_text(json.dumps(d)); _refused(lib, bad, bump, mp, "'gated_deltanet_autoregressive_forward', which this executor has no kernel for")
    d = json.loads(json.dumps(doc)); d["mode"] = "prefill"
    bad.write_text(json.dumps(d)); _refused(lib, bad, bump, mp, "replays lowered-ir-v3 decode files")
    d = json.loads(json.dumps(doc)); d["errors"] = ["op 3: unresolved weight"]
    bad.write_text(json.dumps(d)); _refused(lib, bad, bump, mp, "lowering errors")
    d = json.loads(json.dumps(doc)); d["memory"]["weights"]["entries"][3]["size"] += 64
    bad.write_text(json.dumps(d)); _refused(lib, bad, bump, mp, "bytes in the file and")
    d = json.loads(json.dumps(doc)); d["memory"]["activations"]["buffers"] = [b for b in d["memory"]["activations"]["buffers"] if b["name"] != "logits"]
    bad.write_text(json.dumps(d)); _refused(lib, bad, bump, mp, "memory plan lacks")
    bad.write_text(json.dumps(doc)[:-40]); _refused(lib, bad, bump, mp, "ir:")
    _refused(lib, tmp_path / "missing.json", bump, mp, "cannot open")


# ----------------------------------------------------------------------------- GPU: replay against the interpreter

@pytest.mark.gpu
@pytest.mark.parametrize("use_graph", [1, 0])
@pytest.mark.parametrize("name", list(ir_cases.CASES))
def test_replayed_steps_match_the_cpu_interpretation(ck, orc, tmp_path, name, use_graph):
    bind(ck)
    cfg, cpu, bump, mp = write_model(tmp_path, name)
    want_model = ir_oracle.IrCpuModel(ir_cases.fixture_path(name), bump, mp, orc)
    ck.ckb200_tune_set(b"model_graph", use_graph)
    h = ck.ckb200_ir_open(ir_cases.fixture_path(name).encode(), str(bump).encode(), None)      # the map is found beside the file
    assert h, ck.ckb200_last_error_message()
    try:
        doc = want_model.doc
        assert ck.ckb200_ir_num_ops(h) == len(doc["operations"]) and ck.ckb200_ir_vocab_size(h) == cfg["vocab_size"]
        assert [ck.ckb200_ir_op_symbol(h, i).decode() for i in range(len(doc["operations"]))] == [op["function"] for op in doc["operations"]]
        first = None
        for step, tok in enumerate(TOKENS + [11, 12]):
            want = want_model.decode(tok)
            got = np.full(cfg["vocab_size"], np.nan, np.float32)
            assert ck.ckb200_ir_decode(h, tok, cases.vptr(got)) == 0, ck.ckb200_last_error_message()
            first = got.copy() if first is None else first
            assert cosine(got, want) >= 0.9999, (step, cosine(got, want))
            assert float(np.max(np.abs(got - want))) <= 2e-2 * float(np.max(np.abs(want))), step
            assert ck.ckb200_ir_get_pos(h) == step + 1
            # intermediate state, tighter than logits can be: the cached keys carry the RoPE form, the attention row the attention variant
            # (layer 0 tightly; deeper layers sit behind activation quantisation, where one value rounding the other way moves things by 1e-3)
            layer0 = 2 * cfg["num_kv_heads"] * cfg["max_seq_len"] * cfg["head_dim"]
            for buf, count, tol in (("kv_cache", layer0, 1e-4), ("kv_cache", None, 5e-3), ("attn_scratch", None, 5e-3)):
                size = C.c_size_t()
                dev = ck.ckb200_ir_buffer(h, buf.encode(), C.byref(size))
                have = np.zeros(size.value // 4, np.float32)
                assert ck.ckb200_copy_to_host(cases.vptr(have), C.c_void_p(dev), have.nbytes) == 0
                ref_buf = want_model.buffers[buf][: have.nbytes].view(np.float32)
                have, ref_buf = have[:count], ref_buf[:count]
                assert float(np.max(np.abs(have - ref_buf))) <= tol * float(np.max(np.abs(ref_buf))), (buf, count, step)
        if use_graph:
            assert ck.ckb200_ir_graph_nodes(h) >= len(doc["operations"])
        assert ck.ckb200_ir_reset(h) == 0 and ck.ckb200_ir_get_pos(h) == 0
        again = np.zeros(cfg["vocab_size"], np.float32)
        assert ck.ckb200_ir_decode(h, TOKENS[0], cases.vptr(again)) == 0
        assert np.array_equal(again, first)
    finally:
        ck.ckb200_ir_free(h)
        ck.ckb200_tune_set(b"model_graph", 1)


@pytest.mark.gpu
def test_decode_past_the_context_is_refused(ck, tmp_path):
    bind(ck)
    cfg, cpu, bump, mp = write_model(tmp_path, "qwen2_kquant")
    h = ck.ckb200_ir_open(ir_cases.fixture_path("qwen2_kquant").encode(), str(bump).encode(), str(mp).encode())
    assert h, ck.ckb200_last_error_message()
    try:
        ck.ckb200_ir_set_pos.argtypes = [C.c_void_p, C.c_int]
        assert ck.ckb200_ir_set_pos(h, cfg["max_seq_len"]) == 0
        assert ck.ckb200_ir_decode(h, 1, None) != 0
        assert "past the context length" in ck.ckb200_last_error_message().decode()
        ck.ckb200_clear_error()
    finally:
        ck.ckb200_ir_free(h)


@pytest.mark.gpu
def test_v7_abi_replays_the_call_ir_beside_the_weights(ck, orc, pkg, tmp_path):
    """The reference's run folder (weights.bump, weights_manifest.map, lowered_decode_call.json) opened through ck_model_init as ck_chat.py does."""
    import shutil
    cfg, cpu, bump, mp = write_model(tmp_path, "llama_kquant")
    shutil.copyfile(ir_cases.fixture_path("llama_kquant"), tmp_path / "lowered_decode_call.json")
    want_model = ir_oracle.IrCpuModel(ir_cases.fixture_path("llama_kquant"), bump, mp, orc)
    v7 = C.CDLL(pkg.find_lib("libckb200_model_v7.so"))
    assert v7.ck_model_init(str(bump).encode()) == 0, ck.ckb200_last_error_message()
    try:
        V = v7.ck_model_get_vocab_size()
        assert V == cfg["vocab_size"] and v7.ck_model_get_context_window() == cfg["max_seq_len"]
        prompt = np.array(TOKENS, np.int32)
        assert v7.ck_model_embed_tokens(prompt.ctypes.data_as(C.POINTER(C.c_int32)), len(TOKENS)) == 0
        out = np.zeros(V, np.float32)
        assert v7.ck_model_forward(cases.fptr(out)) == 0
        for tok in TOKENS:
            want = want_model.decode(tok)
        assert cosine(out, want) >= 0.9999 and float(np.max(np.abs(out - want))) <= 2e-2 * float(np.max(np.abs(want)))
        assert v7.ck_model_decode(C.c_int32(9), cases.fptr(out)) == 0
        want = want_model.decode(9)
        assert cosine(out, want) >= 0.9999
        assert v7.ck_model_get_active_tokens() == len(TOKENS) + 1
        v7.ck_model_kv_cache_reset()
        assert v7.ck_model_get_active_tokens() == 0
    finally:
        v7.ck_model_free()


@pytest.mark.gpu
def test_ck_profile_writes_the_reference_rows(ck, tmp_path, monkeypatch):
    """CK_PROFILE / CK_PROFILE_CSV / CK_PROFILE_JSON as in the reference's --profile builds (version/v7/scripts/codegen_v7.py:1595-1685)."""
    bind(ck)
    cfg, cpu, bump, mp = write_model(tmp_path, "qwen2_kquant")
    h = ck.ckb200_ir_open(ir_cases.fixture_path("qwen2_kquant").encode(), str(bump).encode(), str(mp).encode())
    assert h, ck.ckb200_last_error_message()
    csv, js = tmp_path / "prof.csv", tmp_path / "prof.json"
    try:
        plain = np.zeros(cfg["vocab_size"], np.float32)
        assert ck.ckb200_ir_decode(h, 3, cases.vptr(plain)) == 0
        assert ck.ckb200_ir_reset(h) == 0
        monkeypatch.setenv("CK_PROFILE", "1")
        monkeypatch.setenv("CK_PROFILE_CSV", str(csv))
        monkeypatch.setenv("CK_PROFILE_JSON", str(js))
        timed = np.zeros(cfg["vocab_size"], np.float32)
        assert ck.ckb200_ir_decode(h, 3, cases.vptr(timed)) == 0
        assert ck.ckb200_ir_decode(h, 4, None) == 0
        assert np.array_equal(plain, timed)                       # timing changes nothing about the step
    finally:
        ck.ckb200_ir_free(h)
    rows = csv.read_text().strip().splitlines()
    nops = len(json.load(open(ir_cases.fixture_path("qwen2_kquant")))["operations"])
    assert rows[0] == "mode,kernel,op,layer,time_us,token_id" and len(rows) == 1 + 2 * nops
    first = rows[1].split(",")
    assert first[:4] == ["decode", "embedding_forward_q6_k", "dense_embedding_lookup", "-1"] and float(first[4]) >= 0 and first[5] == "0"
    assert rows[-1].split(",")[5] == "1"
    doc = json.loads(js.read_text())
    assert doc["total_entries"] == nops and doc["token_id"] == 1 and doc["entries"][4]["op"] == "q_proj"
