"""The C-ABI surface, checked without a GPU: the library loads, exports every symbol that
include/*.h declares, and refuses to compute when there is no device (no CPU fallback)."""
from __future__ import annotations

import ctypes as C
import glob
import os
import re
import subprocess

import numpy as np
import pytest

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


HEADER_LIB = {"ckb200_model_v7.h": "libckb200_model_v7.so", "ckb200_model_handle.h": "libckb200_model_api.so"}


def declared_symbols(lib_name: str = "libckb200.so") -> dict[str, str]:
    out = {}
    for path in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        if HEADER_LIB.get(os.path.basename(path), "libckb200.so") != lib_name:
            continue
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
        text = re.sub(r"//[^\n]*", " ", text)
        text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
        text = text.replace('extern "C" {', " ")
        for stmt in text.split(";"):
            stmt = " ".join(stmt.split())
            m = re.match(r"^[A-Za-z_][\w\s\*]*?\b([A-Za-z_]\w*)\s*\(", stmt)
            if m and "typedef" not in stmt:
                out[m.group(1)] = os.path.basename(path)
    return out


def test_headers_declare_the_expected_surface():
    syms = declared_symbols()
    for name in ("quantize_row_q8_k", "gemv_q4_k_q8_k", "gemv_q6_k_q8_k", "gemv_q8_0_q8_0", "gemm_nt_q4_k_q8_k",
                 "attention_forward_decode_head_major_gqa_flash", "kv_cache_store", "gemv_q4_k_q8_k_parallel_dispatch",
                 "ckb200_dev_gemv_q4_k_q8_k", "ckb200_register_weights", "ckb200_last_error"):
        assert name in syms, name
    assert len(syms) > 100


@pytest.mark.parametrize("lib_name", ["libckb200.so", "libckb200_model_v7.so", "libckb200_model_api.so"])
def test_library_exports_every_declared_symbol(pkg, lib_name):
    path = pkg.find_lib(lib_name)
    nm = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in nm.splitlines() if " T " in line}
    declared = declared_symbols(lib_name)
    assert len(declared) >= 10
    missing = sorted(s for s in declared if s not in exported)
    assert not missing, f"declared in include/ but not exported by {lib_name}: {missing}"


def test_registry_contract(pkg):
    """ck_op_supported / ck_ir_validate_supported behave like src/ckernel_registry.c:26-60: seven forward ops, no backward ops."""
    lib = pkg.load_lib()
    assert [lib.ck_op_supported(op) for op in range(14)] == [1] * 7 + [0] * 7

    class KernelId(C.Structure):
        _fields_ = [("layer", C.c_uint16), ("node", C.c_uint16)]

    class InputRef(C.Structure):
        _fields_ = [("producer", KernelId), ("out_index", C.c_uint8)]

    class Node(C.Structure):
        _fields_ = [("id", KernelId), ("op", C.c_int), ("inputs", InputRef * 4), ("n_inputs", C.c_uint8), ("n_outputs", C.c_uint8)]

    class Cfg(C.Structure):
        _fields_ = [(n, C.c_int) for n in ("num_layers", "hidden_size", "intermediate_size", "num_heads", "num_kv_heads", "vocab_size", "context_window")] + \
                   [("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("rotary_dim", C.c_int), ("rope_scaling_factor", C.c_float),
                    ("rope_scaling_type", C.c_char * 16)]

    class Graph(C.Structure):
        _fields_ = [("config", Cfg), ("num_nodes", C.c_int), ("nodes", C.POINTER(Node))]

    nodes = (Node * 3)()
    for i, op in enumerate((0, 2, 6)):
        nodes[i].op = op
    g = Graph()
    g.num_nodes, g.nodes = 3, nodes
    assert lib.ck_ir_validate_supported(C.byref(g)) == 0
    nodes[1].op = 9                                   # ATTENTION_BWD
    assert lib.ck_ir_validate_supported(C.byref(g)) == -1
    assert lib.ck_ir_validate_supported(None) == -1
    lib.ckb200_op_kernels.restype = C.c_char_p
    assert b"gemv_q4_k_q8_k" in lib.ckb200_op_kernels(1) and lib.ckb200_op_kernels(9) is None


def test_every_header_entry_cites_the_reference():
    """Each block of declarations carries a reference file:line citation."""
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        assert len(re.findall(r"[\w/\.]+\.(?:c|h|py):\d+", text)) >= 3, path


def _has_gpu() -> bool:
    return os.path.exists("/dev/nvidiactl") or os.path.exists("/dev/nvidia0")


@pytest.mark.skipif(_has_gpu(), reason="checks the behaviour on a machine without a GPU")
def test_no_gpu_means_loud_failure_not_cpu_fallback(pkg):
    lib = pkg.load_lib()
    lib.ckb200_clear_error()
    assert lib.ckb200_init(0) == 4                      # CKB_ERR_NO_DEVICE
    y = np.full(4, np.nan, dtype=np.float32)
    w = cases.synth.make_weights("q4_k", 4, 256, 1)
    xq = np.zeros(292, dtype=np.uint8)
    lib.gemv_q4_k_q8_k(cases.fptr(y), cases.vptr(w), cases.vptr(xq), C.c_int(4), C.c_int(256))
    assert np.isnan(y).all(), "output was written without a GPU: something computed on the CPU"
    assert lib.ckb200_last_error() == 4
    with pytest.raises(RuntimeError):
        pkg.check(lib)
    assert lib.ckb200_last_error() == 0


def test_product_sources_never_touch_the_oracle():
    """The product path must not import, link or call anything under oracle/."""
    pkg_dir = os.path.join(ROOT, "c-kernel-engine_b200")
    for base, _, files in os.walk(pkg_dir):
        if os.path.basename(base) in ("build", "__pycache__"):
            continue
        for f in files:
            if f.endswith((".py", ".c", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.lower(), os.path.join(base, f)
