"""ctypes view of the step executor's C interface (include/ckb200_model.h): the configuration struct, argument types of the
ckb200_model_* entry points, and the two pointer helpers every caller of the library's C ABI needs.  Python only passes
pointers and sizes; all work happens in libckb200.so."""
from __future__ import annotations

import ctypes as C

import numpy as np

c_float_p = C.POINTER(C.c_float)


def fptr(a: np.ndarray):
    """float* of a C-contiguous float32 array."""
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(c_float_p)


def vptr(a: np.ndarray):
    """void* of a C-contiguous array."""
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


class CfgStruct(C.Structure):
    """CKB200ModelConfig, field for field."""
    _fields_ = [(n, C.c_int) for n in ("embed_dim", "num_heads", "num_kv_heads", "head_dim", "intermediate_size", "num_layers", "vocab_size", "max_seq_len")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int) for n in ("fmt_q", "fmt_k", "fmt_v", "fmt_o", "fmt_gate_up", "fmt_down", "fmt_lm_head", "fmt_embedding", "tie_embeddings", "batch", "tp_rank", "tp_size")]


def make_cfg(cfg: dict, batch=1, tp_rank=0, tp_size=1) -> CfgStruct:
    """A configuration with tied embeddings (the LM head doubles as the token table) from a dict of the model fields."""
    s = CfgStruct()
    for k, v in cfg.items():
        setattr(s, k, v)
    s.fmt_embedding = cfg["fmt_lm_head"]
    s.tie_embeddings = 1
    s.batch, s.tp_rank, s.tp_size = batch, tp_rank, tp_size
    return s


def bind_model_api(lib):
    """Declare argument and result types of the ckb200_model_* functions on a ctypes handle of libckb200.so."""
    lib.ckb200_model_create.restype = C.c_void_p
    lib.ckb200_model_create.argtypes = [C.POINTER(CfgStruct)]
    lib.ckb200_model_free.argtypes = [C.c_void_p]
    lib.ckb200_model_free.restype = None
    lib.ckb200_model_open.restype = C.c_void_p
    lib.ckb200_model_open.argtypes = [C.c_char_p, C.c_int]
    lib.ckb200_model_open_bump.restype = C.c_void_p
    lib.ckb200_model_open_bump.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    lib.ckb200_model_config.restype = C.POINTER(CfgStruct)
    lib.ckb200_model_config.argtypes = [C.c_void_p]
    lib.ckb200_model_upload_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t]
    lib.ckb200_model_tensor_bytes.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.ckb200_model_tensor_bytes.restype = C.c_size_t
    lib.ckb200_model_kv_device.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.ckb200_model_kv_device.restype = C.c_void_p
    lib.ckb200_model_kv_element_bytes.argtypes = [C.c_void_p]
    lib.ckb200_model_logits_device.argtypes = [C.c_void_p]
    lib.ckb200_model_logits_device.restype = C.c_void_p
    lib.ckb200_model_set_pos.argtypes = [C.c_void_p, C.c_int]
    lib.ckb200_model_get_pos.argtypes = [C.c_void_p]
    lib.ckb200_model_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ckb200_model_decode_repeat.argtypes = [C.c_void_p, C.c_int]
    lib.ckb200_model_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.ckb200_model_fill_synthetic.argtypes = [C.c_void_p, C.c_ulonglong]
    lib.ckb200_model_fill_kv_synthetic.argtypes = [C.c_void_p, C.c_int, C.c_ulonglong]
    lib.ckb200_model_weight_bytes.argtypes = [C.c_void_p]
    lib.ckb200_model_weight_bytes.restype = C.c_size_t
    lib.ckb200_model_use_tp.argtypes = [C.c_void_p]
    lib.ckb200_model_use_tp.restype = None
    lib.ckb200_copy_to_device.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    lib.ckb200_copy_to_host.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
