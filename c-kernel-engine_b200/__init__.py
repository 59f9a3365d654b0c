"""B200-native drop-in for C-Kernel-Engine's quantised decode/prefill hot path.

Python reaches the CUDA library the way the reference's own tests reach its C library:
a plain ctypes handle on a shared object that exports the reference's C symbols
(unittest/lib_loader.py:10-23 in the reference).  There is no CPU fallback: if the CUDA
library is missing or no GPU is present the calls fail loudly.
"""
from __future__ import annotations

import ctypes
import os

from . import model_api, synth, tp  # noqa: F401

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libckb200.so"


def find_lib(*names: str) -> str:
    """Same contract as the reference's lib_loader.find_lib: first existing candidate wins."""
    for name in names or (LIB_NAME,):
        for base in (os.path.join(PKG_DIR, "build"), PKG_DIR):
            path = os.path.join(base, name)
            if os.path.exists(path):
                return path
    raise FileNotFoundError(
        f"{', '.join(names or (LIB_NAME,))} not built: run `python -c 'import __graft_entry__ as g; g.build()'`")


_LIB = None


def load_lib(*names: str) -> ctypes.CDLL:
    """ctypes handle on the CUDA library (cached).  Raises if it has not been built."""
    global _LIB
    if names:
        return ctypes.CDLL(find_lib(*names))
    if _LIB is None:
        _LIB = ctypes.CDLL(find_lib())
        _LIB.ckb200_last_error_message.restype = ctypes.c_char_p
    return _LIB


def check(lib: ctypes.CDLL | None = None) -> None:
    """Raise RuntimeError if any call since the last check recorded an error (kernels are void)."""
    lib = lib or load_lib()
    code = lib.ckb200_last_error()
    if code != 0:
        msg = lib.ckb200_last_error_message().decode()
        lib.ckb200_clear_error()
        raise RuntimeError(f"ckb200 error {code}: {msg}")
