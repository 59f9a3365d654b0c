"""ctypes loaders for the two CPU checkers (test infrastructure; never imported by the product).

  load_oracle()     -> oracle/libck_oracle.so, this repository's C restatement
  load_reference()  -> oracle/_ref/libck_ref*.so, the reference's own kernels (None if not built)
  load_reference_parity() -> oracle/_ref/libck_ref_parity*.so, the reference's ck_test_* wrappers over those kernels

The reference library comes in two ISA levels; the one the host can execute is chosen
from /proc/cpuinfo so that a host without AVX-512 does not die with SIGILL.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def _cpu_flags() -> set[str]:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def build(reference: str | None = None) -> None:
    """Run the Makefile beside this file (compiles ck_oracle.c; the reference only if its tree exists)."""
    cmd = ["make", "-C", HERE, "-j4", "all"]
    if reference:
        cmd.append(f"REFERENCE={reference}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def load_oracle() -> ctypes.CDLL:
    path = os.path.join(HERE, "libck_oracle.so")
    if not os.path.exists(path):
        build()
    return ctypes.CDLL(path)


def reference_path() -> str | None:
    flags = _cpu_flags()
    v4 = {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512cd", "avx512_vnni"}
    order = ["libck_ref.so", "libck_ref_avx2.so"] if v4 <= flags else ["libck_ref_avx2.so"]
    if "avx2" not in flags or "fma" not in flags:
        return None
    for name in order:
        p = os.path.join(HERE, "_ref", name)
        if os.path.exists(p):
            return p
    return None


def load_reference() -> ctypes.CDLL | None:
    p = reference_path()
    return ctypes.CDLL(p) if p else None


def load_reference_parity() -> ctypes.CDLL | None:
    """The reference's flat parity API (ck_test_*), built beside the kernels.  It wraps more kernels than this path compiles,
    so it is loaded with lazy binding; only the hot-path wrappers may be called."""
    p = reference_path()
    if not p:
        return None
    q = p.replace("libck_ref", "libck_ref_parity")
    if not os.path.exists(q):
        return None
    ctypes.CDLL(p, mode=ctypes.RTLD_GLOBAL)
    return ctypes.CDLL(q, mode=os.RTLD_LAZY)


def host_threads() -> int:
    """Threads the CPU baseline uses: the cores this process may run on, capped at the
    reference pool's hard limit of 64 (include/ck_threadpool.h:48)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(64, n))
