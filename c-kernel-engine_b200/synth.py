"""Seeded synthetic inputs with the block layouts of the reference's quantised formats.

The reference's own kernel tests build their inputs with a seeded numpy generator and
push bytes through ctypes (unittest/test_q4_k_q8_k_matvec.py:63-95,
unittest/test_q6k_q8k_parity.py); these helpers do the same for the benchmark shapes.
Each field is written in struct order (include/ckernel_quant.h:104-157) so every
implementation (CPU or CUDA) sees identical bytes.

Value distributions (uniform-random packed fields, small positive fp16 scales):
  Q4_K  d ~ U(0, 0.02) fp16, dmin ~ U(0, 0.01) fp16, 12 scale bytes and 128 nibble bytes uniform
  Q6_K  ql/qh uniform bytes, int8 scales U{-32..31}, d ~ U(0, 0.02) fp16
  Q8_0  d ~ U(0, 0.01) fp16, int8 quants U{-127..127}
  x     fp32 N(0, 1)
"""
from __future__ import annotations

import numpy as np

QK_K = 256
QK8_0 = 32
BLOCK_BYTES = {"q4_k": 144, "q6_k": 210, "q8_0": 34, "q8_k": 292, "q5_0": 22, "q5_k": 176, "q4_0": 18, "q4_1": 20, "q5_1": 24, "q8_1": 36}
BLOCK_ELEMS = {"q4_k": 256, "q6_k": 256, "q8_0": 32, "q8_k": 256, "q5_0": 32, "q5_k": 256, "q4_0": 32, "q4_1": 32, "q5_1": 32, "q8_1": 32}


def row_bytes(fmt: str, k: int) -> int:
    """Bytes of one weight row of k elements (no row padding, as in the reference)."""
    assert k % BLOCK_ELEMS[fmt] == 0, (fmt, k)
    return (k // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]


def gemv_bytes(fmt: str, m: int, k: int, act: str = "q8") -> int:
    """Algorithmic bytes of one GEMV: weights + activation vector + fp32 outputs."""
    if act == "f32":
        xb = 4 * k
    elif fmt in ("q8_0", "q5_0"):
        xb = row_bytes("q8_0", k)
    else:
        xb = row_bytes("q8_k", k)
    return m * row_bytes(fmt, k) + xb + 4 * m


def make_q4_k(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    nb = rows * (k // QK_K)
    out = np.empty((nb, 144), dtype=np.uint8)
    out[:, 0:2] = rng.uniform(0.0, 0.02, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = rng.uniform(0.0, 0.01, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 4:16] = rng.integers(0, 256, (nb, 12), dtype=np.uint8)
    out[:, 16:144] = rng.integers(0, 256, (nb, 128), dtype=np.uint8)
    return out.reshape(-1)


def make_q6_k(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    nb = rows * (k // QK_K)
    out = np.empty((nb, 210), dtype=np.uint8)
    out[:, 0:128] = rng.integers(0, 256, (nb, 128), dtype=np.uint8)
    out[:, 128:192] = rng.integers(0, 256, (nb, 64), dtype=np.uint8)
    out[:, 192:208] = rng.integers(-32, 32, (nb, 16), dtype=np.int8).view(np.uint8)
    out[:, 208:210] = rng.uniform(0.0, 0.02, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return out.reshape(-1)


def make_q8_0(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    nb = rows * (k // QK8_0)
    out = np.empty((nb, 34), dtype=np.uint8)
    out[:, 0:2] = rng.uniform(0.0, 0.01, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 2:34] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def make_q5_0(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    """block_q5_0: fp16 d ~ U(0, 0.02), 4 bytes of fifth bits, 16 nibble bytes, all uniform random."""
    nb = rows * (k // QK8_0)
    out = np.empty((nb, 22), dtype=np.uint8)
    out[:, 0:2] = rng.uniform(0.0, 0.02, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 2:22] = rng.integers(0, 256, (nb, 20), dtype=np.uint8)
    return out.reshape(-1)




def _half_bytes(rng, lo, hi, n):
    return rng.uniform(lo, hi, n).astype(np.float16).view(np.uint8).reshape(n, 2)


def make_q5_k(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    """fp16 d, fp16 dmin, 12 scale bytes, 32 bytes of fifth bits, 128 nibble bytes (src/kernels/gemm_kernels_q5_k.c:49-55)"""
    nb = rows * (k // QK_K)
    out = rng.integers(0, 256, (nb, 176), dtype=np.uint8)
    out[:, 0:2] = _half_bytes(rng, 0.0, 0.02, nb)
    out[:, 2:4] = _half_bytes(rng, 0.0, 0.01, nb)
    return out.reshape(-1)


def make_block32(rng: np.random.Generator, rows: int, k: int, fmt: str) -> np.ndarray:
    """Q4_0 (d, 16 nibble bytes), Q4_1 (d, m, nibbles), Q5_1 (d, m, 4 bytes of fifth bits, nibbles): include/ckernel_quant.h:33-92"""
    nb = rows * (k // 32)
    out = rng.integers(0, 256, (nb, BLOCK_BYTES[fmt]), dtype=np.uint8)
    out[:, 0:2] = _half_bytes(rng, 0.0, 0.02, nb)
    if fmt != "q4_0":
        out[:, 2:4] = _half_bytes(rng, -0.05, 0.05, nb)
    return out.reshape(-1)


MAKERS = {"q4_k": make_q4_k, "q6_k": make_q6_k, "q8_0": make_q8_0, "q5_0": make_q5_0, "q5_k": make_q5_k, "q4_0": lambda r, rows, k: make_block32(r, rows, k, "q4_0"),
          "q4_1": lambda r, rows, k: make_block32(r, rows, k, "q4_1"), "q5_1": lambda r, rows, k: make_block32(r, rows, k, "q5_1")}


def make_weights(fmt: str, rows: int, k: int, seed: int = 0) -> np.ndarray:
    """uint8 array of rows * row_bytes(fmt, k) bytes."""
    return MAKERS[fmt](np.random.default_rng(seed), rows, k)


def make_x(k: int, seed: int = 0, k_valid: int | None = None, rows: int = 1) -> np.ndarray:
    """fp32 N(0,1) activations [rows, k]; columns >= k_valid are zero (K=896 padded to 1024)."""
    x = np.random.default_rng(seed + 7919).standard_normal((rows, k)).astype(np.float32)
    if k_valid is not None and k_valid < k:
        x[:, k_valid:] = 0.0
    return x if rows > 1 else x.reshape(k)


# Sweep of the quant-format GEMV benchmark: (out, in).  K = 896 runs natively for Q8_0
# (28 blocks per row) and zero-padded to 1024 for the K-quants, which need K % 256 == 0
# (the reference's own padded test: unittest/test_q4_k_q8_k_matvec.py:63-71, :313-314).
SWEEP_SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (151936, 896)]


def k_for(fmt: str, k: int) -> int:
    if fmt in ("q8_0", "q5_0"):
        return k
    return ((k + QK_K - 1) // QK_K) * QK_K
