"""Seeded test cases for the hot path and one runner that drives any library exporting the
reference's C signatures: the reference itself (prefix ""), the CPU oracle (prefix
"oracle_") or the CUDA library (prefix "", host pointers in, host pointers out).

The same case definitions feed tests/golden/make_golden.py, so a golden file is the
reference's output on exactly the inputs the tests rebuild from the seed.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

synth = load_package().synth

c_float_p = C.POINTER(C.c_float)
c_int32_p = C.POINTER(C.c_int32)


def fptr(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(c_float_p)


def vptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def fn(lib, prefix: str, name: str, restype=None):
    f = getattr(lib, prefix + name)
    f.restype = restype
    return f


# ----------------------------------------------------------------------------- quantisers

def q8k_edge_input() -> np.ndarray:
    """Five 256-blocks that hit the quantiser's corner cases: all zero; +max and -max tied
    (first index wins and sets the sign); negative max first; products landing on .5 ties;
    one huge value among tiny ones."""
    x = np.zeros((5, 256), dtype=np.float32)
    x[1, 10], x[1, 200] = 3.0, -3.0
    x[1, 11:40] = np.linspace(-2.9, 2.9, 29, dtype=np.float32)
    x[2, 7], x[2, 8] = -5.0, 5.0
    x[2, 100:140] = np.linspace(-4.0, 4.0, 40, dtype=np.float32)
    x[3, 0] = 127.0
    x[3, 1:128] = np.arange(1, 128, dtype=np.float32) - 0.5      # iscale = -1 -> exact .5 ties
    x[3, 128:255] = -(np.arange(1, 128, dtype=np.float32) - 0.5)
    x[4, 33] = -1.0e20
    x[4, 34:60] = 1.0e-20
    return x.reshape(-1)


def quantize_q8_k(lib, prefix, x: np.ndarray, rows: int = 1) -> np.ndarray:
    k = x.size // rows
    out = np.zeros(rows * synth.row_bytes("q8_k", k), dtype=np.uint8)
    x = np.ascontiguousarray(x.reshape(-1))
    if rows == 1:
        fn(lib, prefix, "quantize_row_q8_k")(fptr(x), vptr(out), C.c_int(k))
    else:
        fn(lib, prefix, "quantize_batch_q8_k")(fptr(x), vptr(out), C.c_int(rows), C.c_int(k))
    return out


def quantize_q8_0(lib, prefix, x: np.ndarray, rows: int = 1) -> np.ndarray:
    k = x.size // rows
    out = np.zeros(rows * synth.row_bytes("q8_0", k), dtype=np.uint8)
    x = np.ascontiguousarray(x.reshape(-1))
    if rows == 1:
        fn(lib, prefix, "quantize_row_q8_0")(fptr(x), vptr(out), C.c_int(k))
    else:
        fn(lib, prefix, "quantize_batch_q8_0")(fptr(x), vptr(out), C.c_int(rows), C.c_int(k))
    return out


# ----------------------------------------------------------------------------- GEMV / GEMM

GEMV_SYMBOL = {"q4_k": "gemv_q4_k_q8_k", "q6_k": "gemv_q6_k_q8_k", "q8_0": "gemv_q8_0_q8_0", "q5_0": "gemv_q5_0_q8_0"}
GEMM_NT_SYMBOL = {"q4_k": "gemm_nt_q4_k_q8_k", "q6_k": "gemm_nt_q6_k_q8_k", "q8_0": "gemm_nt_q8_0_q8_0", "q5_0": "gemm_nt_q5_0_q8_0"}


def quantize_act(lib, prefix, fmt: str, x: np.ndarray, rows: int = 1) -> np.ndarray:
    return quantize_q8_0(lib, prefix, x, rows) if fmt in ("q8_0", "q5_0") else quantize_q8_k(lib, prefix, x, rows)


def gemv(lib, prefix, fmt: str, w: np.ndarray, xq: np.ndarray, m: int, k: int, symbol: str | None = None) -> np.ndarray:
    y = np.full(m, np.nan, dtype=np.float32)
    fn(lib, prefix, symbol or GEMV_SYMBOL[fmt])(fptr(y), vptr(w), vptr(xq), C.c_int(m), C.c_int(k))
    return y


def gemv_f32(lib, prefix, fmt: str, w: np.ndarray, x: np.ndarray, m: int, k: int, symbol: str | None = None) -> np.ndarray:
    """fp32-activation GEMV (gemv_q8_0 / gemv_q4_k / gemv_q6_k)."""
    y = np.full(m, np.nan, dtype=np.float32)
    fn(lib, prefix, symbol or ("gemv_" + fmt))(fptr(y), vptr(w), fptr(np.ascontiguousarray(x)), C.c_int(m), C.c_int(k))
    return y


def gemm_nt(lib, prefix, fmt: str, aq: np.ndarray, w: np.ndarray, bias, m: int, n: int, k: int) -> np.ndarray:
    c = np.full((m, n), np.nan, dtype=np.float32)
    b = fptr(bias) if bias is not None else c_float_p()
    fn(lib, prefix, GEMM_NT_SYMBOL[fmt])(vptr(aq), vptr(w), b, fptr(c), C.c_int(m), C.c_int(n), C.c_int(k))
    return c


def dequant_row(lib, prefix, fmt: str, w: np.ndarray, n: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    fn(lib, prefix, f"dequant_{fmt}_row")(vptr(w), fptr(out), C.c_size_t(n))
    return out


# ----------------------------------------------------------------------------- attention + glue

def attention_inputs(seed: int, heads: int, kv_heads: int, d: int, tokens: int, cap: int):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((heads, d)).astype(np.float32)
    kc = np.zeros((kv_heads, cap, d), dtype=np.float32)
    vc = np.zeros((kv_heads, cap, d), dtype=np.float32)
    kc[:, :tokens] = rng.standard_normal((kv_heads, tokens, d)).astype(np.float32)
    vc[:, :tokens] = rng.standard_normal((kv_heads, tokens, d)).astype(np.float32)
    return q, kc, vc


def attention_decode(lib, prefix, q, kc, vc, tokens: int) -> np.ndarray:
    heads, d = q.shape
    kv_heads, cap, _ = kc.shape
    out = np.full((heads, d), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_decode_head_major_gqa_flash")(
        fptr(q), fptr(kc), fptr(vc), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens),
        C.c_int(cap), C.c_int(d), C.c_int(d))
    return out


GOLDEN_PREFILL_ATTN = [(8, 4, 64, 64, 37, 40, 61), (4, 2, 64, 40, 9, 9, 62)]   # heads, kv heads, ad, head_dim, tokens, kv stride, seed


def prefill_attention_inputs(seed: int, heads: int, kv_heads: int, ad: int, hd: int, tokens: int, stride: int):
    """q [H][T][ad], k/v [Hkv][stride][ad]; the pad columns [hd, ad) hold garbage on purpose: the kernels must ignore them."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((heads, tokens, ad)).astype(np.float32)
    k = rng.standard_normal((kv_heads, stride, ad)).astype(np.float32)
    v = rng.standard_normal((kv_heads, stride, ad)).astype(np.float32)
    return q, k, v


def attention_prefill(lib, prefix, q, k, v, hd: int, causal: bool = True) -> np.ndarray:
    heads, tokens, ad = q.shape
    kv_heads, stride, _ = k.shape
    out = np.full((heads, tokens, ad), np.nan, dtype=np.float32)
    name = "attention_forward_causal_head_major_gqa_flash_strided" if causal else "attention_forward_full_head_major_gqa_flash_strided"
    fn(lib, prefix, name)(fptr(q), fptr(k), fptr(v), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(hd), C.c_int(ad),
                          C.c_int(stride))
    return out


def attention_prefill_sliding(lib, prefix, q, k, v, hd: int, window: int) -> np.ndarray:
    heads, tokens, ad = q.shape
    kv_heads, stride, _ = k.shape
    out = np.full((heads, tokens, ad), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_causal_head_major_gqa_flash_strided_sliding")(
        fptr(q), fptr(k), fptr(v), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(hd), C.c_int(ad), C.c_int(stride),
        C.c_int(window))
    return out


def attention_decode_sliding(lib, prefix, q, kc, vc, tokens: int, window: int) -> np.ndarray:
    heads, d = q.shape
    kv_heads, cap, _ = kc.shape
    out = np.full((heads, d), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_decode_head_major_gqa_flash_sliding")(
        fptr(q), fptr(kc), fptr(vc), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(cap), C.c_int(d), C.c_int(d),
        C.c_int(window))
    return out


def attention_decode_f16cache(lib, prefix, q, kc16, vc16, tokens: int, hd: int | None = None) -> np.ndarray:
    """kc16, vc16: uint16 arrays [Hkv][cap][ad] holding IEEE halves."""
    heads, d = q.shape
    kv_heads, cap, _ = kc16.shape
    out = np.full((heads, d), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_decode_head_major_gqa_flash_f16cache")(
        fptr(q), vptr(kc16), vptr(vc16), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(cap),
        C.c_int(hd or d), C.c_int(d))
    return out


def attention_decode_f16kv(lib, prefix, q, kc, vc, tokens: int, hd: int | None = None) -> np.ndarray:
    heads, d = q.shape
    kv_heads, cap, _ = kc.shape
    out = np.full((heads, d), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_decode_head_major_gqa_flash_f16kv")(
        fptr(q), fptr(kc), fptr(vc), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(cap), C.c_int(hd or d), C.c_int(d))
    return out


def attention_prefill_f16kv(lib, prefix, q, k, v, hd: int) -> np.ndarray:
    heads, tokens, ad = q.shape
    kv_heads, stride, _ = k.shape
    out = np.full((heads, tokens, ad), np.nan, dtype=np.float32)
    fn(lib, prefix, "attention_forward_causal_head_major_gqa_flash_strided_f16kv")(
        fptr(q), fptr(k), fptr(v), fptr(out), C.c_int(heads), C.c_int(kv_heads), C.c_int(tokens), C.c_int(hd), C.c_int(ad), C.c_int(stride))
    return out


def kv_cache_store_f16(lib, prefix, kc16, vc16, k, v, pos: int):
    kv_heads, cap, d = kc16.shape
    fn(lib, prefix, "kv_cache_store_f16")(vptr(kc16), vptr(vc16), fptr(k), fptr(v), C.c_int(0), C.c_int(pos), C.c_int(kv_heads),
                                          C.c_int(d), C.c_int(cap))


def kv_cache_store(lib, prefix, kc, vc, k, v, pos: int):
    kv_heads, cap, d = kc.shape
    fn(lib, prefix, "kv_cache_store")(fptr(kc), fptr(vc), fptr(k), fptr(v), C.c_int(0), C.c_int(pos),
                                      C.c_int(kv_heads), C.c_int(d), C.c_int(cap))


def rope_cache(lib, prefix, max_seq: int, d: int, theta: float):
    cos = np.zeros((max_seq, d // 2), dtype=np.float32)
    sin = np.zeros((max_seq, d // 2), dtype=np.float32)
    fn(lib, prefix, "rope_precompute_cache_split")(fptr(cos), fptr(sin), C.c_int(max_seq), C.c_int(d), C.c_float(theta))
    return cos, sin


def rope_qk(lib, prefix, q, k, cos, sin, pos: int, tokens: int = 1):
    """q [H, tokens, d], k [Hkv, tokens, d]; rotated in place."""
    heads, d = q.shape[0], q.shape[-1]
    fn(lib, prefix, "rope_forward_qk")(fptr(q), fptr(k), fptr(cos), fptr(sin), C.c_int(heads), C.c_int(k.shape[0]),
                                       C.c_int(tokens), C.c_int(d), C.c_int(d), C.c_int(pos))


def rmsnorm(lib, prefix, x, gamma, d_model: int, eps: float) -> np.ndarray:
    tokens, aligned = x.shape
    out = np.full_like(x, np.nan)
    fn(lib, prefix, "rmsnorm_forward")(fptr(x), fptr(gamma), fptr(out), c_float_p(), C.c_int(tokens),
                                       C.c_int(d_model), C.c_int(aligned), C.c_float(eps))
    return out


def swiglu(lib, prefix, x, dim: int) -> np.ndarray:
    tokens = x.shape[0]
    out = np.full((tokens, dim), np.nan, dtype=np.float32)
    fn(lib, prefix, "swiglu_forward")(fptr(x), fptr(out), C.c_int(tokens), C.c_int(dim))
    return out


def residual_add(lib, prefix, a, b) -> np.ndarray:
    out = np.full_like(a, np.nan)
    name = "residual_add_token_major" if prefix else "ck_residual_add_token_major"
    fn(lib, prefix, name)(fptr(a), fptr(b), fptr(out), C.c_int(a.shape[0]), C.c_int(a.shape[1]))
    return out


def embedding(lib, prefix, fmt: str, ids, table, vocab: int, embed: int, aligned: int) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.full((len(ids), aligned), np.nan, dtype=np.float32)
    fn(lib, prefix, f"embedding_forward_{fmt}")(ids.ctypes.data_as(c_int32_p), C.c_int(len(ids)), C.c_int(vocab),
                                               vptr(table), c_float_p(), fptr(out), C.c_int(embed), C.c_int(aligned),
                                               C.c_int(len(ids)), C.c_int(0))
    return out



# ----------------------------------------------------------------------------- fp32-activation GEMMs, contract forms, pairwise RoPE, copies

def gemm_nt_f32(lib, prefix, name: str, a: np.ndarray, w: np.ndarray, bias, m: int, n: int, k: int) -> np.ndarray:
    """gemm_nt_q4_k / gemm_nt_q6_k[_ref/_sse] / gemm_nt_q8_0 / gemm_nt_q8_0_q8_0_contract: A fp32 [m][k], B [n][k] blocks -> C [m][n]."""
    c = np.full((m, n), np.nan, dtype=np.float32)
    b = fptr(bias) if bias is not None else c_float_p()
    fn(lib, prefix, name)(fptr(np.ascontiguousarray(a.reshape(-1))), vptr(w), b, fptr(c), C.c_int(m), C.c_int(n), C.c_int(k))
    return c


def gemm_f32(lib, prefix, name: str, w: np.ndarray, x: np.ndarray, m: int, n: int, k: int) -> np.ndarray:
    """gemm_q4_k / gemm_q6_k / gemm_q8_0: W [m][k] blocks, X fp32 [n][k] -> Y [n][m]."""
    y = np.full((n, m), np.nan, dtype=np.float32)
    fn(lib, prefix, name)(fptr(y), vptr(w), fptr(np.ascontiguousarray(x.reshape(-1))), C.c_int(m), C.c_int(n), C.c_int(k))
    return y


def gemv_contract(lib, prefix, w: np.ndarray, x: np.ndarray, m: int, k: int) -> np.ndarray:
    y = np.full(m, np.nan, dtype=np.float32)
    fn(lib, prefix, "gemv_q8_0_q8_0_contract")(fptr(y), vptr(w), fptr(np.ascontiguousarray(x)), C.c_int(m), C.c_int(k))
    return y


def rope_cache_general(lib, prefix, max_seq: int, d: int, theta: float, rotary_dim: int, scaling: bytes | None, factor: float):
    rot = rotary_dim if 0 < rotary_dim <= d else d
    cos = np.zeros((max_seq, rot // 2), dtype=np.float32)
    sin = np.zeros((max_seq, rot // 2), dtype=np.float32)
    fn(lib, prefix, "rope_precompute_cache")(fptr(cos), fptr(sin), C.c_int(max_seq), C.c_int(d), C.c_float(theta), C.c_int(rotary_dim),
                                             C.c_char_p(scaling), C.c_float(factor))
    return cos, sin


def rope_qk_pairwise(lib, prefix, q, k, cos, sin, pos: int, hd: int, rotary_dim: int):
    """q [H, tokens, ad], k [Hkv, tokens, ad]; pairs (2i, 2i+1) of the first rotary_dim elements rotated in place."""
    fn(lib, prefix, "rope_forward_qk_pairwise_with_rotary_dim")(
        fptr(q), fptr(k), fptr(cos), fptr(sin), C.c_int(q.shape[0]), C.c_int(k.shape[0]), C.c_int(q.shape[1]), C.c_int(hd),
        C.c_int(q.shape[2]), C.c_int(pos), C.c_int(rotary_dim))


def add_inplace(lib, prefix, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    out = a.copy()
    fn(lib, prefix, "add_inplace_f32")(fptr(out), fptr(b), C.c_size_t(out.size))
    return out


def logits_copy(lib, prefix, src: np.ndarray, rows: int, position: int) -> np.ndarray:
    dst = np.zeros((rows, src.size), dtype=np.float32)
    fn(lib, prefix, "logits_copy_to_position")(fptr(src), fptr(dst), C.c_int(position), C.c_int(src.size))
    return dst


F16KV_DECODE = [(8, 2, 128, 300, 320, 81), (14, 2, 64, 70, 96, 82), (4, 4, 64, 1, 8, 83)]      # heads, kv heads, d, tokens, capacity, seed
F16KV_PREFILL = [(8, 4, 64, 64, 37, 40, 84), (4, 2, 72, 64, 9, 9, 85)]                          # heads, kv heads, ad, head_dim, tokens, kv stride, seed


def boundary_outputs(lib, prefix: str) -> dict[str, np.ndarray]:
    """Seeded cases for the entry points above; run through the reference (golden file), the oracle and the CUDA library."""
    out: dict[str, np.ndarray] = {}
    for fmt, m, n, k, seed in [("q4_k", 3, 9, 512, 71), ("q6_k", 2, 7, 512, 72), ("q8_0", 3, 6, 160, 73)]:
        w = synth.make_weights(fmt, n, k, seed)
        a = synth.make_x(k, seed, rows=m).reshape(m, k)
        bias = np.random.default_rng(seed).standard_normal(n).astype(np.float32)
        out[f"gemm_nt_f32_{fmt}"] = gemm_nt_f32(lib, prefix, f"gemm_nt_{fmt}", a, w, bias, m, n, k)
        out[f"gemm_f32_{fmt}"] = gemm_f32(lib, prefix, f"gemm_{fmt}", w, a, n, m, k)
    w = synth.make_weights("q6_k", 5, 768, 74)
    a = synth.make_x(768, 74, rows=2).reshape(2, 768)
    out["gemm_nt_q6_k_sse"] = gemm_nt_f32(lib, prefix, "gemm_nt_q6_k_sse", a, w, None, 2, 5, 768)
    w = synth.make_weights("q8_0", 11, 896, 75)
    x = synth.make_x(896, 75)
    out["gemv_contract"] = gemv_contract(lib, prefix, w, x, 11, 896)
    a = synth.make_x(896, 76, rows=3).reshape(3, 896)
    bias = np.random.default_rng(76).standard_normal(11).astype(np.float32)
    out["gemm_nt_contract"] = gemm_nt_f32(lib, prefix, "gemm_nt_q8_0_q8_0_contract", a, w, bias, 3, 11, 896)

    rng = np.random.default_rng(77)
    cos, sin = rope_cache_general(lib, prefix, 48, 128, 5.0e5, 0, None, 1.0)
    out["rope_general_cos"], out["rope_general_sin"] = cos, sin
    cos2, sin2 = rope_cache_general(lib, prefix, 33, 64, 1.0e4, 32, b"linear", 4.0)
    out["rope_linear_cos"], out["rope_linear_sin"] = cos2, sin2
    q = rng.standard_normal((8, 3, 128)).astype(np.float32)
    k = rng.standard_normal((2, 3, 128)).astype(np.float32)
    rope_qk_pairwise(lib, prefix, q, k, cos, sin, pos=41, hd=128, rotary_dim=0)
    out["rope_pair_q"], out["rope_pair_k"] = q, k
    q = rng.standard_normal((4, 2, 72)).astype(np.float32)          # aligned head 72 > head_dim 64 > rotary 32: the tail is untouched
    k = rng.standard_normal((4, 2, 72)).astype(np.float32)
    rope_qk_pairwise(lib, prefix, q, k, cos2, sin2, pos=30, hd=64, rotary_dim=32)
    out["rope_pair_partial_q"], out["rope_pair_partial_k"] = q, k

    for i, (heads, kv_heads, d, tokens, cap, seed) in enumerate(F16KV_DECODE):
        q, kc, vc = attention_inputs(seed, heads, kv_heads, d, tokens, cap)
        out[f"attn_f16kv_decode_{i}"] = attention_decode_f16kv(lib, prefix, q, kc, vc, tokens)
    for i, (heads, kv_heads, ad, hd, tokens, stride, seed) in enumerate(F16KV_PREFILL):
        q, k, v = prefill_attention_inputs(seed, heads, kv_heads, ad, hd, tokens, stride)
        out[f"attn_f16kv_prefill_{i}"] = attention_prefill_f16kv(lib, prefix, q, k, v, hd)

    a = rng.standard_normal(1000).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    out["add_inplace"] = add_inplace(lib, prefix, a, b)
    out["logits_copy"] = logits_copy(lib, prefix, rng.standard_normal(77).astype(np.float32), 4, 2)
    return out


# Outputs the oracle reproduces bit for bit (the reference computes them in scalar order, or they are integer work plus one fp32 product per block)
BOUNDARY_BIT_EXACT = ("gemm_nt_f32_q6_k", "gemm_f32_q6_k", "add_inplace", "logits_copy", "gemv_contract", "gemm_nt_contract", "rope_", "attn_f16kv_")

# ----------------------------------------------------------------------------- the golden case list

GOLDEN_GEMV = [  # fmt, M, K, K_valid, seed
    ("q4_k", 12, 1024, 896, 11),
    ("q4_k", 5, 2048, None, 12),
    ("q6_k", 12, 1024, 896, 13),
    ("q6_k", 3, 4864, None, 14),     # 19 superblocks per row: rows are only 2-byte aligned
    ("q8_0", 9, 896, None, 15),      # 28 blocks per row: rows are 8-byte aligned
    ("q8_0", 4, 4096, None, 16),
]
GOLDEN_ATTN = [  # heads, kv_heads, d, tokens, capacity, seed
    (14, 2, 64, 70, 96, 21),
    (8, 2, 128, 45, 64, 22),
    (4, 4, 64, 1, 8, 23),
]


def golden_outputs(lib, prefix: str) -> dict[str, np.ndarray]:
    """Run every golden case through `lib` and return name -> output array."""
    out: dict[str, np.ndarray] = {}
    xe = q8k_edge_input()
    out["q8k_edge"] = quantize_q8_k(lib, prefix, xe)
    x = synth.make_x(2048, seed=1)
    out["q8k_rand"] = quantize_q8_k(lib, prefix, x)
    out["q8k_batch"] = quantize_q8_k(lib, prefix, synth.make_x(512, seed=2, rows=3), rows=3)
    out["q80_rand"] = quantize_q8_0(lib, prefix, synth.make_x(896, seed=3))
    x0 = synth.make_x(128, seed=4).copy()
    x0[32:64] = 0.0
    out["q80_zero_block"] = quantize_q8_0(lib, prefix, x0)

    for fmt, m, k, kv, seed in GOLDEN_GEMV:
        w = synth.make_weights(fmt, m, k, seed)
        x = synth.make_x(k, seed, k_valid=kv)
        xq = quantize_act(lib, prefix, fmt, x)
        tag = f"{fmt}_{m}x{k}"
        ref_symbol = {"q4_k": "gemv_q4_k_q8_k_ref", "q6_k": "gemv_q6_k_q8_k_ref", "q8_0": "gemv_q8_0_q8_0"}[fmt]
        if prefix:  # the oracle exports one scalar-order function per format
            ref_symbol = GEMV_SYMBOL[fmt]
        out[f"gemv_ref_{tag}"] = gemv(lib, prefix, fmt, w, xq, m, k, ref_symbol)
        if not prefix:
            out[f"gemv_dispatch_{tag}"] = gemv(lib, prefix, fmt, w, xq, m, k)
        out[f"dequant_{tag}"] = dequant_row(lib, prefix, fmt, w, k)
        if fmt == "q8_0":
            out[f"gemv_f32_{tag}"] = gemv_f32(lib, prefix, fmt, w, x, m, k, "gemv_q8_0" if prefix else "gemv_q8_0_ref")

    for fmt, m, n, k, seed in [("q4_k", 3, 7, 512, 31), ("q6_k", 2, 5, 512, 32), ("q8_0", 3, 6, 128, 33)]:
        w = synth.make_weights(fmt, n, k, seed)
        a = synth.make_x(k, seed, rows=m)
        aq = quantize_act(lib, prefix, fmt, a, rows=m)
        bias = np.random.default_rng(seed).standard_normal(n).astype(np.float32)
        out[f"gemm_nt_{fmt}"] = gemm_nt(lib, prefix, fmt, aq, w, bias, m, n, k)

    for heads, kvh, d, tokens, cap, seed in GOLDEN_ATTN:
        q, kc, vc = attention_inputs(seed, heads, kvh, d, tokens, cap)
        out[f"attn_{heads}_{kvh}_{d}_{tokens}"] = attention_decode(lib, prefix, q, kc, vc, tokens)

    heads, kvh, d, tokens, cap, seed = GOLDEN_ATTN[0]
    q, kc, vc = attention_inputs(seed, heads, kvh, d, tokens, cap)
    out[f"attn_f16cache_{heads}_{kvh}_{d}_{tokens}"] = attention_decode_f16cache(lib, prefix, q, kc.astype(np.float16).view(np.uint16),
                                                                                  vc.astype(np.float16).view(np.uint16), tokens)
    kc16, vc16 = np.zeros((2, 16, 64), np.uint16), np.zeros((2, 16, 64), np.uint16)
    r16 = np.random.default_rng(43)
    kv_cache_store_f16(lib, prefix, kc16, vc16, (r16.standard_normal((2, 64)) * 100).astype(np.float32), r16.standard_normal((2, 64)).astype(np.float32), pos=9)
    out["kv_store_f16_k"], out["kv_store_f16_v"] = kc16, vc16

    for heads, kvh, ad, hd, tokens, stride, seed in GOLDEN_PREFILL_ATTN:
        q, k, v = prefill_attention_inputs(seed, heads, kvh, ad, hd, tokens, stride)
        out[f"prefill_attn_{heads}_{kvh}_{ad}_{hd}_{tokens}"] = attention_prefill(lib, prefix, q, k, v, hd, True)

    rng = np.random.default_rng(41)
    cos, sin = rope_cache(lib, prefix, 40, 64, 1.0e6)
    out["rope_cos"], out["rope_sin"] = cos, sin
    q = rng.standard_normal((14, 1, 64)).astype(np.float32)
    k = rng.standard_normal((2, 1, 64)).astype(np.float32)
    rope_qk(lib, prefix, q, k, cos, sin, pos=37)
    out["rope_q"], out["rope_k"] = q, k

    x = np.zeros((2, 1024), dtype=np.float32)
    x[:, :896] = rng.standard_normal((2, 896)).astype(np.float32)
    x[:, 896:] = 5.0  # garbage in the padding must not reach the statistics and must come out zero
    gamma = (1.0 + 0.1 * rng.standard_normal(1024)).astype(np.float32)
    out["rmsnorm"] = rmsnorm(lib, prefix, x, gamma, 896, 1.0e-6)
    out["swiglu"] = swiglu(lib, prefix, (3.0 * rng.standard_normal((2, 2 * 304))).astype(np.float32), 304)
    if hasattr(lib, prefix + "residual_add_token_major") or hasattr(lib, "ck_residual_add_token_major"):
        out["residual"] = residual_add(lib, prefix, x, x[::-1].copy())

    kc = np.zeros((2, 16, 64), dtype=np.float32)
    vc = np.zeros((2, 16, 64), dtype=np.float32)
    kv_cache_store(lib, prefix, kc, vc, rng.standard_normal((2, 64)).astype(np.float32),
                   rng.standard_normal((2, 64)).astype(np.float32), pos=5)
    out["kv_store_k"], out["kv_store_v"] = kc, vc

    for fmt, embed, aligned, seed in [("q4_k", 896, 1024, 51), ("q6_k", 512, 512, 52), ("q8_0", 896, 896, 53)]:
        table = synth.make_weights(fmt, 20, aligned, seed)
        out[f"embed_{fmt}"] = embedding(lib, prefix, fmt, [3, 19, 25, -1], table, 20, embed, aligned)
    return out


# Outputs for which the oracle keeps the reference's fp32 evaluation order and must match bit for bit.
BIT_EXACT = ("q8k_", "q80_", "gemv_ref_q4_k", "gemv_ref_q6_k", "gemv_ref_q8_0", "gemv_f32_", "dequant_", "gemm_nt_q4_k",
             "gemm_nt_q8_0", "kv_store", "residual", "embed_", "rope_cos", "rope_sin")
