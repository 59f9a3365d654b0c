"""CPU decode step assembled from the oracle's kernels in the order the reference's generated
ck_decode() issues them (version/v7/scripts/codegen_v7.py:886-931); the checker for the
device-resident step executor.  One sequence at a time; weights and caches are numpy arrays."""
from __future__ import annotations

import ctypes as C

import numpy as np

import cases

synth = cases.synth
FMT = {0: "q4_k", 1: "q6_k", 2: "q8_0", 3: "q5_0"}
T = dict(LN1=0, WQ=1, WK=2, WV=3, WO=4, LN2=5, W1=6, W2=7, FINAL_GAMMA=100, LM_HEAD=101, EMBEDDING=102)


def round256(v):
    return (v + 255) // 256 * 256


def cols_for(fmt, k):
    return (k + 31) // 32 * 32 if fmt in (2, 3) else round256(k)


def embed_row(lib, fmt, table, token, vocab, d, table_cols, da):
    """One embedding row, padded with zeros to da floats.  The reference's lookup takes its table row stride from the aligned width it is given
    (src/kernels/embedding_kernels.c:155), so it is called with the table's own row width."""
    x = np.zeros(da, np.float32)
    x[:table_cols] = cases.embedding(lib, "oracle_", FMT[fmt], [token], table, vocab, d, table_cols)[0]
    return x


class CpuModel:
    """Whole (unsharded) model on the host: random weights in the reference's block formats."""

    def __init__(self, cfg: dict, seed: int, kv_f16: bool = False):
        """kv_f16: keep the caches as IEEE halves (kv_cache_store_f16 + the _f16cache decode attention of the reference)."""
        self.cfg = cfg
        self.kv_f16 = kv_f16
        D, H, Hkv, d, I, L, V = (cfg[k] for k in ("embed_dim", "num_heads", "num_kv_heads", "head_dim", "intermediate_size", "num_layers", "vocab_size"))
        self.Da, self.A, self.Aa = round256(D), H * d, round256(H * d)
        rng = np.random.default_rng(seed)
        s = seed * 100
        self.layers = []
        for _ in range(L):
            lay = {}
            lay["LN1"] = (1.0 + 0.1 * rng.standard_normal(self.Da)).astype(np.float32)
            lay["LN2"] = (1.0 + 0.1 * rng.standard_normal(self.Da)).astype(np.float32)
            for name, fmt, rows, k in (("WQ", cfg["fmt_q"], H * d, D), ("WK", cfg["fmt_k"], Hkv * d, D), ("WV", cfg["fmt_v"], Hkv * d, D),
                                       ("WO", cfg["fmt_o"], D, H * d), ("W1", cfg["fmt_gate_up"], 2 * I, D), ("W2", cfg["fmt_down"], D, I)):
                s += 1
                lay[name] = (fmt, rows, cols_for(fmt, k), synth.make_weights(FMT[fmt], rows, cols_for(fmt, k), seed=s))
            self.layers.append(lay)
        self.final_gamma = (1.0 + 0.1 * rng.standard_normal(self.Da)).astype(np.float32)
        fmt = cfg["fmt_lm_head"]
        self.lm_head = (fmt, V, cols_for(fmt, D), synth.make_weights(FMT[fmt], V, cols_for(fmt, D), seed=s + 1))
        S = cfg["max_seq_len"]
        self.kc = np.zeros((L, Hkv, S, d), np.float32)
        self.vc = np.zeros((L, Hkv, S, d), np.float32)

    def prefill_kv(self, tokens: int, seed: int):
        rng = np.random.default_rng(seed)
        self.kc[:, :, :tokens] = rng.standard_normal(self.kc[:, :, :tokens].shape).astype(np.float32)
        self.vc[:, :, :tokens] = rng.standard_normal(self.vc[:, :, :tokens].shape).astype(np.float32)
        if self.kv_f16:
            self.kc16 = self.kc.astype(np.float16).view(np.uint16)
            self.vc16 = self.vc.astype(np.float16).view(np.uint16)

    def _matvec(self, lib, w, x_row):
        fmt, rows, cols, data = w
        x = np.zeros(cols, np.float32)
        x[:min(cols, x_row.size)] = x_row[:cols]
        xq = cases.quantize_act(lib, "oracle_", FMT[fmt], x)
        return cases.gemv(lib, "oracle_", FMT[fmt], data, xq, rows, cols)

    def decode(self, lib, token: int, pos: int) -> np.ndarray:
        c = self.cfg
        D, H, Hkv, d, I = c["embed_dim"], c["num_heads"], c["num_kv_heads"], c["head_dim"], c["intermediate_size"]
        efmt, _, ecols, edata = self.lm_head
        x = embed_row(lib, efmt, edata, token, c["vocab_size"], D, ecols, self.Da)
        cos, sin = cases.rope_cache(lib, "oracle_", c["max_seq_len"], d, c["rope_theta"])
        for l, lay in enumerate(self.layers):
            h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), lay["LN1"], D, c["rms_eps"])[0]
            q = self._matvec(lib, lay["WQ"], h).reshape(H, 1, d).copy()
            k = self._matvec(lib, lay["WK"], h).reshape(Hkv, 1, d).copy()
            v = self._matvec(lib, lay["WV"], h).reshape(Hkv, d).copy()
            cases.rope_qk(lib, "oracle_", q, k, cos, sin, pos)
            if self.kv_f16:
                cases.kv_cache_store_f16(lib, "oracle_", self.kc16[l], self.vc16[l], np.ascontiguousarray(k.reshape(Hkv, d)), v, pos)
                att = cases.attention_decode_f16cache(lib, "oracle_", np.ascontiguousarray(q.reshape(H, d)), self.kc16[l], self.vc16[l], pos + 1).reshape(-1)
            else:
                cases.kv_cache_store(lib, "oracle_", self.kc[l], self.vc[l], np.ascontiguousarray(k.reshape(Hkv, d)), v, pos)
                att = cases.attention_decode(lib, "oracle_", np.ascontiguousarray(q.reshape(H, d)), self.kc[l], self.vc[l], pos + 1).reshape(-1)
            o = self._matvec(lib, lay["WO"], att)
            x[:D] += o
            h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), lay["LN2"], D, c["rms_eps"])[0]
            gu = self._matvec(lib, lay["W1"], h)
            mm = cases.swiglu(lib, "oracle_", gu.reshape(1, -1), I)[0]
            x[:D] += self._matvec(lib, lay["W2"], mm)
        h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), self.final_gamma, D, c["rms_eps"])[0]
        return self._matvec(lib, self.lm_head, h)


# the ctypes view of the executor's C interface lives in the package (bench.py uses it too)
_model_api = cases.load_package().model_api
CfgStruct, make_cfg, bind_model_api = _model_api.CfgStruct, _model_api.make_cfg, _model_api.bind_model_api


def upload_whole_model(lib, handle, cpu: CpuModel, batch: int):
    """tp_size == 1: tensors go up as they are; the KV cache of sequence 0 is replicated to every sequence."""
    for l, lay in enumerate(cpu.layers):
        for name in ("LN1", "LN2"):
            assert lib.ckb200_model_upload_tensor(handle, l, T[name], cases.vptr(lay[name]), lay[name].nbytes) == 0
        for name in ("WQ", "WK", "WV", "WO", "W1", "W2"):
            data = lay[name][3]
            assert lib.ckb200_model_upload_tensor(handle, l, T[name], cases.vptr(data), data.nbytes) == 0, (l, name)
    assert lib.ckb200_model_upload_tensor(handle, -1, T["FINAL_GAMMA"], cases.vptr(cpu.final_gamma), cpu.final_gamma.nbytes) == 0
    assert lib.ckb200_model_upload_tensor(handle, -1, T["LM_HEAD"], cases.vptr(cpu.lm_head[3]), cpu.lm_head[3].nbytes) == 0
    for l in range(len(cpu.layers)):
        for is_v, cache in ((0, cpu.kc16), (1, cpu.vc16)) if cpu.kv_f16 else ((0, cpu.kc), (1, cpu.vc)):
            base = lib.ckb200_model_kv_device(handle, l, is_v)
            slab = np.ascontiguousarray(cache[l])
            for b in range(batch):
                assert lib.ckb200_copy_to_device(C.c_void_p(base + b * slab.nbytes), cases.vptr(slab), slab.nbytes) == 0


# ----------------------------------------------------------------------------- tensor-parallel sharding

BLOCK = {0: (256, 144), 1: (256, 210), 2: (32, 34), 3: (32, 22)}     # fmt -> (elements, bytes) per block


def _rows(w, r0, r1):
    fmt, rows, cols, data = w
    rb = data.size // rows
    return (fmt, r1 - r0, cols, np.ascontiguousarray(data.reshape(rows, rb)[r0:r1]).reshape(-1))


def _cols(w, c0, c1):
    """Input columns [c0, c1) of every row; both must fall on block boundaries (256 for the K-quants)."""
    fmt, rows, cols, data = w
    be, bb = BLOCK[fmt]
    assert c0 % be == 0 and c1 % be == 0
    blocks = data.reshape(rows, cols // be, bb)[:, c0 // be:c1 // be]
    return (fmt, rows, c1 - c0, np.ascontiguousarray(blocks).reshape(-1))


def shard_layer(cfg, lay, rank, tp):
    """Column-parallel q/k/v/gate/up (whole heads, matching gate/up rows), row-parallel o/down split at block boundaries."""
    H, Hkv, d, I = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["intermediate_size"]
    Hl, Hkvl, Il = H // tp, Hkv // tp, I // tp
    out = {"LN1": lay["LN1"], "LN2": lay["LN2"]}
    out["WQ"] = _rows(lay["WQ"], rank * Hl * d, (rank + 1) * Hl * d)
    out["WK"] = _rows(lay["WK"], rank * Hkvl * d, (rank + 1) * Hkvl * d)
    out["WV"] = _rows(lay["WV"], rank * Hkvl * d, (rank + 1) * Hkvl * d)
    g = _rows(lay["W1"], rank * Il, (rank + 1) * Il)
    u = _rows(lay["W1"], I + rank * Il, I + (rank + 1) * Il)
    out["W1"] = (g[0], 2 * Il, g[2], np.concatenate([g[3], u[3]]))
    out["WO"] = _cols(lay["WO"], rank * Hl * d, (rank + 1) * Hl * d)
    out["W2"] = _cols(lay["W2"], rank * Il, (rank + 1) * Il)
    return out


class TpShard:
    """One rank's view of a CpuModel: sharded layers, its own KV heads, the whole LM head."""

    def __init__(self, cpu: CpuModel, rank: int, tp: int):
        c = cpu.cfg
        assert c["num_heads"] % tp == 0 and c["num_kv_heads"] % tp == 0 and c["intermediate_size"] % tp == 0
        self.cpu, self.rank, self.tp = cpu, rank, tp
        self.layers = [shard_layer(c, lay, rank, tp) for lay in cpu.layers]
        Hkvl = c["num_kv_heads"] // tp
        self.kc = np.ascontiguousarray(cpu.kc[:, rank * Hkvl:(rank + 1) * Hkvl])
        self.vc = np.ascontiguousarray(cpu.vc[:, rank * Hkvl:(rank + 1) * Hkvl])

    def decode(self, lib, token: int, pos: int, allreduce) -> np.ndarray:
        """Same op order as CpuModel.decode on this rank's shard; `allreduce(vec)` sums a vector over ranks in place."""
        cpu, c, tp = self.cpu, self.cpu.cfg, self.tp
        D, d = c["embed_dim"], c["head_dim"]
        Hl, Hkvl, Il = c["num_heads"] // tp, c["num_kv_heads"] // tp, c["intermediate_size"] // tp
        efmt, _, ecols, edata = cpu.lm_head
        x = embed_row(lib, efmt, edata, token, c["vocab_size"], D, ecols, cpu.Da)
        cos, sin = cases.rope_cache(lib, "oracle_", c["max_seq_len"], d, c["rope_theta"])
        for l, lay in enumerate(self.layers):
            h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), lay["LN1"], D, c["rms_eps"])[0]
            q = cpu._matvec(lib, lay["WQ"], h).reshape(Hl, 1, d).copy()
            k = cpu._matvec(lib, lay["WK"], h).reshape(Hkvl, 1, d).copy()
            v = cpu._matvec(lib, lay["WV"], h).reshape(Hkvl, d).copy()
            cases.rope_qk(lib, "oracle_", q, k, cos, sin, pos)
            cases.kv_cache_store(lib, "oracle_", self.kc[l], self.vc[l], np.ascontiguousarray(k.reshape(Hkvl, d)), v, pos)
            att = cases.attention_decode(lib, "oracle_", np.ascontiguousarray(q.reshape(Hl, d)), self.kc[l], self.vc[l], pos + 1).reshape(-1)
            o = cpu._matvec(lib, lay["WO"], att)
            allreduce(o)
            x[:D] += o
            h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), lay["LN2"], D, c["rms_eps"])[0]
            gu = cpu._matvec(lib, lay["W1"], h)
            mm = cases.swiglu(lib, "oracle_", gu.reshape(1, -1), Il)[0]
            dn = cpu._matvec(lib, lay["W2"], mm)
            allreduce(dn)
            x[:D] += dn
        h = cases.rmsnorm(lib, "oracle_", x.reshape(1, -1), cpu.final_gamma, D, c["rms_eps"])[0]
        return cpu._matvec(lib, cpu.lm_head, h)


def upload_shard(lib, handle, shard: TpShard, batch: int = 1):
    cpu = shard.cpu
    for l, lay in enumerate(shard.layers):
        for name in ("LN1", "LN2"):
            assert lib.ckb200_model_upload_tensor(handle, l, T[name], cases.vptr(lay[name]), lay[name].nbytes) == 0
        for name in ("WQ", "WK", "WV", "WO", "W1", "W2"):
            data = lay[name][3]
            assert lib.ckb200_model_upload_tensor(handle, l, T[name], cases.vptr(data), data.nbytes) == 0, (l, name)
    assert lib.ckb200_model_upload_tensor(handle, -1, T["FINAL_GAMMA"], cases.vptr(cpu.final_gamma), cpu.final_gamma.nbytes) == 0
    assert lib.ckb200_model_upload_tensor(handle, -1, T["LM_HEAD"], cases.vptr(cpu.lm_head[3]), cpu.lm_head[3].nbytes) == 0
    for l in range(len(shard.layers)):
        for is_v, cache in ((0, shard.kc), (1, shard.vc)):
            base = lib.ckb200_model_kv_device(handle, l, is_v)
            slab = np.ascontiguousarray(cache[l])
            for b in range(batch):
                assert lib.ckb200_copy_to_device(C.c_void_p(base + b * slab.nbytes), cases.vptr(slab), slab.nbytes) == 0
