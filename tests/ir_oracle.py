"""A CPU interpreter of the reference's lowered call IR (lowered-ir-v3, decode mode) over the oracle's kernels: every op's `function` is
looked up in the oracle library (prefix oracle_) or in the reference build itself (no prefix) and called with the arguments the IR
lists, in the IR's order.  This is what the generated C of version/v7/scripts/codegen_v7.py:569-931 does, one call per op; it is the
checker for the device executor of the same files."""
from __future__ import annotations

import ctypes as C
import json
import struct

import numpy as np

FLOAT_ARGS = {"eps"}


def read_map(path):
    out = {}
    for line in open(path):
        if line.startswith("#") or not line.strip():
            continue
        name, dtype, off, size, _ = line.strip().split("|")
        out[name] = (dtype, int(off, 0), int(size, 0))
    return out


class IrCpuModel:
    def __init__(self, call_json, bump_path, map_path, lib, prefix="oracle_"):
        self.doc = json.load(open(call_json))
        assert self.doc["format"] == "lowered-ir-v3" and self.doc["mode"] == "decode" and not self.doc["errors"]
        self.lib, self.prefix = lib, prefix
        cfg = self.doc["config"]
        self.cfg = cfg
        self.vocab, self.max_seq = cfg["vocab_size"], cfg.get("max_seq_len", cfg["context_length"])
        raw = open(bump_path, "rb").read()
        fmap = read_map(map_path)
        self.weights = {}
        for e in self.doc["memory"]["weights"]["entries"]:
            _, off, size = fmap[e["name"]]
            assert size == e["size"], e["name"]
            self.weights[e["name"]] = np.frombuffer(raw, np.uint8, size, off).copy()
        self.buffers = {b["name"]: np.zeros(b["size"] + 64, np.uint8) for b in self.doc["memory"]["activations"]["buffers"]}
        self.kv = self.buffers["kv_cache"][: self.buffers["kv_cache"].size // 4 * 4].view(np.float32)
        rotary = cfg.get("rotary_dim") or cfg["head_dim"]
        half = self.max_seq * (rotary // 2)
        rope = self.buffers["rope_cache"][: 8 * half].view(np.float32)
        self.cos, self.sin = rope[:half], rope[half:]
        scaling = cfg.get("rope_scaling_type", "none") or "none"
        fn = getattr(lib, prefix + "rope_precompute_cache")
        fn.restype = None
        fn(self._p(self.cos), self._p(self.sin), C.c_int(self.max_seq), C.c_int(cfg["head_dim"]), C.c_float(cfg["rope_theta"]), C.c_int(rotary),
           C.c_char_p(scaling.encode()) if scaling != "none" else None, C.c_float(cfg.get("rope_scaling_factor", 1.0)))
        self.pos = 0

    @staticmethod
    def _p(a):
        return C.c_void_p(a.ctypes.data)

    def _arg(self, op, a):
        src, name = a["source"], a["name"]
        if src == "null":
            return None
        if "weight_ref" in a:
            return self._p(self.weights[a["weight_ref"]])
        if "buffer_ref" in a:
            return self._p(self.buffers[a["buffer_ref"]])
        if src == "runtime:rope_cos":
            return self._p(self.cos)
        if src == "runtime:rope_sin":
            return self._p(self.sin)
        if src in ("runtime:kv_cache_k_layer", "runtime:kv_cache_v_layer"):
            per = self.cfg["num_kv_heads"] * self.max_seq * self.cfg["head_dim"]
            idx = op["layer"] * 2 + (1 if src.endswith("v_layer") else 0)
            return C.c_void_p(self.kv.ctypes.data + 4 * idx * per)
        if src == "runtime:pos":
            return C.c_int(self.pos)
        if src == "runtime:kv_tokens":
            return C.c_int(self.pos + 1)
        if src == "runtime:layer":
            return C.c_int(op["layer"])
        if src.startswith(("dim:", "const:")):
            return C.c_float(float(a["expr"])) if name in FLOAT_ARGS else C.c_int(int(float(a["expr"])))
        raise ValueError(f"op {op['function']}: cannot bind {name} from {src}")

    def decode(self, token: int) -> np.ndarray:
        self.buffers["token_ids"][:4] = np.frombuffer(struct.pack("<i", token), np.uint8)
        for op in self.doc["operations"]:
            f = op["function"]
            if f == "memcpy":
                args = {a["name"]: a for a in op["args"]}
                n = int(args["size"]["expr"])
                self.buffers[args["dst"]["buffer_ref"]][:n] = self.buffers[args["src"]["buffer_ref"]][:n]
                continue
            if f == "ck_residual_add_token_major" and not hasattr(self.lib, self.prefix + f):
                # lives in the reference's orchestration file, which the reference build under oracle/_ref leaves out; one fp32 add per element
                args = {a["name"]: a for a in op["args"]}
                n = 4 * int(args["tokens"]["expr"]) * int(args["aligned_embed_dim"]["expr"])
                a_, b_ = (self.buffers[args[k]["buffer_ref"]][:n].view(np.float32) for k in ("a", "b"))
                self.buffers[args["out"]["buffer_ref"]][:n].view(np.float32)[:] = a_ + b_
                continue
            fn = getattr(self.lib, self.prefix + f)
            fn.restype = None
            fn(*[self._arg(op, a) for a in op["args"]])
        self.pos += 1
        return self.buffers["logits"][: 4 * self.vocab].view(np.float32).copy()
