"""Writer of small BUMPWGT5 weight files for the loader's tests, in the layout of the reference's converter
(include/ckernel_bump_v5.h:19-52; version/v7/scripts/convert_gguf_to_bump_v7.py:2826-2945, tensor order :3218-3395): 128-byte
header, 24 reserved bytes, u32 dtype-table length + table, tensors, then the JSON metadata blob and its 48-byte footer; beside it
the sidecar map the reference's C loader reads (name|dtype|file_offset|size|runtime_offset)."""
from __future__ import annotations

import hashlib
import json
import struct

import numpy as np

import step_oracle as so

DTYPE_NAME = {0: "q4_k", 1: "q6_k", 2: "q8_0", 3: "q5_0"}
DTYPE_CODE = {"fp32": 0, "q4_k": 6, "q6_k": 7, "q8_0": 9, "q5_0": 11}     # codes only label the table; the loader goes by the map


def write_bump(path, map_path, cpu: so.CpuModel, *, with_biases=True, bias_value=0.0, untied_head=False, meta=True):
    """cpu: the host model of the step oracle.  Returns the list of (name, dtype, offset, size)."""
    c = cpu.cfg
    D, H, Hkv, d, I = c["embed_dim"], c["num_heads"], c["num_kv_heads"], c["head_dim"], c["intermediate_size"]
    tensors = []

    def add(name, dtype, data):
        tensors.append((name, dtype, np.ascontiguousarray(data).view(np.uint8).reshape(-1)))

    def bias(name, n):
        if with_biases:
            add(name, "fp32", np.full(n, bias_value, np.float32))

    add("token_emb", DTYPE_NAME[cpu.lm_head[0]], cpu.lm_head[3])
    if untied_head:
        add("output.weight", DTYPE_NAME[cpu.lm_head[0]], cpu.lm_head[3])
    for l, lay in enumerate(cpu.layers):
        p = f"layer.{l}."
        add(p + "ln1_gamma", "fp32", lay["LN1"][:D])
        add(p + "ln2_gamma", "fp32", lay["LN2"][:D])
        for name, key, b, n in (("wq", "WQ", "bq", H * d), ("wk", "WK", "bk", Hkv * d), ("wv", "WV", "bv", Hkv * d), ("wo", "WO", "bo", D),
                                ("w1", "W1", "b1", 2 * I), ("w2", "W2", "b2", D)):
            add(p + name, DTYPE_NAME[lay[key][0]], lay[key][3])
            bias(p + b, n)
    add("final_ln_weight", "fp32", cpu.final_gamma[:D])
    bias("final_ln_bias", D)

    table = bytes(DTYPE_CODE[t[1]] for t in tensors)
    payload = bytearray(struct.pack("<I", len(table)) + table)
    entries = []
    for name, dtype, data in tensors:
        payload += b"\0" * (-(152 + len(payload)) % 64)                # the converter aligns every tensor to a cache line
        entries.append((name, dtype, 152 + len(payload), data.size))
        payload += data.tobytes()
    header = b"BUMPWGT5" + struct.pack("<10I", 5, 1, c["num_layers"], c["vocab_size"], D, I, c["max_seq_len"], H, Hkv, d)
    header += struct.pack("<4Q", D, d, I, c["max_seq_len"]) + struct.pack("<2I", 0, 0) + hashlib.sha256(payload).digest() + b"\0" * 8
    assert len(header) == 128
    blob = b""
    if meta:
        js = json.dumps({"format": "BUMPWGT5", "config": {"model_type": "llama", "rope_theta": c["rope_theta"], "rms_eps": c["rms_eps"],
                                                          "tie_word_embeddings": not untied_head}}).encode()
        blob = js + b"BUMPV5MD" + struct.pack("<Q", len(js)) + hashlib.sha256(js).digest()
    with open(path, "wb") as f:
        f.write(header + b"\0" * 24 + bytes(payload) + blob)
    with open(map_path, "w") as f:
        f.write("# name|dtype|file_offset|size|runtime_offset\n")
        for i, (name, dtype, off, size) in enumerate(entries):
            f.write(f"{name}|{dtype}|0x{off:x}|{size}|0x{i * 64:x}\n")
    return entries
