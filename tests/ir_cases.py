"""Model shapes of the lowered-IR fixtures (tests/golden/ir/call_<name>.json) and the manifest the reference's IR builder wants for them.
Shared by the script that generates the fixtures with the reference's own build_ir_v7.py and by the tests that replay them."""
from __future__ import annotations

import os

FMT_NAME = {0: "q4_k", 1: "q6_k", 2: "q8_0", 3: "q5_0"}

_KQUANT = dict(embed_dim=512, num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1024, num_layers=2, vocab_size=777,
               max_seq_len=64, rms_eps=1e-5, rope_theta=5.0e5, fmt_q=0, fmt_k=0, fmt_v=1, fmt_o=0, fmt_gate_up=0, fmt_down=1, fmt_lm_head=1)
_Q5_0 = dict(embed_dim=384, num_heads=6, num_kv_heads=2, head_dim=64, intermediate_size=768, num_layers=2, vocab_size=500,
             max_seq_len=96, rms_eps=1e-6, rope_theta=1.0e6, fmt_q=3, fmt_k=3, fmt_v=3, fmt_o=3, fmt_gate_up=3, fmt_down=1, fmt_lm_head=2)

# name -> (template the reference lowers with, model shape, seed of the weights)
CASES = {
    "llama_kquant": ("llama", _KQUANT, 31),      # pair-rotated RoPE, fp16-rounded attention (the llama template's kernels)
    "qwen2_kquant": ("qwen2", _KQUANT, 32),      # half-rotated RoPE, fp32 flash decode attention
    "qwen2_q5_0": ("qwen2", _Q5_0, 33),          # Q5_0 projections and a Q8_0 head: Q8_0 activations
}


def fixture_path(name: str) -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ir", f"call_{name}.json")


def manifest_dict(arch: str, c: dict, entries) -> dict:
    """What convert_gguf_to_bump_v7.py writes as weights_manifest.json (version/v7/scripts/convert_gguf_to_bump_v7.py:3410-3520), reduced to
    the keys build_ir_v7.py reads: config, quant_summary, the dimensions and the tensor entries."""
    cfg = {"model": arch, "embed_dim": c["embed_dim"], "attn_out_dim": c["num_heads"] * c["head_dim"], "num_layers": c["num_layers"],
           "num_heads": c["num_heads"], "num_kv_heads": c["num_kv_heads"], "head_dim": c["head_dim"], "intermediate_size": c["intermediate_size"],
           "context_length": c["max_seq_len"], "rope_theta": c["rope_theta"], "rotary_dim": c["head_dim"], "rope_scaling_type": "none",
           "rope_scaling_factor": 1.0, "rope_original_context_length": 0, "rope_beta_fast": 32.0, "rope_beta_slow": 1.0, "rope_attn_factor": 1.0,
           "vocab_size": c["vocab_size"], "rms_eps": c["rms_eps"], "tie_word_embeddings": True}
    quant = {"token_emb": FMT_NAME[c["fmt_lm_head"]], "lm_head": FMT_NAME[c["fmt_lm_head"]]}
    for layer in range(c["num_layers"]):
        quant[f"layer.{layer}"] = {"wq": FMT_NAME[c["fmt_q"]], "wk": FMT_NAME[c["fmt_k"]], "wv": FMT_NAME[c["fmt_v"]], "wo": FMT_NAME[c["fmt_o"]],
                                   "w1": FMT_NAME[c["fmt_gate_up"]], "w2": FMT_NAME[c["fmt_down"]]}
    return {"version": 5, "model": arch, "config": cfg, "quant_summary": quant, "num_layers": c["num_layers"], "embed_dim": c["embed_dim"],
            "num_heads": c["num_heads"], "num_kv_heads": c["num_kv_heads"], "head_dim": c["head_dim"], "intermediate_size": c["intermediate_size"],
            "vocab_size": c["vocab_size"], "context_length": c["max_seq_len"], "has_attention_biases": False, "has_qk_norm": False, "num_merges": 0,
            "total_vocab_bytes": 0, "entries": [{"name": n, "dtype": t, "file_offset": o, "size": s} for n, t, o, s in entries]}
