"""Loader of the reference-generated Llama fixture (tests/golden/llama_golden.npz)."""

from pathlib import Path

import numpy as np

# the configuration tests/golden/make_golden.py used (a two-layer Llama with head dimension 64)
LLAMA_CONFIG = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64, vocab_size=256, max_position_embeddings=64,
                    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)


def expected_shapes(cfg):
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (v, d), "lm_head.weight": (v, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (q, d), p + "self_attn.k_proj.weight": (kv, d),
                       p + "self_attn.v_proj.weight": (kv, d), p + "self_attn.o_proj.weight": (d, q),
                       p + "mlp.gate_proj.weight": (f, d), p + "mlp.up_proj.weight": (f, d),
                       p + "mlp.down_proj.weight": (d, f)})
    return shapes


def load_llama_golden():
    """(weights: HF name -> (bytes, shape, "Q8_0") or FP32 norm vector, prompt [1,T], greedy tokens [3], logits [4,V])."""
    shapes = expected_shapes(LLAMA_CONFIG)
    weights = {}
    with np.load(Path(__file__).resolve().parent / "golden" / "llama_golden.npz") as data:
        for key in data.files:
            if key.startswith("q8:"):
                weights[key[3:]] = (data[key], shapes[key[3:]], "Q8_0")
            elif key.startswith("norm:"):
                weights[key[5:]] = data[key]
        return weights, data["prompt"], data["greedy_tokens"], data["logits"]
