"""Writes a small GGUF file for the loader tests: two MoE layers with the same expert bytes (layer 0
with separate gate / up banks, layer 1 with the fused gate_up tensor), router, shared expert and its
admission gate, and one Llama-style attention projection. Returns the host arrays that went in."""

import numpy as np

from mylocal_llm_b200.quantize import random_packed

E, D, F, K = 6, 512, 256, 2
TYPES = ("Q4_K", "Q4_K", "Q6_K")


def write_moe_gguf(path, seed=0):
    from gguf import GGMLQuantizationType as QT
    from gguf import GGUFWriter
    rng = np.random.default_rng(seed)
    writer = GGUFWriter(str(path), "qwen3next")
    writer.add_uint32("qwen3next.block_count", 2)
    writer.add_uint32("qwen3next.embedding_length", D)
    writer.add_uint32("qwen3next.expert_count", E)
    writer.add_uint32("qwen3next.expert_used_count", K)
    writer.add_float32("qwen3next.attention.layer_norm_rms_epsilon", 1e-5)
    arrays = {}

    def add_packed(name, raw2d, fmt):
        writer.add_tensor(name, raw2d, raw_dtype=getattr(QT, fmt))
        arrays[name] = raw2d.reshape(-1).copy()

    def random_bank(shape, fmt, s):
        w = random_packed(fmt, shape, seed=s, d=1.0 / 256, dmin=1.0 / 512)
        rows = int(np.prod(shape[:-1]))
        return np.asarray(w.data).reshape(shape[:-1] + (w.nbytes // rows,)).copy()

    gate = random_bank((E, F, D), TYPES[0], 1)
    up = random_bank((E, F, D), TYPES[1], 2)
    down = random_bank((E, D, F), TYPES[2], 3)
    shared = [random_bank(shape, fmt, 4 + i) for i, (shape, fmt) in
              enumerate(zip(((F, D), (F, D), (D, F)), TYPES))]
    router = rng.normal(0, 0.3, (E, D)).astype(np.float32)
    shexp_gate = rng.normal(0, 0.1, (D,)).astype(np.float32)
    for layer in range(2):
        stem = f"blk.{layer}."
        if layer == 0:
            add_packed(stem + "ffn_gate_exps.weight", gate, TYPES[0])
            add_packed(stem + "ffn_up_exps.weight", up, TYPES[1])
        else:
            add_packed(stem + "ffn_gate_up_exps.weight", np.concatenate([gate, up], axis=1), TYPES[0])
        add_packed(stem + "ffn_down_exps.weight", down, TYPES[2])
        writer.add_tensor(stem + "ffn_gate_inp.weight", router)
        writer.add_tensor(stem + "ffn_gate_inp_shexp.weight", shexp_gate)
        for name, raw, fmt in zip(("ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight"),
                                  shared, TYPES):
            add_packed(stem + name, raw, fmt)
    add_packed("blk.0.attn_q.weight", random_bank((256, 512), "Q8_0", 50), "Q8_0")
    writer.write_header_to_file()
    writer.write_kv_data_to_file()
    writer.write_tensors_to_file()
    writer.close()
    arrays.update(gate=gate, up=up, down=down, router=router, shexp_gate=shexp_gate, shared=shared)
    return arrays
