"""CPU restatement (NumPy, FP64) of the Llama-family decoder the reference runs for GGUF models.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing else); the product never calls it.

Follows ``mini_llm/external/llama_model.py:75-178`` (weight names and orientation: HF ``[out, in]``),
the native block it drives (pre-norm residual block: ``x += attn(norm1(x)); x += ffn(norm2(x))``,
``mini_llm/blocks/transformer_block_inference.py:344-364``), RMSNorm
(``mini_llm/ops/rmsnorm_inference.py:80-119``), rotate-half RoPE with
``theta_i = pos / base**(2i/d_head)`` (``mini_llm/ops/attention_inference.py:255-277``), causal
attention scaled by ``1/sqrt(d_head)`` with grouped KV heads, and the SwiGLU FFN
``down(silu(gate x) * (up x))``. Packed matrices enter through the bit-exact dequantiser of
``packed_oracle``.

Parity is PINNED: ``tests/test_llama_golden.py`` checks ``llama_logits`` against logits the reference's
own ``ExternalLlamaModel`` produced in this repository's build container (NumPy backend, FP32, Q8_0
weights handed over dequantised as its GGUF reader does; ``tests/golden/make_golden.py llama`` ->
``tests/golden/llama_golden.npz``): the prompt's last position and three greedy decode steps agree
within FP32 rounding (rtol 2e-4).
"""

import numpy as np

from . import packed_oracle as po


def _dense(w):
    """(data, shape, fmt) packed triple or ndarray -> float64 matrix."""
    if isinstance(w, tuple):
        data, shape, fmt = w
        return po.dequantize(data, shape, fmt).astype(np.float64)
    return np.asarray(w, dtype=np.float64)


def rope_half(x, positions, base):
    """x [T, H, Dh]; rotate-half layout."""
    d = x.shape[-1]
    half = d // 2
    inv = 1.0 / (float(base) ** (2.0 * np.arange(half) / d))
    ang = np.asarray(positions, np.float64)[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([x0 * cos - x1 * sin, x0 * sin + x1 * cos], axis=-1)


def llama_logits(weights, config, token_ids):
    """Logits [T, vocab] for one sequence of token ids (full causal forward)."""
    d, heads, kv_heads, dh = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"], \
        config["head_dim"]
    eps, base = config["rms_norm_eps"], config["rope_theta"]
    t = len(token_ids)
    embed = _dense(weights["model.embed_tokens.weight"])
    x = embed[np.asarray(token_ids)]
    pos = np.arange(t)
    mask = np.triu(np.full((t, t), -np.inf), 1)
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = po.rmsnorm_fp64(x, np.asarray(weights[p + "input_layernorm.weight"], np.float64), eps)
        q = (h @ _dense(weights[p + "self_attn.q_proj.weight"]).T).reshape(t, heads, dh)
        k = (h @ _dense(weights[p + "self_attn.k_proj.weight"]).T).reshape(t, kv_heads, dh)
        v = (h @ _dense(weights[p + "self_attn.v_proj.weight"]).T).reshape(t, kv_heads, dh)
        q, k = rope_half(q, pos, base), rope_half(k, pos, base)
        rep = heads // kv_heads
        k, v = np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1)
        scores = np.einsum("thd,shd->hts", q, k) / np.sqrt(dh) + mask[None]
        scores -= scores.max(axis=-1, keepdims=True)
        prob = np.exp(scores)
        prob /= prob.sum(axis=-1, keepdims=True)
        ctx = np.einsum("hts,shd->thd", prob, v).reshape(t, heads * dh)
        x = x + ctx @ _dense(weights[p + "self_attn.o_proj.weight"]).T
        h = po.rmsnorm_fp64(x, np.asarray(weights[p + "post_attention_layernorm.weight"], np.float64), eps)
        g = h @ _dense(weights[p + "mlp.gate_proj.weight"]).T
        u = h @ _dense(weights[p + "mlp.up_proj.weight"]).T
        x = x + (po.silu64(g) * u) @ _dense(weights[p + "mlp.down_proj.weight"]).T
    x = po.rmsnorm_fp64(x, np.asarray(weights["model.norm.weight"], np.float64), eps)
    head = weights.get("lm_head.weight", weights["model.embed_tokens.weight"])
    return x @ _dense(head).T
