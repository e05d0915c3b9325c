"""Llama-family decoder whose every linear runs on the packed GGUF kernels.

Mirrors the surface of the reference's ``ExternalLlamaModel``
(``mini_llm/external/llama_model.py:16-178``: ``expected_shapes``, ``set_weights`` with canonical HF
names, ``create_generation_state``, ``prefill``, ``decode_one``) and of its configuration
(``mini_llm/external/config.py``). The reference expands GGUF weights to dense FP16/FP32 for this
adapter; here they stay packed and resident in HBM, which is the point of the exercise:

* q/k/v/o, gate/up (one fused SwiGLU launch), down and the LM head are ``quantized_linear`` /
  ``quantized_swiglu`` on ``DevicePackedGGUFWeight`` (tile layouts where they exist);
* RMSNorm is ``b200q_rmsnorm`` / the fused residual-add variant; the residual stream is FP32;
* embedding rows are gathered as packed bytes and decoded by ``b200q_dequantize``;
* the one-token step runs rotate-half RoPE, the KV-cache store and single-query attention over the cache as one
  kernel (``b200q_rope_attention``; ``b200q_rope_kv_store`` + ``b200q_decode_attention`` are the two-launch form), and ``b200q_silu_mul`` on
  the output of the stacked gate|up projection; prefill (and ``fused_decode = False``) does the
  RoPE / cache / attention bookkeeping with plain torch ops. The decode step has static shapes - the cache is written at a
  device-side position and attention stops at that position - so ``decode_one`` can be captured in
  a CUDA graph.
"""

import ctypes
import os
from dataclasses import dataclass

import numpy as np

from . import _lib
from .moe_layer import RMSNormInference
from .quantized_linear import (GEMM_MIN_TOKENS, DevicePackedGGUFWeight, dequantize_device, packed_to_device, quantized_linear,
                               quantized_swiglu, retile_enabled, retile_gate_up, retile_weight)
from .quantized_weight import PackedGGUFWeight, block_format


def _torch():
    import torch
    return torch


@dataclass
class ExternalLlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False

    def validate(self):
        if min(self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
               self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.max_position_embeddings) <= 0:
            raise ValueError("Llama configuration values must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for rotary embeddings")


class GenerationState:
    """KV cache ``[layers, B, kv_heads, horizon, head_dim]`` and the device-side position."""

    def __init__(self, config, batch, horizon, dtype, device):
        torch = _torch()
        shape = (config.num_hidden_layers, batch, config.num_key_value_heads, horizon, config.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.position = torch.zeros(1, dtype=torch.int64, device=device)      # tokens already in the cache
        self.length = 0                                                        # host copy, for checks only
        self.batch, self.horizon = batch, horizon


class ExternalLlamaModel:
    def __init__(self, config, *, dtype="bfloat16", device="cuda"):
        if not isinstance(config, ExternalLlamaConfig):
            raise TypeError("config must be ExternalLlamaConfig")
        config.validate()
        torch = _torch()
        if dtype not in ("float32", "float16", "bfloat16"):
            raise ValueError("dtype must be float32, float16 or bfloat16")
        self.config, self.dtype, self.device = config, getattr(torch, dtype), device
        self.fused_decode = True       # one-token steps use the RoPE+store and attention kernels
        # ... and run each residual-add + RMSNorm inside the projection that consumes it (``B200Q_NORM_GEMV=0``: as a
        # launch of its own; the results are the same bits)
        self.fused_norm_linear = os.environ.get("B200Q_NORM_GEMV", "1") != "0"
        self._loaded = False

    def expected_shapes(self):
        cfg = self.config
        d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
        result = {"model.embed_tokens.weight": (v, d), "model.norm.weight": (d,)}
        for i in range(cfg.num_hidden_layers):
            stem = f"model.layers.{i}."
            result.update({
                stem + "input_layernorm.weight": (d,), stem + "post_attention_layernorm.weight": (d,),
                stem + "self_attn.q_proj.weight": (q, d), stem + "self_attn.k_proj.weight": (kv, d),
                stem + "self_attn.v_proj.weight": (kv, d), stem + "self_attn.o_proj.weight": (d, q),
                stem + "mlp.gate_proj.weight": (f, d), stem + "mlp.up_proj.weight": (f, d),
                stem + "mlp.down_proj.weight": (d, f),
            })
        if not cfg.tie_word_embeddings:
            result["lm_head.weight"] = (v, d)
        return result

    # ------------------------------------------------------------------------------ weights
    def _matrix(self, value, *, tile=True):
        """Host ``PackedGGUFWeight`` / device packed weight -> device packed weight (tiled if possible)."""
        if isinstance(value, PackedGGUFWeight):
            value = packed_to_device(value)
        if not isinstance(value, DevicePackedGGUFWeight):
            raise TypeError("Llama projection weights must be packed GGUF matrices")
        if tile and retile_enabled():
            value = retile_weight(value, force=self.dtype != _torch().float32)
        return value

    def set_weights(self, weights, *, strict=True):
        """Bind canonical HF-named tensors: matrices packed (host or device), norm vectors dense.
        Incomplete or mis-shaped imports are rejected before anything is uploaded."""
        torch = _torch()
        expected = self.expected_shapes()
        missing = sorted(set(expected) - set(weights))
        optional = {"lm_head.weight"} if self.config.tie_word_embeddings else set()
        extra = sorted(set(weights) - set(expected) - optional)
        if missing or (strict and extra):
            raise ValueError(f"Invalid Llama weight names: missing={missing[:5]}, extra={extra[:5]}")
        for name, shape in expected.items():
            if tuple(int(s) for s in weights[name].shape) != shape:
                raise ValueError(f"{name}: expected shape {shape}, got {tuple(weights[name].shape)}")
        cfg = self.config

        def norm(name):
            module = RMSNormInference(cfg.hidden_size, eps=cfg.rms_norm_eps)
            gamma = torch.as_tensor(np.asarray(weights[name], dtype=np.float32)).to(self.device, self.dtype)
            module.set_weights(gamma.contiguous())
            return module

        def stacked(names):
            """Rows of several same-format matrices with equal K as one device matrix (one launch for
            all of them), or None when the formats differ."""
            parts = [self._matrix(weights[n], tile=False) for n in names]
            if len({w.quant_type for w in parts}) != 1 or len({w.shape[1] for w in parts}) != 1:
                return None
            data = torch.cat([w.data for w in parts])
            rows = sum(w.shape[0] for w in parts)
            return with_prefill_copy(DevicePackedGGUFWeight(data, (rows, parts[0].shape[1]), parts[0].quant_type))

        def with_prefill_copy(native):
            """The matrix in the layout the decode kernels read (a tile layout where there is one) and,
            kept beside it under ``native_of``, the GGUF-layout bytes when they differ: the tensor-core
            GEMM that serves many-token calls (prefill) reads the GGUF layout. Costs one more copy of
            the packed bytes in HBM (1.8 GB for a 1.7B Q8_0 model); ``B200Q_PREFILL_GEMM=0`` skips it."""
            native = self._matrix(native, tile=False)
            decode = self._matrix(native)
            if (decode is not native and self.dtype == torch.bfloat16
                    and os.environ.get("B200Q_PREFILL_GEMM", "1") != "0"):
                self.native_of[id(decode)] = native
            return decode

        self.native_of = {}
        self.embed = self._matrix(weights["model.embed_tokens.weight"], tile=False)     # rows are gathered
        self.lm_head = self.embed if cfg.tie_word_embeddings else self._matrix(weights["lm_head.weight"])
        if cfg.tie_word_embeddings and retile_enabled():
            self.lm_head = self._matrix(self.embed)
        self.final_norm = norm("model.norm.weight")
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            self.layers.append({
                "norm1": norm(p + "input_layernorm.weight"), "norm2": norm(p + "post_attention_layernorm.weight"),
                "qkv": stacked([p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                                p + "self_attn.v_proj.weight"]),
                "o": with_prefill_copy(weights[p + "self_attn.o_proj.weight"]),
                "gate": self._matrix(weights[p + "mlp.gate_proj.weight"], tile=False),
                "up": self._matrix(weights[p + "mlp.up_proj.weight"], tile=False),
                "down": with_prefill_copy(weights[p + "mlp.down_proj.weight"]),
            })
            layer = self.layers[-1]
            if layer["qkv"] is None:
                for key, name in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj")):
                    layer[key] = with_prefill_copy(weights[p + f"self_attn.{name}.weight"])
            layer["gate_up"] = None
            if layer["gate"].quant_type == layer["up"].quant_type == "Q8_0" and retile_enabled():
                # no fused SwiGLU kernel reads Q8_0 tiles: one tiled GEMV for both, then the product
                layer["gate_up"] = stacked([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"])
                if layer["gate_up"] is not None and layer["gate_up"].quant_type != "Q8_0_TILED":
                    layer["gate_up"] = None
            if layer["gate_up"] is not None:
                layer["gate"] = layer["up"] = None
            elif retile_enabled():
                layer["gate"], layer["up"] = retile_gate_up(layer["gate"], layer["up"], self.dtype != torch.float32)
        half = cfg.head_dim // 2
        inv = 1.0 / (float(cfg.rope_theta) ** (2.0 * np.arange(half) / cfg.head_dim))
        ang = np.arange(cfg.max_position_embeddings)[:, None] * inv[None, :]
        self._cos = torch.as_tensor(np.cos(ang), dtype=torch.float32).to(self.device)
        self._sin = torch.as_tensor(np.sin(ang), dtype=torch.float32).to(self.device)
        self._loaded = True

    @property
    def packed_bytes(self):
        total = self.embed.nbytes + (0 if self.config.tie_word_embeddings else self.lm_head.nbytes)
        for layer in self.layers:
            total += sum(layer[n].nbytes for n in ("qkv", "q", "k", "v", "o", "gate_up", "gate", "up", "down")
                         if layer.get(n) is not None)
        return total + sum(w.nbytes for w in self.native_of.values())

    # ------------------------------------------------------------------------------ running
    def _require_weights(self):
        if not self._loaded:
            raise RuntimeError("External weights have not been loaded")

    def create_generation_state(self, batch_size=1, max_length=None):
        self._require_weights()
        max_length = self.config.max_position_embeddings if max_length is None else int(max_length)
        if not 1 <= max_length <= self.config.max_position_embeddings:
            raise ValueError("Requested KV horizon exceeds configured positions")
        return GenerationState(self.config, int(batch_size), max_length, self.dtype, self.device)

    def _embed(self, token_ids):
        torch = _torch()
        v, d = self.embed.shape
        qk, qb = block_format(self.embed.quant_type)
        rows = self.embed.data.view(v, d // qk * qb).index_select(0, token_ids.reshape(-1)).contiguous()
        return dequantize_device(rows.reshape(-1), rows.shape[0], d, self.embed.quant_type)      # FP32 [n, d]

    def _rope(self, x, positions):
        """x [B, T, H, Dh] (FP32), positions [T] int64 device tensor; rotate-half layout."""
        torch = _torch()
        half = x.shape[-1] // 2
        cos = self._cos.index_select(0, positions)[None, :, None, :]
        sin = self._sin.index_select(0, positions)[None, :, None, :]
        x0, x1 = x[..., :half], x[..., half:]
        return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)

    def _linear(self, x, weight, out_dtype=None):
        """Packed projection: calls of many BF16 rows (prefill) read the GGUF-layout copy, which the
        tensor-core GEMM serves with one pass over the weights; everything else reads the decode layout."""
        native = self.native_of.get(id(weight))
        if native is not None and x.dtype == _torch().bfloat16 and x.shape[0] >= GEMM_MIN_TOKENS.get(native.quant_type, 1 << 30):
            return quantized_linear(x, native, out_dtype=out_dtype)
        return quantized_linear(x, weight, out_dtype=out_dtype)

    def _norm_linear(self, norm, residual, branch, weight, out_dtype):
        """``(residual + branch, rmsnorm(residual + branch) @ weight.T)``: one launch (``b200q_gemv_norm``) where the
        fused kernel covers the case - tile-layout Q6_K / Q8_0 weight, 16-bit model type, a few rows - else the
        norm kernel followed by the projection."""
        torch = _torch()
        rows, d = residual.shape
        n, k = weight.shape
        fmt = _lib.FORMAT_ID.get(weight.quant_type, -1)
        dt = _lib.DTYPE_ID[str(norm.gamma.dtype).replace("torch.", "")]
        # (one row only: every CTA of the projection normalises the rows itself, one after the other)
        if (self.fused_norm_linear and rows == 1 and branch.is_contiguous() and residual.is_contiguous() and k == d
                and _lib.load().b200q_gemv_norm_supported(fmt, n, k, dt, rows)):
            ptr = lambda x: ctypes.c_void_p(x.data_ptr())
            res_out = torch.empty_like(residual)
            y = torch.empty((rows, n), dtype=out_dtype or norm.gamma.dtype, device=residual.device)
            _lib.call("b200q_gemv_norm", ptr(weight.data), fmt, n, k, ptr(residual), ptr(branch),
                      _lib.DTYPE_ID[str(branch.dtype).replace("torch.", "")], 1.0, ptr(norm.gamma), dt, float(norm.eps),
                      rows, ptr(res_out), ptr(y), _lib.DTYPE_ID[str(y.dtype).replace("torch.", "")],
                      _lib.current_stream())
            return res_out, y
        residual, hidden = norm.forward_residual_add(residual, branch)
        return residual, self._linear(hidden, weight, out_dtype)

    def _silu_linear(self, gu, weight):
        """``(silu(gate) * up) @ weight.T`` for the stacked FP32 gate|up output ``gu`` [B, 2F]: ``b200q_silu_mul``
        followed by the projection. ``B200Q_SILU_GEMV=1`` makes it one launch (``b200q_gemv_silu``, same bits) for a
        tile-layout Q6_K / Q8_0 weight and one row - measured slower at the 1.7B shape (778 against 828 tokens/s:
        every CTA of the projection computes the 8192 activations itself before it starts on its weights, which
        costs more than the 1.8 us of the chained element-wise launch)."""
        import os
        torch = _torch()
        b, f = gu.shape[0], gu.shape[1] // 2
        n, k = weight.shape
        ptr = lambda x: ctypes.c_void_p(x.data_ptr())
        dt = _lib.DTYPE_ID[str(self.dtype).replace("torch.", "")]
        fmt = _lib.FORMAT_ID.get(weight.quant_type, -1)
        if (b == 1 and k == f and gu.is_contiguous() and gu.data_ptr() % 16 == 0 and self.dtype != torch.float32
                and os.environ.get("B200Q_SILU_GEMV", "0") == "1"
                and _lib.load().b200q_gemv_silu_supported(fmt, n, k, dt, b)):
            y = torch.empty((b, n), dtype=self.dtype, device=gu.device)
            _lib.call("b200q_gemv_silu", ptr(weight.data), fmt, n, k, ptr(gu), dt, b, ptr(y), dt, _lib.current_stream())
            return y
        act = torch.empty((b, f), dtype=self.dtype, device=gu.device)
        _lib.call("b200q_silu_mul", ptr(gu), b, f, ptr(act), dt, _lib.current_stream())
        return self._linear(act, weight)

    def _rope_attention(self, q2, k2, v2, positions, state, layer_index, ctx):
        """RoPE of the new query / key, the KV-cache store and single-query attention of a one-token step: one
        launch (``b200q_rope_attention``), or the two separate ones with ``B200Q_ROPE_ATTENTION=0`` (same bits)."""
        import os
        cfg = self.config
        heads, kv_heads, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        b = q2.shape[0]
        ptr = lambda x: ctypes.c_void_p(x.data_ptr())
        cache_id = _lib.DTYPE_ID[str(self.dtype).replace("torch.", "")]
        kc, vc = state.k[layer_index], state.v[layer_index]
        if os.environ.get("B200Q_ROPE_ATTENTION", "1") != "0":
            _lib.call("b200q_rope_attention", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0),
                      ptr(positions), ptr(self._cos), ptr(self._sin), int(self._cos.shape[0]), b, heads, kv_heads, dh,
                      state.horizon, ptr(kc), ptr(vc), cache_id, float(dh ** -0.5), ptr(ctx), cache_id,
                      _lib.current_stream())
            return
        _lib.call("b200q_rope_kv_store", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0),
                  ptr(positions), ptr(self._cos), ptr(self._sin), int(self._cos.shape[0]), b, 1, heads, kv_heads, dh,
                  state.horizon, ptr(kc), ptr(vc), cache_id, _lib.current_stream())
        _lib.call("b200q_decode_attention", ptr(q2), q2.stride(0), ptr(kc), ptr(vc), cache_id, ptr(positions), b, heads,
                  kv_heads, dh, state.horizon, float(dh ** -0.5), ptr(ctx), cache_id, _lib.current_stream())

    def _forward_one_token(self, token_ids, state, positions):
        """The one-token step with every residual-add + RMSNorm deferred into the projection that follows it
        (stacked qkv, stacked gate|up, LM head). Returns FP32 logits [B, vocab]."""
        torch = _torch()
        cfg = self.config
        b = token_ids.shape[0]
        heads, kv_heads, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        qd, kd = heads * dh, kv_heads * dh
        ptr = lambda x: ctypes.c_void_p(x.data_ptr())
        cache_id = _lib.DTYPE_ID[str(self.dtype).replace("torch.", "")]
        residual = self._embed(token_ids)                                         # FP32 [B, d]
        pending = None                                                            # (norm, branch) not applied yet
        for i, layer in enumerate(self.layers):
            if pending is None:
                qkv = self._linear(layer["norm1"].forward_residual(residual), layer["qkv"], torch.float32)
            else:
                residual, qkv = self._norm_linear(layer["norm1"], residual, pending, layer["qkv"], torch.float32)
            q2, k2, v2 = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
            ctx = torch.empty((b, heads * dh), dtype=self.dtype, device=residual.device)
            self._rope_attention(q2, k2, v2, positions, state, i, ctx)
            attn = quantized_linear(ctx, layer["o"])
            residual, gu = self._norm_linear(layer["norm2"], residual, attn, layer["gate_up"], torch.float32)
            pending = self._silu_linear(gu, layer["down"])
        _, logits = self._norm_linear(self.final_norm, residual, pending, self.lm_head, torch.float32)
        return logits

    def _forward(self, token_ids, state, positions, mask):
        """token_ids [B, T]; positions [T] device int64; mask [T, horizon] additive FP32. Returns the
        final normalised hidden states [B*T, d] in the model dtype."""
        torch = _torch()
        cfg = self.config
        b, t = token_ids.shape
        heads, kv_heads, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        residual = self._embed(token_ids)                                         # FP32 [B*T, d]
        hidden = self.layers[0]["norm1"].forward_residual(residual)
        for i, layer in enumerate(self.layers):
            qd, kd = heads * dh, kv_heads * dh
            if layer["qkv"] is not None:                     # one launch for the three projections
                qkv = self._linear(hidden, layer["qkv"], torch.float32)
                q2, k2, v2 = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
            else:
                q2 = self._linear(hidden, layer["q"], torch.float32)
                k2 = self._linear(hidden, layer["k"], torch.float32)
                v2 = self._linear(hidden, layer["v"], torch.float32)
            if t == 1 and dh in (64, 128) and self.fused_decode:
                # one-token step: RoPE + cache store, then single-query attention, one kernel each
                ptr = lambda x: ctypes.c_void_p(x.data_ptr())
                cache_id = _lib.DTYPE_ID[str(self.dtype).replace("torch.", "")]
                ctx = torch.empty((b, heads * dh), dtype=self.dtype, device=hidden.device)
                self._rope_attention(q2, k2, v2, positions, state, i, ctx)
                attn = quantized_linear(ctx, layer["o"])
                residual, hidden = layer["norm2"].forward_residual_add(residual, attn)
                hidden, residual = self._ffn(i, layer, hidden, residual)
                continue
            q, k, v = q2.reshape(b, t, heads, dh), k2.reshape(b, t, kv_heads, dh), v2.reshape(b, t, kv_heads, dh)
            q, k = self._rope(q, positions), self._rope(k, positions)
            state.k[i].index_copy_(2, positions, k.permute(0, 2, 1, 3).to(self.dtype))
            state.v[i].index_copy_(2, positions, v.permute(0, 2, 1, 3).to(self.dtype))
            keys, values = state.k[i].float(), state.v[i].float()                 # [B, kv, horizon, dh]
            if kv_heads != heads:
                keys = keys.repeat_interleave(heads // kv_heads, dim=1)
                values = values.repeat_interleave(heads // kv_heads, dim=1)
            scores = torch.matmul(q.permute(0, 2, 1, 3), keys.transpose(-1, -2)) * (dh ** -0.5) + mask
            ctx = torch.matmul(torch.softmax(scores, dim=-1), values)            # [B, heads, T, dh]
            ctx = ctx.permute(0, 2, 1, 3).reshape(b * t, heads * dh).to(self.dtype).contiguous()
            attn = self._linear(ctx, layer["o"])
            residual, hidden = layer["norm2"].forward_residual_add(residual, attn)
            hidden, residual = self._ffn(i, layer, hidden, residual)
        return hidden

    def _ffn(self, i, layer, hidden, residual):
        """SwiGLU FFN on the normalised ``hidden``; returns the next layer's normalised input and the
        updated FP32 residual stream."""
        torch = _torch()
        if layer["gate_up"] is not None:
            gu = self._linear(hidden, layer["gate_up"], torch.float32)
            f = gu.shape[1] // 2
            act = torch.empty((gu.shape[0], f), dtype=self.dtype, device=gu.device)
            _lib.call("b200q_silu_mul", ctypes.c_void_p(gu.data_ptr()), gu.shape[0], f, ctypes.c_void_p(act.data_ptr()),
                      _lib.DTYPE_ID[str(self.dtype).replace("torch.", "")], _lib.current_stream())
        else:
            act = quantized_swiglu(hidden, layer["gate"], layer["up"])
        ffn = self._linear(act, layer["down"])
        nxt = self.layers[i + 1]["norm1"] if i + 1 < len(self.layers) else self.final_norm
        residual, hidden = nxt.forward_residual_add(residual, ffn)
        return hidden, residual

    def prefill(self, token_ids, state):
        """token_ids [B, T] int64 CUDA tensor; fills the cache from position 0; returns the logits of
        the last position, FP32 [B, vocab]."""
        self._require_weights()
        torch = _torch()
        b, t = token_ids.shape
        if b != state.batch or t > state.horizon:
            raise ValueError("prompt does not fit the generation state")
        positions = torch.arange(t, device=self.device)
        cols = torch.arange(state.horizon, device=self.device)
        mask = torch.where(cols[None, :] <= positions[:, None], 0.0, float("-inf")).float()
        hidden = self._forward(token_ids, state, positions, mask).reshape(b, t, -1)
        state.position.fill_(t)
        state.length = t
        return quantized_linear(hidden[:, -1].contiguous(), self.lm_head, out_dtype=torch.float32)

    def decode_one(self, token_ids, state):
        """token_ids [B] int64 CUDA tensor: appends one position; returns FP32 logits [B, vocab].
        All shapes are static and the position lives on the device (CUDA-graph capturable; the host
        counter ``state.length`` is advisory and is not advanced inside a captured graph)."""
        self._require_weights()
        torch = _torch()
        if state.length >= state.horizon:
            raise ValueError("generation state is full")
        positions = state.position.clone()
        cfg = self.config
        if (self.fused_decode and self.fused_norm_linear and cfg.head_dim in (64, 128)
                and all(layer["qkv"] is not None and layer["gate_up"] is not None for layer in self.layers)):
            logits = self._forward_one_token(token_ids.reshape(-1, 1), state, positions)
            state.position.add_(1)
            state.length += 1
            return logits
        cols = torch.arange(state.horizon, device=self.device)
        mask = torch.where(cols[None, :] <= positions[:, None], 0.0, float("-inf")).float()
        hidden = self._forward(token_ids.reshape(-1, 1), state, positions, mask)
        state.position.add_(1)
        state.length += 1
        return quantized_linear(hidden, self.lm_head, out_dtype=torch.float32)

    @classmethod
    def synthetic(cls, config, *, fmt="Q8_0", dtype="bfloat16", seed=0, device="cuda"):
        """Random-init model with packed weights generated on the device (benchmark input): uniform
        random codes with small finite block scales, layout and sizes of a real ``fmt`` model."""
        torch = _torch()
        if fmt != "Q8_0":
            raise NotImplementedError("synthetic weights are generated for Q8_0")
        model = cls(config, dtype=dtype, device=device)
        gen = torch.Generator(device=device)

        def matrix(shape, index):
            gen.manual_seed(seed * 100003 + index)
            blocks = shape[0] * shape[1] // 32
            raw = torch.randint(0, 256, (blocks, 34), dtype=torch.uint8, device=device, generator=gen)
            scale = np.frombuffer(np.float16(0.02 / 127 * 3).tobytes(), np.uint8)
            raw[:, 0], raw[:, 1] = int(scale[0]), int(scale[1])
            return DevicePackedGGUFWeight(raw.reshape(-1), shape, "Q8_0")

        weights, index = {}, 0
        for name, shape in model.expected_shapes().items():
            index += 1
            weights[name] = matrix(shape, index) if len(shape) == 2 else np.ones(shape, np.float32)
        model.set_weights(weights)
        return model
