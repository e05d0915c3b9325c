"""GGUF file seam: packed tensors of a model file -> device-resident banks and MoE layers.

Mirrors the parts of the reference's loaders that feed the quantized operators:

* ``GGUFWeightMap.get_packed`` / ``shape_of`` (``mini_llm/external/gguf_loader.py:136-188``): a
  memory-mapped tensor as a zero-copy ``PackedGGUFWeight`` with the canonical ``[out, in]`` shape;
* ``Qwen3NextGGUFIndex`` (``mini_llm/external/qwen3next_gguf.py:60-169``): metadata, layer
  validation, ``expert_weights(layer, expert)`` with the fused ``ffn_gate_up_exps`` row split;
* ``resolve_gguf_weight`` / ``project_gguf_linear`` / ``project_gguf_swiglu``
  (``mini_llm/external/gguf_projection.py:12-97``): lazy, caller-cached promotion of one tensor to
  the GPU and the projection through the packed kernels;
* the inverse Q/K row permutation of llama.cpp's converter
  (``gguf_loader.py:123-133``), here applied to packed rows (rows are independent byte strings, so
  the permutation is exact and needs no dequantization).

What differs from the reference: a B200 holds every expert, so ``expert_bank(layer)`` uploads the
three banks of a layer whole (one host->device copy per tensor straight from the mapping, the fused
gate/up tensor split on the device) and ``moe_layer(layer)`` returns a ready ``PackedMoELayer``;
dense (F32/F16/BF16) tensors are only decoded for the small router / gate / norm vectors.
The file is read with the ``gguf`` package's ``GGUFReader`` (metadata + mmap), as in the reference.
"""

from pathlib import Path

import numpy as np

from .quantized_weight import BLOCK_FORMATS, PackedGGUFWeight

_SHARED = ("ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight")


def _torch():
    import torch
    return torch


def _shape(tensor):
    """GGUF stores shapes input-dimension first; canonical shapes are ``[..., out, in]``."""
    return tuple(int(d) for d in reversed(tensor.shape))


def _meta(reader, name, default=None):
    field = reader.fields.get(name)
    return default if field is None else field.contents(0)


def _packed(tensor):
    kind = tensor.tensor_type.name
    if kind not in BLOCK_FORMATS:
        raise NotImplementedError(f"{tensor.name}: GGUF {kind} has no packed kernel here")
    return PackedGGUFWeight(tensor.data, _shape(tensor), kind)


def row_range(weight, first, last):
    """Zero-copy contiguous rows ``[first, last)`` of a packed ``[out, in]`` matrix."""
    if len(weight.shape) != 2 or not 0 <= first < last <= weight.shape[0]:
        raise ValueError("Invalid packed matrix row range")
    qk, qb = BLOCK_FORMATS[weight.quant_type]
    if weight.shape[1] % qk:
        raise ValueError("Cannot split an unaligned packed GGUF projection")
    row_bytes = weight.shape[1] // qk * qb
    return PackedGGUFWeight(weight.data[first * row_bytes:last * row_bytes], (last - first, weight.shape[1]),
                            weight.quant_type)


def restore_hf_rope_rows_packed(weight, num_heads):
    """Undo the converter's Q/K row permutation ``[heads, 2, half, in] -> [heads, half, 2, in]`` on
    packed rows; returns a new host ``PackedGGUFWeight`` (one copy of the matrix)."""
    rows, columns = weight.shape
    if num_heads <= 0 or rows % (2 * num_heads):
        raise ValueError("Invalid Q/K head shape for GGUF inverse RoPE permutation")
    qk, qb = BLOCK_FORMATS[weight.quant_type]
    row_bytes = columns // qk * qb
    half = rows // (num_heads * 2)
    data = np.asarray(weight.data).reshape(num_heads, half, 2, row_bytes).swapaxes(1, 2)
    return PackedGGUFWeight(np.ascontiguousarray(data).reshape(-1), (rows, columns), weight.quant_type)


def decode_dense(tensor):
    """F32 / F16 / BF16 tensor -> float32 ndarray of the canonical shape."""
    kind = tensor.tensor_type.name
    raw = np.asarray(tensor.data)
    if kind == "F32":
        values = raw.view(np.float32) if raw.dtype != np.float32 else raw
    elif kind == "F16":
        values = (raw.view(np.float16) if raw.dtype != np.float16 else raw).astype(np.float32)
    elif kind == "BF16":
        bits = raw.view(np.uint16).astype(np.uint32) << 16
        values = bits.view(np.float32)
    else:
        raise TypeError(f"{tensor.name}: {kind} is not a dense tensor type")
    return np.ascontiguousarray(values, dtype=np.float32).reshape(_shape(tensor))


class GGUFPackedIndex:
    """Tensor index of one GGUF file; nothing is read until a tensor is asked for."""

    def __init__(self, reader, source_path=None):
        self.reader = reader
        self.source_path = source_path
        self.tensors = {t.name: t for t in reader.tensors}
        if len(self.tensors) != len(reader.tensors):
            raise ValueError("Duplicate GGUF tensor name")
        self.architecture = str(_meta(reader, "general.architecture", ""))
        prefix = self.architecture
        self.layers = int(_meta(reader, f"{prefix}.block_count", 0) or 0)
        self.d_model = int(_meta(reader, f"{prefix}.embedding_length", 0) or 0)
        self.expert_count = int(_meta(reader, f"{prefix}.expert_count", 0) or 0)
        self.experts_per_token = int(_meta(reader, f"{prefix}.expert_used_count", 0) or 0)
        self.rms_eps = float(_meta(reader, f"{prefix}.attention.layer_norm_rms_epsilon", 1e-6) or 1e-6)

    @classmethod
    def open(cls, path):
        try:
            from gguf import GGUFReader
        except ImportError as exc:
            raise RuntimeError("GGUF loading requires the 'gguf' package") from exc
        path = Path(path).expanduser().resolve()
        if not path.is_file():
            raise FileNotFoundError(f"GGUF model not found: {path}")
        return cls(GGUFReader(str(path)), source_path=path)

    # ---- generic access (GGUFWeightMap surface) -------------------------------------------
    def __contains__(self, name):
        return name in self.tensors

    def shape_of(self, name):
        return _shape(self.tensors[name])

    def tensor_type(self, name):
        return self.tensors[name].tensor_type.name

    def get_packed(self, name):
        """The mmap-backed packed bytes of one tensor, never dequantized."""
        tensor = self.tensors[name]
        if tensor.tensor_type.name not in BLOCK_FORMATS:
            raise TypeError(f"{name} is not a packed GGUF tensor")
        return _packed(tensor)

    def non_expert_weight(self, name):
        """One small dense tensor as float32 (router, gates, norms); expert banks are refused."""
        if name.endswith("_exps.weight"):
            raise ValueError(f"{name}: routed expert banks require expert_weights() / expert_bank()")
        tensor = self.tensors[name]
        if tensor.tensor_type.name in BLOCK_FORMATS:
            raise TypeError(f"{name} is packed; use get_packed()")
        return decode_dense(tensor)

    # ---- MoE access (Qwen3NextGGUFIndex surface) -------------------------------------------
    def _expert_tensors(self, layer_id):
        layer_id = int(layer_id)
        if not 0 <= layer_id < max(self.layers, 1):
            raise IndexError(f"Invalid layer {layer_id}")
        stem = f"blk.{layer_id}."
        down_name = stem + "ffn_down_exps.weight"
        if down_name not in self.tensors:
            raise ValueError(f"layer {layer_id}: missing {down_name}")
        down = _packed(self.tensors[down_name])
        if len(down.shape) != 3:
            raise ValueError(f"{down_name}: expected [E, D, F], got {down.shape}")
        e, d, f = down.shape
        fused_name = stem + "ffn_gate_up_exps.weight"
        if fused_name in self.tensors:
            fused = _packed(self.tensors[fused_name])
            if fused.shape != (e, 2 * f, d):
                raise ValueError(f"{fused_name}: expected {(e, 2 * f, d)}, got {fused.shape}")
            return stem, (e, d, f), fused, None, None, down
        gate_name, up_name = stem + "ffn_gate_exps.weight", stem + "ffn_up_exps.weight"
        if gate_name not in self.tensors or up_name not in self.tensors:
            raise ValueError(f"layer {layer_id}: no gate/up expert tensors")
        gate, up = _packed(self.tensors[gate_name]), _packed(self.tensors[up_name])
        if gate.shape != (e, f, d) or up.shape != (e, f, d):
            raise ValueError(f"layer {layer_id}: gate/up shapes {gate.shape} / {up.shape}, expected {(e, f, d)}")
        return stem, (e, d, f), None, gate, up, down

    def expert_weights(self, layer_id, expert_id):
        """Three zero-copy packed host matrices ``(gate [F,D], up [F,D], down [D,F])`` of one expert."""
        _, (e, d, f), fused, gate, up, down = self._expert_tensors(layer_id)
        expert_id = int(expert_id)
        if not 0 <= expert_id < e:
            raise IndexError(f"Invalid expert ({layer_id}, {expert_id})")
        if fused is not None:
            both = fused.select_outer(expert_id)          # the converter concatenates [gate, up] along rows
            return row_range(both, 0, f), row_range(both, f, 2 * f), down.select_outer(expert_id)
        return gate.select_outer(expert_id), up.select_outer(expert_id), down.select_outer(expert_id)

    def expert_bank(self, layer_id):
        """All experts of a layer as a device-resident ``PackedExpertBank`` (GGUF byte layout)."""
        from .experts_inference import PackedExpertBank
        from .quantized_linear import packed_bytes_to_device
        _, (e, d, f), fused, gate, up, down = self._expert_tensors(layer_id)
        down_dev = packed_bytes_to_device(down.data)
        if fused is not None:
            both = packed_bytes_to_device(fused.data).reshape(e, 2, -1)     # [E, gate|up, F rows of bytes]
            gate_dev, up_dev = both[:, 0].contiguous().reshape(-1), both[:, 1].contiguous().reshape(-1)
            kind = fused.quant_type
            return PackedExpertBank(gate_dev, up_dev, down_dev, kind, kind, down.quant_type, e, d, f)
        return PackedExpertBank(packed_bytes_to_device(gate.data), packed_bytes_to_device(up.data), down_dev,
                                gate.quant_type, up.quant_type, down.quant_type, e, d, f)

    def shared_expert(self, layer_id):
        """``(gate, up, down)`` device weights of the always-on shared expert, or ``None``."""
        from .quantized_linear import packed_to_device
        stem = f"blk.{int(layer_id)}."
        if not all(stem + name in self.tensors for name in _SHARED):
            return None
        return tuple(packed_to_device(self.get_packed(stem + name)) for name in _SHARED)

    def moe_layer(self, layer_id, top_k=None, *, normalization_floor=2.0 ** -14):
        """A ``PackedMoELayer`` built from the file: bank, expert-major router weight, shared expert
        and its admission gate when the file has them."""
        from .moe_layer import PackedMoELayer
        torch = _torch()
        stem = f"blk.{int(layer_id)}."
        bank = self.expert_bank(layer_id)
        k = int(top_k or self.experts_per_token)
        if k <= 0:
            raise ValueError("top_k is neither given nor recorded in the file")
        router = self.non_expert_weight(stem + "ffn_gate_inp.weight")         # [E, D]: expert-major already
        if router.shape != (bank.n_experts, bank.d_model):
            raise ValueError(f"router weight shape {router.shape}, expected {(bank.n_experts, bank.d_model)}")
        router_t = torch.from_numpy(router).cuda()
        gate_name = stem + "ffn_gate_inp_shexp.weight"
        shared_gate = None
        if gate_name in self.tensors:
            shared_gate = torch.from_numpy(self.non_expert_weight(gate_name).reshape(-1)).cuda()
        return PackedMoELayer(bank, router_t.t().contiguous(), k, shared=self.shared_expert(layer_id),
                              shared_gate=shared_gate, layer_id=int(layer_id),
                              normalization_floor=normalization_floor)


# ---- lazy projection helpers (gguf_projection surface) ---------------------------------------------
def resolve_gguf_weight(index, tensor_name, host_cache, device_cache, cache_key, *, upload=None):
    """Lazily resolve one canonical ``[out, in]`` weight using caller-owned caches: packed tensors
    stay packed on the host and are promoted to the GPU once; dense tensors become FP32 CUDA tensors."""
    from .quantized_linear import packed_to_device
    torch = _torch()
    upload = packed_to_device if upload is None else upload
    weight = host_cache.get(cache_key)
    if weight is None:
        tensor = index.tensors[tensor_name]
        weight = _packed(tensor) if tensor.tensor_type.name in BLOCK_FORMATS else decode_dense(tensor)
        host_cache[cache_key] = weight
    if cache_key not in device_cache:
        device_cache[cache_key] = upload(weight) if isinstance(weight, PackedGGUFWeight) \
            else torch.from_numpy(weight).cuda()
    return device_cache[cache_key]


def project_gguf_linear(hidden, index, tensor_name, host_cache, device_cache, cache_key, *, linear=None, upload=None):
    """Project ``[B, T, in]`` by a lazily resolved GGUF ``[out, in]`` tensor (packed or dense)."""
    from .quantized_linear import DevicePackedGGUFWeight, quantized_linear
    weight = resolve_gguf_weight(index, tensor_name, host_cache, device_cache, cache_key, upload=upload)
    if isinstance(host_cache[cache_key], PackedGGUFWeight):
        return (quantized_linear if linear is None else linear)(hidden.contiguous(), weight)
    if isinstance(weight, DevicePackedGGUFWeight):
        raise TypeError("dense host tensor resolved to a packed device weight")
    return (hidden.float() @ weight.t()).to(hidden.dtype)


def project_gguf_swiglu(hidden, index, gate_tensor_name, up_tensor_name, host_cache, device_cache, gate_cache_key,
                        up_cache_key, *, upload=None):
    """``SiLU(hidden @ gate.T) * (hidden @ up.T)``: one fused launch when both tensors are packed."""
    from .quantized_linear import DevicePackedGGUFWeight, quantized_swiglu
    torch = _torch()
    gate = resolve_gguf_weight(index, gate_tensor_name, host_cache, device_cache, gate_cache_key, upload=upload)
    up = resolve_gguf_weight(index, up_tensor_name, host_cache, device_cache, up_cache_key, upload=upload)
    if isinstance(gate, DevicePackedGGUFWeight) and isinstance(up, DevicePackedGGUFWeight):
        return quantized_swiglu(hidden.contiguous(), gate, up)
    g = project_gguf_linear(hidden, index, gate_tensor_name, host_cache, device_cache, gate_cache_key, upload=upload)
    u = project_gguf_linear(hidden, index, up_tensor_name, host_cache, device_cache, up_cache_key, upload=upload)
    return (torch.nn.functional.silu(g.float()) * u.float()).to(hidden.dtype)
