"""Single-row grouped packed expert inference over a pointer table.

Host-side mirror of the reference's ``mini_llm/ops/grouped_quantized_experts.py``
(``supports_grouped_quantized_experts`` :141-151, ``grouped_quantized_experts_forward`` :159-217,
eligibility rules :82-138). The caller supplies handles and routing weights in ascending
expert-id order; repeated handles are legal and stay separate ordered terms; unsupported calls
raise ``ValueError`` and never fall back. Graph: packed gate/up GEMVs -> FP32 SwiGLU -> packed down
GEMV -> FP32 multiply by the route weight (stored) -> sequential FP32 adds from zero in handle
order.
"""

import numpy as np

from . import moe_ops
from .quantized_linear import DevicePackedGGUFWeight, PackedExpertFFNInference
from .quantized_weight import block_format

MAX_GROUPED_EXPERTS = 64


def _torch():
    import torch
    return torch


def _unsupported_reason(x, experts, routing_weights, block_k, routing_slots=None):
    torch = _torch()
    if block_k not in (256, 512, 1024):
        return "block_k must be 256, 512 or 1024"
    if not isinstance(x, torch.Tensor) or not x.is_cuda or x.dtype != torch.float32:
        return "x must be a CUDA FP32 tensor"
    if x.ndim != 2 or x.shape[0] != 1 or x.shape[1] <= 0 or not x.is_contiguous():
        return "x must be contiguous [1, D] with positive D"
    if not isinstance(experts, (list, tuple)) or not 1 <= len(experts) <= MAX_GROUPED_EXPERTS:
        return f"experts must be a nonempty list/tuple of at most {MAX_GROUPED_EXPERTS} handles"
    if routing_slots is not None and (
            not isinstance(routing_slots, (tuple, list)) or len(routing_slots) != len(experts)
            or any(not isinstance(slot, (int, np.integer)) or isinstance(slot, bool)
                   or not 0 <= slot < len(experts) for slot in routing_slots)):
        return "routing_slots must be host integer indices into the [E] routing weights"
    if (not isinstance(routing_weights, torch.Tensor) or not routing_weights.is_cuda
            or routing_weights.dtype != torch.float32 or tuple(routing_weights.shape) != (len(experts),)):
        return "routing_weights must be a CUDA FP32 [E] tensor (slices allowed)"
    if routing_weights.device != x.device:
        return "all operands must be on the current CUDA device"
    signature = None
    for expert in experts:
        if not isinstance(expert, PackedExpertFFNInference):
            return "experts must contain PackedExpertFFNInference handles"
        projections = (expert.gate, expert.up, expert.down)
        if not all(isinstance(w, DevicePackedGGUFWeight) for w in projections):
            return "all projections must be DevicePackedGGUFWeight (no host fallback)"
        gate, up, down = projections
        if (len(gate.shape) != 2 or min(gate.shape) <= 0 or gate.shape != up.shape
                or gate.shape[1] != x.shape[1] or down.shape != (x.shape[1], gate.shape[0])):
            return "expert shapes must be gate/up [F, D], down [D, F] matching x"
        current = tuple((w.shape, w.quant_type) for w in projections)
        if signature is not None and current != signature:
            return "all experts must share per-projection shapes and quantization formats"
        signature = current
        for w in projections:
            qk, qb = block_format(w.quant_type)       # GGUF bytes or a device tile layout of them
            if (w.data.dtype != torch.uint8 or not w.data.is_contiguous() or w.shape[1] % qk
                    or int(w.data.numel()) != w.shape[0] * w.shape[1] // qk * qb):
                return "invalid packed projection storage or block alignment"
            if w.data.device != x.device:
                return "all operands must be on the current CUDA device"
    return None


def supports_grouped_quantized_experts(x, experts, routing_weights, *, block_k=512, routing_slots=None):
    """Metadata-only support check; no allocation, transfer or kernel launch."""
    return _unsupported_reason(x, experts, routing_weights, block_k, routing_slots) is None


def grouped_quantized_experts_forward(x, experts, routing_weights, *, block_k=512, routing_slots=None):
    """Fresh FP32 ``[1, D]`` weighted expert sum on the current stream."""
    reason = _unsupported_reason(x, experts, routing_weights, block_k, routing_slots)
    if reason is not None:
        raise ValueError(f"Unsupported grouped quantized experts: {reason}")
    torch = _torch()
    e, d, f = len(experts), x.shape[1], experts[0].gate.shape[0]
    pointers = np.asarray([[int(w.data.data_ptr()) for w in (h.gate, h.up, h.down)] for h in experts], dtype=np.int64)
    aligned = bool(np.all(pointers % 16 == 0))
    table = torch.from_numpy(np.ascontiguousarray(pointers.T)).to(x.device)     # [3, E]
    routes = routing_weights
    if routing_slots is not None:
        routes = routing_weights[torch.as_tensor(list(routing_slots), dtype=torch.int64, device=x.device)]
    routes = routes.contiguous()
    ids = torch.arange(e, dtype=torch.int32, device=x.device).reshape(1, e)      # handle order = expert order
    plan = moe_ops.moe_plan(ids, e)
    gate, up, down = experts[0].gate, experts[0].up, experts[0].down
    hbuf = moe_ops.moe_gate_up(x, plan, None, None, gate.quant_type, up.quant_type, f, d, 0, 0,
                               gate_table=table[0], up_table=table[1], tables_aligned16=aligned)
    terms = moe_ops.moe_down(hbuf, routes, plan, None, down.quant_type, d, f, 0, down_table=table[2],
                             tables_aligned16=aligned)
    return moe_ops.moe_combine(terms, plan, d, out_dtype=torch.float32)
