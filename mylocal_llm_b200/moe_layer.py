"""Packed sparse-MoE layer: renormalised routed SwiGLU experts plus a (sigmoid-gated) shared expert.

Mirrors the forward of the reference's ``Qwen3NextMoEInference``
(``mini_llm/external/qwen3next_moe.py:129-147``):

    weights, ids = router(hidden)                      # softmax over all E, top-k, renormalised
    routed       = experts(hidden, weights, ids)       # ascending-expert ordered FP32 sum
    shared       = down_sh( silu(hidden@gate_sh.T) * (hidden@up_sh.T) )
    out          = routed + shared * sigmoid(hidden @ shared_gate)

``shared_gate`` is optional: without it the shared expert is always on (weight 1), which is the
variant the benchmark configuration describes. The reference requires FP32 hidden states; this
layer also accepts BF16/FP16 (accumulation stays FP32, the output is rounded once).

``RMSNormInference`` mirrors ``mini_llm/ops/rmsnorm_inference.py:304-318,451-495,525-539``.
"""

import ctypes
import os

from . import _lib, moe_ops
from .experts_inference import ExpertsInference, PackedExpertBank, ResidentExpertExecutor
from .quantized_linear import (DevicePackedGGUFWeight, quantized_linear, quantized_swiglu, retile_enabled,
                               retile_gate_up, retile_weight)
from .router_inference import RouterInference


def _torch():
    import torch
    return torch


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _dtype_id(t):
    return _lib.DTYPE_ID[str(t.dtype).replace("torch.", "")]


class RMSNormInference:
    """``y = x / sqrt(mean(x^2) + eps) * gamma`` with FP32 math; optional fused residual add."""

    def __init__(self, d_model, eps=1e-6, dtype="float32"):
        self.d_model = int(d_model)
        self.eps = float(eps)
        self.dtype = dtype
        self.gamma = None

    def set_weights(self, gamma):
        self.gamma = gamma

    def _check(self, x):
        if self.gamma is None:
            raise RuntimeError("RMSNorm weights are not set")
        if x.shape[-1] != self.d_model or tuple(self.gamma.shape) != (self.d_model,):
            raise ValueError("RMSNorm expects [..., d_model] input and a [d_model] weight")
        if not x.is_contiguous() or not self.gamma.is_contiguous():
            raise ValueError("RMSNorm operands must be contiguous")

    def forward(self, x):
        """Output has x's shape and dtype."""
        torch = _torch()
        self._check(x)
        y = torch.empty_like(x)
        rows = x.numel() // self.d_model
        if rows:
            _lib.call("b200q_rmsnorm", _ptr(x), _dtype_id(x), _ptr(self.gamma), _dtype_id(self.gamma), rows,
                      self.d_model, self.eps, _ptr(y), _dtype_id(y), _lib.current_stream())
        return y

    def forward_residual(self, x):
        """Normalise an FP32 residual stream directly into the weight's dtype."""
        torch = _torch()
        self._check(x)
        y = torch.empty(x.shape, dtype=self.gamma.dtype, device=x.device)
        rows = x.numel() // self.d_model
        if rows:
            _lib.call("b200q_rmsnorm", _ptr(x), _dtype_id(x), _ptr(self.gamma), _dtype_id(self.gamma), rows,
                      self.d_model, self.eps, _ptr(y), _dtype_id(y), _lib.current_stream())
        return y

    def forward_residual_add(self, residual, branch, alpha=1.0):
        """``res = residual + alpha*branch`` (FP32), ``y = rmsnorm(res)`` in the weight's dtype."""
        torch = _torch()
        self._check(residual)
        if residual.dtype != torch.float32:
            raise TypeError("the residual stream must be FP32")
        if branch.shape != residual.shape or not branch.is_contiguous():
            raise ValueError("branch must be contiguous and shaped like the residual")
        res_out = torch.empty_like(residual)
        y = torch.empty(residual.shape, dtype=self.gamma.dtype, device=residual.device)
        rows = residual.numel() // self.d_model
        if rows:
            _lib.call("b200q_residual_rmsnorm", _ptr(residual), _ptr(branch), _dtype_id(branch), float(alpha),
                      _ptr(self.gamma), _dtype_id(self.gamma), rows, self.d_model, self.eps, _ptr(res_out), _ptr(y),
                      _dtype_id(y), _lib.current_stream())
        return res_out, y


class PackedMoELayer:
    """Router + routed expert bank + shared expert, all packed and resident in HBM."""

    def __init__(self, bank, router_weight, top_k, *, shared=None, shared_gate=None, layer_id=0,
                 normalization_floor=2.0 ** -14, executor=None):
        """bank: PackedExpertBank; router_weight: FP32 [D, E] CUDA tensor; shared: optional
        (gate, up, down) DevicePackedGGUFWeight triple; shared_gate: optional FP32 [D] vector."""
        if not isinstance(bank, PackedExpertBank):
            raise TypeError("bank must be a PackedExpertBank")
        self.shared_native = shared          # as given, before any conversion to a tile layout
        if retile_enabled() and executor is None:
            # Q6_K down projections are re-ordered once into the tile layout the fast kernel reads
            bank = bank.retiled()
            if shared is not None and len(shared) == 3 and isinstance(shared[2], DevicePackedGGUFWeight):
                gate_t, up_t = retile_gate_up(shared[0], shared[1])
                shared = (gate_t, up_t, retile_weight(shared[2]))
        self.bank = bank
        self.layer_id = int(layer_id)
        self.router = RouterInference(bank.d_model, bank.n_experts, top_k, renormalize_selected=True,
                                      normalization_floor=normalization_floor)
        self.router.W_router = router_weight
        self.router.b_router = None
        self.executor = executor or ResidentExpertExecutor({self.layer_id: bank})
        self.experts = ExpertsInference(bank.d_model, bank.d_ff, bank.n_experts, expert_executor=self.executor,
                                        layer_id=self.layer_id)
        if shared is not None:
            if len(shared) != 3 or not all(isinstance(w, DevicePackedGGUFWeight) for w in shared):
                raise TypeError("shared expert must be three DevicePackedGGUFWeight projections")
            if shared[0].shape != shared[1].shape or shared[2].shape != (shared[0].shape[1], shared[0].shape[0]):
                raise ValueError("shared expert shapes must be gate/up [F, D], down [D, F]")
        self.shared = shared
        self.shared_gate = shared_gate
        # A shared expert with the routed experts' shape and formats runs through the grouped kernels
        # as expert id E (the highest id, hence added last), addressed through pointer tables.
        self._tables = None
        # B200Q_FUSE_PLAN=0: separate top-k and plan launches for a one-row step as well
        self.fuse_row_plan = os.environ.get("B200Q_FUSE_PLAN", "1") != "0"
        if shared is not None and all(
                w.shape == ref_shape and w.quant_type == ref_type for w, ref_shape, ref_type in zip(
                    shared, ((bank.d_ff, bank.d_model), (bank.d_ff, bank.d_model), (bank.d_model, bank.d_ff)),
                    (bank.gate_type, bank.up_type, bank.down_type))) and bank.n_experts < 1024:
            self._tables = bank.pointer_tables(extra=shared)

    def can_fuse_residual_norm(self):
        """Whether ``forward(hidden, residual_norm=...)`` is available: the resident executor's grouped
        path with at most 16 terms per row (top-k plus the shared expert)."""
        terms = self.router.k + (1 if self._tables is not None else 0)
        return isinstance(self.executor, ResidentExpertExecutor) and terms <= moe_ops.COMBINE_NORM_MAX_K

    def forward(self, hidden, residual_norm=None):
        """hidden [B, T, D] -> [B, T, D] in hidden's dtype. With ``residual_norm = (norm, residual)``
        (``RMSNormInference``, FP32 residual stream shaped like ``hidden``) the layer's last kernel also
        adds the branch to the residual and normalises it, and the result is ``(new residual, normalised
        activations)``: the same bits as ``norm.forward_residual_add(residual, self.forward(hidden))``."""
        torch = _torch()
        if not isinstance(hidden, torch.Tensor) or not hidden.is_cuda:
            raise TypeError("MoE layer requires a CUDA tensor")
        if hidden.ndim != 3 or hidden.shape[0] < 1 or hidden.shape[-1] != self.bank.d_model:
            raise ValueError("hidden must have shape [positive batch,time,d_model]")
        if residual_norm is not None and not self.can_fuse_residual_norm():
            raise NotImplementedError("this layer cannot fuse the residual add and norm into its combine")
        if not hidden.shape[1]:
            if residual_norm is not None:
                return residual_norm[0].forward_residual_add(residual_norm[1], torch.empty_like(hidden))
            return torch.empty_like(hidden)
        batch, seq, d = hidden.shape
        fused = {}
        if residual_norm is not None:
            norm, residual = residual_norm
            if residual.shape != hidden.shape or residual.dtype != torch.float32 or not residual.is_contiguous():
                raise ValueError("the residual stream must be contiguous FP32 and shaped like hidden")
            fused = {"residual_norm": (norm, residual.reshape(batch * seq, d))}

        def shaped(out):
            if residual_norm is None:
                return out.reshape(batch, seq, d)
            return out[0].reshape(batch, seq, d), out[1].reshape(batch, seq, d)

        x2d = hidden.reshape(batch * seq, d)
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        logits = self.router.logits(x2d)
        if self._tables is not None:
            scale = moe_ops.shared_gate(x2d, self.shared_gate) if self.shared_gate is not None else None
            if (x2d.shape[0] == 1 and self.fuse_row_plan and isinstance(self.executor, ResidentExpertExecutor)
                    and self.bank.n_experts <= 1024 and self.router.k <= 31):
                # one token: the top-k kernel writes the routing plan itself (one launch fewer)
                weights, ids, plan = moe_ops.router_topk_plan_row(
                    logits, self.router.k, self.bank.n_experts + 1, renormalize=True,
                    floor=self.router.normalization_floor, extra_id=self.bank.n_experts, extra_weight=scale)
                fused = dict(fused, plan=plan)
            else:
                weights, ids = moe_ops.router_topk(logits, self.router.k, renormalize=True,
                                                   floor=self.router.normalization_floor,
                                                   extra_id=self.bank.n_experts, extra_weight=scale)
            tables, aligned = self._tables
            out = self.executor.forward_routed(self.layer_id, x2d, weights, ids, out_dtype=hidden.dtype,
                                               tables=tables, tables_aligned16=aligned,
                                               n_experts=self.bank.n_experts + 1, **fused)
            return shaped(out)
        weights, ids = moe_ops.router_topk(logits, self.router.k, renormalize=True,
                                           floor=self.router.normalization_floor)
        extra = extra_scale = None
        if self.shared is not None:
            gate, up, down = self.shared
            # (the GEMV kernels whatever the number of rows: a layer's result must not depend on how a batch is
            # split over calls or ranks, and the tensor-core GEMM rounds its weights to BF16)
            shared_hidden = quantized_swiglu(x2d, gate, up, out_dtype=torch.float32, allow_gemm=False)
            extra = quantized_linear(shared_hidden, down, allow_gemm=False)
            if self.shared_gate is not None:
                extra_scale = moe_ops.shared_gate(x2d, self.shared_gate)
        out = self.executor.forward_routed(self.layer_id, x2d, weights, ids, extra=extra, extra_scale=extra_scale,
                                           out_dtype=hidden.dtype, **fused)
        return shaped(out)
