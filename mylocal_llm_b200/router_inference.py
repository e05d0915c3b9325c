"""MoE router for inference: full softmax over all experts, top-k, optional renormalisation.

Host-side mirror of the reference's ``mini_llm/ops/router_inference.py`` (``RouterInference``
:10-61), ``mini_llm/ops/router.py`` (``expert_topk_forward`` :21-43) and
``mini_llm/ops/router_decode.py`` (``try_normalized_topk`` :247-273). The logits product and the
softmax/top-k both run as kernels of ``libb200q.so`` for any number of rows (the reference fuses
only the single-row case); selection order is descending logit, ties to the lower id, NaN last.
"""

import math

from . import moe_ops


def _torch():
    import torch
    return torch


def expert_topk_forward(logits, k, output_dtype=None, return_cache=True):
    """Softmax over all experts, then top-k *without* renormalisation.

    Returns ``(weights, indices, cache)`` like the reference; ``cache`` is always ``None`` here
    (it only serves the reference's training backward pass).
    """
    torch = _torch()
    if logits.ndim < 1 or not (1 <= int(k) <= int(logits.shape[-1])):
        raise ValueError("expert router expects 1 <= k <= n_experts")
    flat = logits.reshape(-1, logits.shape[-1]).float().contiguous()
    weights, ids = moe_ops.router_topk(flat, int(k), renormalize=False)
    lead = tuple(logits.shape[:-1])
    weights = weights.reshape(lead + (int(k),))
    if output_dtype is not None and output_dtype in (torch.float16, torch.bfloat16):
        weights = weights.to(output_dtype)
    return weights, ids.reshape(lead + (int(k),)), None


def try_normalized_topk(logits, k, normalization_floor):
    """Renormalised top-k of FP32 logits, or ``None`` when the arguments are outside the kernel's
    range (n <= 4096, k <= 32, finite positive floor) - the reference's decline contract."""
    torch = _torch()
    if (not isinstance(logits, torch.Tensor) or not logits.is_cuda or logits.dtype != torch.float32
            or not logits.is_contiguous() or logits.ndim < 1
            or not 1 <= logits.shape[-1] <= 4096 or not 1 <= k <= min(32, logits.shape[-1])
            or not (normalization_floor > 0 and math.isfinite(normalization_floor))):
        return None
    flat = logits.reshape(-1, logits.shape[-1])
    weights, ids = moe_ops.router_topk(flat, int(k), renormalize=True, floor=float(normalization_floor))
    shape = tuple(logits.shape[:-1]) + (int(k),)
    return weights.reshape(shape), ids.reshape(shape)


class RouterInference:
    """Full-softmax-then-top-k router; optional inference-only renormalisation.

    ``W_router`` is a contiguous FP32 ``[d_model, n_experts]`` CUDA tensor, ``b_router`` FP32
    ``[n_experts]`` or ``None``. ``forward`` takes ``[B, T, d_model]`` activations (FP32, FP16 or
    BF16) and returns ``(weights [B,T,k], ids [B,T,k] int64)``.
    """

    def __init__(self, d_model, n_experts, k, dtype="float32", *, renormalize_selected=False,
                 normalization_floor=1e-30):
        self.d_model = d_model
        self.n_experts = n_experts
        if not (1 <= int(k) <= int(n_experts)):
            raise ValueError("expert router expects 1 <= k <= n_experts")
        self.k = int(k)
        if not isinstance(renormalize_selected, bool):
            raise TypeError("renormalize_selected must be bool")
        if not math.isfinite(normalization_floor) or normalization_floor <= 0:
            raise ValueError("normalization_floor must be finite and positive")
        self.renormalize_selected = renormalize_selected
        self.normalization_floor = float(normalization_floor)
        self._w = None
        self._w_expert_major = None
        self.b_router = None

    @property
    def W_router(self):
        """FP32 ``[d_model, n_experts]`` weight (the reference's orientation)."""
        return self._w

    @W_router.setter
    def W_router(self, value):
        # Keep an expert-major [E, D] copy: the decode kernel gives every expert row its own warp.
        self._w = value
        self._w_expert_major = None if value is None else value.t().contiguous()

    def set_expert_major_weight(self, weight_t):
        """Use an ``[n_experts, d_model]`` weight directly (the orientation stored in GGUF files). The
        expert-major kernel reads four columns per load; other widths keep a ``[d_model, n_experts]`` copy."""
        self._w = None if weight_t.shape[1] % 4 == 0 else weight_t.t().contiguous()
        self._w_expert_major = weight_t

    def set_weights(self, router):
        self.W_router = router.W_router_param.data
        self.b_router = router.b_router_param.data

    def logits(self, x2d):
        if self._w_expert_major is not None and x2d.shape[1] % 4 == 0:
            return moe_ops.router_logits_t(x2d, self._w_expert_major, self.b_router)
        return moe_ops.router_logits(x2d, self._w, self.b_router)

    def forward(self, x):
        torch = _torch()
        batch, seq, _ = x.shape
        x2d = x.reshape(batch * seq, self.d_model)
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        logits = self.logits(x2d)
        weights, ids = moe_ops.router_topk(logits, self.k, renormalize=self.renormalize_selected,
                                           floor=self.normalization_floor)
        if x.dtype in (torch.float16, torch.bfloat16):
            weights = weights.to(x.dtype)
        return weights.reshape(batch, seq, self.k), ids.reshape(batch, seq, self.k)
