"""Integer-dot mode: Q8_1 activations for packed linears (opt-in, separately toleranced).

Host-side mirror of the reference's Q8_1 activation codec (``mini_llm/ops/q8_1_gpu.py:30-58``:
``quantize_q8_1``) and of its mixed Q8 linear (``mini_llm/ops/mixed_q8_gpu.py:203-251``: ``q8_linear``).
The activations are quantised once to blocks of 32 int8 codes with an FP16 scale; the packed weight
codes then meet them in 4-way integer dots, which removes the per-weight floating-point decode that
bounds the Q4_K GEMV. The result differs from the FP32-activation path by the int8 rounding of the
activations (about 0.4 % of a block's largest value per element), so nothing selects this mode
implicitly: a caller asks for it by calling these functions.
"""

import ctypes

from . import _lib
from .quantized_linear import DevicePackedGGUFWeight

Q8_1_BLOCK_BYTES = 36
Q8_1_BLOCK_ELEMENTS = 32
SUPPORTED_Q8_1_WEIGHT_TYPES = frozenset({"Q4_K", "Q4_K_TILED", "Q5_K", "Q5_K_TILED"})


def _torch():
    import torch
    return torch


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def quantize_q8_1(x):
    """x ``[..., K]`` (FP32 / FP16 / BF16 CUDA tensor, K a multiple of 32) -> uint8 ``[rows, K/32, 36]``."""
    torch = _torch()
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("quantize_q8_1 expects a torch CUDA tensor")
    if not x.is_contiguous() or x.ndim < 1 or x.shape[-1] % Q8_1_BLOCK_ELEMENTS:
        raise ValueError("x must be contiguous with a last dimension that is a multiple of 32")
    name = str(x.dtype).replace("torch.", "")
    if name not in _lib.DTYPE_ID:
        raise TypeError("x must be FP32, FP16 or BF16")
    k = x.shape[-1]
    rows = x.numel() // k
    out = torch.empty((rows, k // Q8_1_BLOCK_ELEMENTS, Q8_1_BLOCK_BYTES), dtype=torch.uint8, device=x.device)
    if rows:
        _lib.call("b200q_quantize_q8_1", _ptr(x), _lib.DTYPE_ID[name], rows, k, _ptr(out), _lib.current_stream())
    return out


def q8_1_linear(blocks, weight, *, out_dtype=None):
    """``dequant(blocks) @ weight.T`` with integer dots; blocks from ``quantize_q8_1`` -> ``[rows, N]`` (FP32
    unless ``out_dtype`` says otherwise)."""
    torch = _torch()
    if not isinstance(weight, DevicePackedGGUFWeight):
        raise TypeError("Expected a DevicePackedGGUFWeight")
    if weight.quant_type not in SUPPORTED_Q8_1_WEIGHT_TYPES:
        raise NotImplementedError(f"No Q8_1 integer-dot kernel for {weight.quant_type}")
    n, k = weight.shape
    if (blocks.dtype != torch.uint8 or blocks.ndim != 3 or blocks.shape[1] * Q8_1_BLOCK_ELEMENTS != k
            or blocks.shape[2] != Q8_1_BLOCK_BYTES or not blocks.is_contiguous()):
        raise ValueError("Input K does not match packed weight K (expected uint8 [rows, K/32, 36] blocks)")
    rows = blocks.shape[0]
    out = torch.empty((rows, n), dtype=out_dtype or torch.float32, device=blocks.device)
    if rows:
        _lib.call("b200q_gemv_q8_1", _ptr(weight.data), _lib.FORMAT_ID[weight.quant_type], n, k, _ptr(blocks), rows,
                  _ptr(out), _lib.DTYPE_ID[str(out.dtype).replace("torch.", "")], _lib.current_stream())
    return out


def quantized_linear_q8_1(x, weight, *, out_dtype=None):
    """``quantized_linear`` in the integer-dot mode: quantise ``x`` to Q8_1, then ``q8_1_linear``; the output has
    x's leading shape and, by default, x's dtype."""
    y = q8_1_linear(quantize_q8_1(x), weight, out_dtype=out_dtype or x.dtype)
    return y.reshape(tuple(x.shape[:-1]) + (weight.shape[0],))
