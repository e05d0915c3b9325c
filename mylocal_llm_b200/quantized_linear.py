"""Quantized GGUF linear / SwiGLU / expert-FFN operators on device-resident packed bytes.

Host-side mirror of the reference's ``mini_llm/ops/quantized_linear.py``:

* ``DevicePackedGGUFWeight`` (:45-74), ``packed_to_device`` (:77-86),
  ``supports_packed_gpu_type`` / ``SUPPORTED_GPU_PACKED_FORMATS`` (:34-41)
* ``quantized_linear(x, weight, *, block_k=512, cpu_packed_backend="reference")`` (:272-335)
* ``quantized_swiglu(x, gate, up, *, block_k=512)`` (:338-400)
* ``PackedExpertFFNInference(gate, up, down, *, fuse_gate_up=True).forward(x)`` (:403-424)

Contract kept: ``y[..., N] = x[..., K] @ W[N, K].T`` with FP32 accumulation, output dtype =
activation dtype, activations contiguous 2-D or 3-D, packed bytes never expanded. Device
arrays are torch CUDA tensors (the reference uses CuPy); the launch stream is torch's current
stream. ``block_k`` is validated for error parity and otherwise unused (the kernels choose
their own tiling). A host ``PackedGGUFWeight`` is rejected: there is no CPU execution path.
"""

from dataclasses import dataclass
import ctypes
import math

import os

import numpy as np

from . import _lib
from .quantized_weight import BLOCK_FORMATS, DEVICE_LAYOUTS, PackedGGUFWeight, block_format

SUPPORTED_GPU_PACKED_FORMATS = frozenset(name for name in _lib.FORMAT_ID if name in BLOCK_FORMATS)
_BLOCK_K = (256, 512, 1024)


def supports_packed_gpu_type(quant_type):
    """Kernel format support, independent of whether a GPU is present."""
    return quant_type in SUPPORTED_GPU_PACKED_FORMATS


def _torch():
    import torch
    return torch


def _is_cuda_tensor(x):
    torch = _torch()
    return isinstance(x, torch.Tensor) and x.is_cuda


def _dtype_id(t):
    name = str(t.dtype).replace("torch.", "")
    if name not in _lib.DTYPE_ID:
        raise TypeError("GPU input must be FP16, BF16, or FP32")
    return _lib.DTYPE_ID[name]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@dataclass(frozen=True)
class DevicePackedGGUFWeight:
    """GPU-resident packed matrix ``[N, K]``; same layout contract as ``PackedGGUFWeight``."""

    data: object
    shape: tuple
    quant_type: str

    def __post_init__(self):
        if self.quant_type not in BLOCK_FORMATS and self.quant_type not in DEVICE_LAYOUTS:
            raise ValueError(f"Unsupported GGUF type {self.quant_type}")
        if self.quant_type not in _lib.FORMAT_ID:
            raise NotImplementedError(f"No packed GPU kernel for {self.quant_type}")
        torch = _torch()
        if not isinstance(self.data, torch.Tensor) or self.data.dtype != torch.uint8 or not self.data.is_cuda:
            raise TypeError("Device packed bytes must be a torch CUDA uint8 tensor")
        if not self.data.is_contiguous():
            raise ValueError("Device packed bytes must be contiguous")
        shape = tuple(int(i) for i in self.shape)
        if len(shape) != 2 or min(shape) <= 0:
            raise ValueError("Device packed linear weights must be [N, K]")
        qk, qb = block_format(self.quant_type)
        if shape[-1] % qk or int(self.data.numel()) != math.prod(shape) // qk * qb:
            raise ValueError("Invalid packed byte length or K block alignment")
        object.__setattr__(self, "shape", shape)

    @property
    def nbytes(self):
        return int(self.data.numel())


def packed_bytes_to_device(raw):
    """Copy a host uint8 array to the current CUDA device (one transfer, no decoding)."""
    torch = _torch()
    if not torch.cuda.is_available():
        raise RuntimeError("Packed GPU weights require a CUDA device")
    host = np.ascontiguousarray(raw, dtype=np.uint8)
    if not host.flags.writeable:
        # read-only file mappings: the tensor is only the source of the copy and is never written
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)
            return torch.from_numpy(host).cuda()
    return torch.from_numpy(host).cuda()


def packed_to_device(weight):
    """Transfer the packed bytes of one matrix/expert to HBM once."""
    if not isinstance(weight, PackedGGUFWeight) or len(weight.shape) != 2:
        raise TypeError("Expected a two-dimensional PackedGGUFWeight")
    if not supports_packed_gpu_type(weight.quant_type):
        raise NotImplementedError(f"No packed GPU kernel for {weight.quant_type}")
    return DevicePackedGGUFWeight(packed_bytes_to_device(weight.data), weight.shape, weight.quant_type)


# The tiled kernel keeps the activation fragments of the whole K range in shared memory (two FP16
# planes for FP32 activations): 4096 is the largest K that fits for every activation type.
TILED_MAX_K = 4096


def retile_enabled():
    """Whether uploads of Q6_K down projections are re-ordered into the tile layout (default on;
    ``B200Q_RETILE=0`` keeps the native GGUF bytes and the kernels that read them)."""
    import os
    return os.environ.get("B200Q_RETILE", "1") != "0"


_RETILE = {"Q6_K": ("b200q_q6k_retile", "Q6_K_TILED"), "Q4_K": ("b200q_q4k_retile", "Q4_K_TILED"),
           "Q5_K": ("b200q_q5k_retile", "Q5_K_TILED"),
           "Q8_0": ("b200q_q8_0_retile", "Q8_0_TILED")}
_UNTILE = {"Q6_K_TILED": "b200q_q6k_untile", "Q4_K_TILED": "b200q_q4k_untile", "Q8_0_TILED": "b200q_q8_0_untile",
           "Q5_K_TILED": "b200q_q5k_untile"}


def retile_bytes(data, rows, k, quant_type):
    """Native ``quant_type`` bytes of a ``[rows, k]`` matrix (or a bank of experts, ``rows`` = all
    rows) -> new tensor in the 16-row tile layout (same size; lossless, see ``untile_bytes``)."""
    torch = _torch()
    out = torch.empty_like(data)
    _lib.call(_RETILE[quant_type][0], _ptr(data), _ptr(out), int(rows), int(k), _lib.current_stream())
    return out


def untile_bytes(data, rows, k, tiled_type):
    """Inverse of ``retile_bytes``: restores the GGUF bytes bit for bit."""
    torch = _torch()
    out = torch.empty_like(data)
    _lib.call(_UNTILE[tiled_type], _ptr(data), _ptr(out), int(rows), int(k), _lib.current_stream())
    return out


def retile_q6k(data, rows, k):
    return retile_bytes(data, rows, k, "Q6_K")


def untile_q6k(data, rows, k):
    return untile_bytes(data, rows, k, "Q6_K_TILED")


def can_retile(quant_type, rows, k, force=False):
    return quant_type in _RETILE and rows % 16 == 0 and k % 256 == 0 and (k <= TILED_MAX_K or force)


def retile_weight(weight, force=False):
    """``DevicePackedGGUFWeight`` in the tile layout when its type has one (Q4_K, Q5_K, Q6_K, Q8_0) and the
    shape allows it (rows a multiple of 16, K a multiple of 256 and <= TILED_MAX_K); otherwise the
    weight itself. ``force`` lifts the K limit for callers that only ever pass 16-bit activations
    (Q4_K and Q8_0 up to K = 8192)."""
    if not can_retile(weight.quant_type, weight.shape[0], weight.shape[1], force):
        return weight
    if weight.quant_type == "Q6_K" and weight.shape[1] > TILED_MAX_K:
        return weight
    return DevicePackedGGUFWeight(retile_bytes(weight.data, weight.shape[0], weight.shape[1], weight.quant_type),
                                  weight.shape, _RETILE[weight.quant_type][1])


def retile_gate_up(gate, up, force=False):
    """Gate / up pair for the fused SwiGLU launch: both in the tile layout when the fused kernel reads
    it (Q4_K or Q5_K for both), otherwise both unchanged."""
    if gate.quant_type == up.quant_type and gate.quant_type in ("Q4_K", "Q5_K"):
        gate_t, up_t = retile_weight(gate, force), retile_weight(up, force)
        if gate_t.quant_type == up_t.quant_type:
            return gate_t, up_t
    return gate, up


def dequantize_device(data, rows, k, quant_type):
    """FP32 ``[rows, k]`` CUDA tensor decoded from packed device bytes (verification helper)."""
    torch = _torch()
    if quant_type in DEVICE_LAYOUTS:
        data, quant_type = untile_bytes(data, rows, k, quant_type), DEVICE_LAYOUTS[quant_type]
    out = torch.empty((rows, k), dtype=torch.float32, device=data.device)
    _lib.call("b200q_dequantize", _ptr(data), _lib.FORMAT_ID[quant_type], rows, k, _ptr(out),
              _lib.current_stream())
    return out


def _check_activation(x, what="Packed linear input"):
    if isinstance(x, np.ndarray):
        return
    if not _is_cuda_tensor(x):
        raise TypeError(f"{what} must be a NumPy array or a torch CUDA tensor")


def quantized_linear(x, weight, *, block_k=512, cpu_packed_backend="reference", out_dtype=None, allow_gemm=True):
    """``x @ weight.T`` for packed GGUF ``[out_features, in_features]`` on the GPU.

    ``out_dtype`` (an addition to the reference signature) selects the output element type;
    by default the output has the activation dtype, as in the reference. ``allow_gemm=False`` keeps the call on
    the GEMV kernels (exact products) whatever the number of tokens: for callers whose result must not depend on
    how a batch is split."""
    _check_activation(x)
    if x.ndim not in (2, 3):
        raise ValueError("Expected x as [M, K] or [B, T, K]")
    if x.shape[-1] != weight.shape[-1]:
        raise ValueError("Input K does not match packed weight K")
    if len(weight.shape) != 2:
        raise ValueError("Packed linear weights must be [N, K]")
    if isinstance(weight, PackedGGUFWeight):
        raise RuntimeError("Host-packed weights have no execution path here (no CPU fallback); "
                           "upload them once with packed_to_device()")
    if not isinstance(weight, DevicePackedGGUFWeight):
        raise TypeError("Expected PackedGGUFWeight or DevicePackedGGUFWeight")
    if not _is_cuda_tensor(x):
        raise TypeError("Device-packed weight requires a torch CUDA activation tensor (NumPy input given)")
    if not x.is_contiguous():
        raise ValueError("GPU input must be a contiguous tensor")
    dt = _dtype_id(x)
    if block_k not in _BLOCK_K:
        raise ValueError("block_k must be 256, 512 or 1024")
    if x.device != weight.data.device:
        raise ValueError("activation and packed weight must be on the same CUDA device")
    torch = _torch()
    n, k = weight.shape
    m = int(x.numel()) // k
    out = torch.empty((m, n), dtype=out_dtype or x.dtype, device=x.device)
    if m and allow_gemm and _use_gemm(weight, x, m, n, k, dt):
        fmt = _lib.FORMAT_ID[weight.quant_type]
        # shapes with few weight-row tiles split K over several CTAs, given scratch for the partial results
        nbytes = int(_lib.load().b200q_gemm_workspace_bytes(fmt, n, k, dt, m))
        if nbytes and os.environ.get("B200Q_GEMM_SPLITK", "1") != "0":
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
            _lib.call("b200q_gemm_ws", _ptr(weight.data), fmt, n, k, _ptr(x), dt, m, _ptr(out), _dtype_id(out),
                      _ptr(scratch), nbytes, _lib.current_stream())
        else:
            _lib.call("b200q_gemm", _ptr(weight.data), fmt, n, k, _ptr(x), dt, m, _ptr(out), _dtype_id(out),
                      _lib.current_stream())
    elif m:
        _lib.call("b200q_gemv", _ptr(weight.data), _lib.FORMAT_ID[weight.quant_type], n, k, _ptr(x), dt, m,
                  _ptr(out), _dtype_id(out), _lib.current_stream())
    return out.reshape(tuple(x.shape[:-1]) + (n,))


# Tokens from which the tensor-core GEMM beats the GEMV kernels: more than one 8-token tile. A GEMV pass over two
# tiles (9-16 tokens) reads the weights once but takes 21-29 us on the [8192 x 2048] shapes where the GEMM needs
# 12-18 us (a 1.7B Llama step at batch 16: 4167 -> 5883 tokens/s); one tile (<= 8 tokens) stays on the GEMV kernels
# with their exact products.
GEMM_MIN_TOKENS = {"Q4_K": 9, "Q5_K": 9, "Q6_K": 9, "Q8_0": 9}


# quantized_swiglu: from three 8-token passes on, two GEMMs and an element-wise kernel beat the fused GEMV passes.
SWIGLU_GEMM_MIN_TOKENS = 17


def _use_gemm(weight, x, m, n, k, dt):
    """Enough tokens of BF16 activations on a GGUF-layout weight go to the tcgen05 GEMM (``b200q_gemm``:
    weights read once, BF16-weight precision); everything else stays on the GEMV kernels (exact
    products, FP32 / FP16 activations, device tile layouts). ``B200Q_GEMM=0`` keeps every call on the
    GEMV path."""
    import os
    if (weight.quant_type in DEVICE_LAYOUTS or m < GEMM_MIN_TOKENS.get(weight.quant_type, 1 << 30)
            or os.environ.get("B200Q_GEMM", "1") == "0" or os.environ.get("B200Q_KERNEL", "auto") != "auto"):
        return False
    if x.data_ptr() % 16 or weight.data.data_ptr() % (4 if weight.quant_type == "Q8_0" else 2):
        return False
    return bool(_lib.load().b200q_gemm_supported(_lib.FORMAT_ID[weight.quant_type], n, k, dt, m))


def quantized_swiglu(x, gate, up, *, block_k=512, out_dtype=None, allow_gemm=True):
    """``SiLU(x @ gate.T) * (x @ up.T)`` in one launch; gate/up formats may differ."""
    if not isinstance(gate, (PackedGGUFWeight, DevicePackedGGUFWeight)) or not isinstance(
            up, (PackedGGUFWeight, DevicePackedGGUFWeight)):
        raise TypeError("gate and up must be packed GGUF weights")
    if type(gate) is not type(up):
        raise TypeError("gate and up must both be host-packed or both device-packed")
    if len(gate.shape) != 2 or up.shape != gate.shape:
        raise ValueError("gate/up must share two-dimensional [F,K] shape")
    _check_activation(x, "Quantized SwiGLU input")
    if x.ndim not in (2, 3):
        raise ValueError("Expected x as [M,K] or [B,T,K]")
    f, k = gate.shape
    if x.shape[-1] != k:
        raise ValueError("Input K does not match gate/up K")
    if isinstance(gate, PackedGGUFWeight):
        raise RuntimeError("Host-packed gate/up have no execution path here (no CPU fallback); "
                           "upload them once with packed_to_device()")
    if not _is_cuda_tensor(x) or not x.is_contiguous():
        raise ValueError("GPU activations must be a contiguous torch CUDA tensor")
    dt = _dtype_id(x)
    if block_k not in _BLOCK_K:
        raise ValueError("block_k must be 256, 512 or 1024")
    torch = _torch()
    m = int(x.numel()) // k
    out = torch.empty((m, f), dtype=out_dtype or x.dtype, device=x.device)
    if (allow_gemm and m >= SWIGLU_GEMM_MIN_TOKENS and _use_gemm(gate, x, m, f, k, dt)
            and _use_gemm(up, x, m, f, k, dt)):
        # many BF16 tokens on GGUF-layout weights: the two projections on the tensor-core GEMM (weights read once
        # instead of once per 8-token pass), then the element-wise SiLU(gate) * up of the fused kernel
        x2d = x.reshape(m, k)
        gu = torch.cat([quantized_linear(x2d, gate, out_dtype=torch.float32),
                        quantized_linear(x2d, up, out_dtype=torch.float32)], dim=1)
        _lib.call("b200q_silu_mul", _ptr(gu), m, f, _ptr(out), _dtype_id(out), _lib.current_stream())
    elif m:
        _lib.call("b200q_swiglu", _ptr(gate.data), _lib.FORMAT_ID[gate.quant_type], _ptr(up.data),
                  _lib.FORMAT_ID[up.quant_type], f, k, _ptr(x), dt, m, _ptr(out), _dtype_id(out),
                  _lib.current_stream())
    return out.reshape(tuple(x.shape[:-1]) + (f,))


class PackedExpertFFNInference:
    """Three packed projections of one SwiGLU expert (gate/up ``[F, D]``, down ``[D, F]``)."""

    def __init__(self, gate, up, down, *, fuse_gate_up=True):
        self.gate, self.up, self.down = gate, up, down
        self.fuse_gate_up = bool(fuse_gate_up)
        if gate.shape != up.shape:
            raise ValueError("Gate and up projections must have identical dimensions")
        if down.shape != (gate.shape[1], gate.shape[0]):
            raise ValueError("Down projection dimensions must be transposed")

    def forward(self, x):
        if self.fuse_gate_up:
            h = quantized_swiglu(x, self.gate, self.up)
        else:
            torch = _torch()
            g = quantized_linear(x, self.gate).float()
            u = quantized_linear(x, self.up).float()
            h = (torch.nn.functional.silu(g) * u).to(x.dtype)
        return quantized_linear(h.contiguous(), self.down)
