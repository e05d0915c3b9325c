"""b200q: B200-native (sm_100a) kernels for MyLocal_LLM's packed-GGUF quantized inference path.

The public names mirror the reference's operator API (``mini_llm/ops`` and
``mini_llm/external``); device arrays are torch CUDA tensors and every operator runs the
hand-written CUDA kernels of ``libb200q.so`` through ctypes.
"""

from .quantized_weight import BLOCK_FORMATS, PackedGGUFWeight
from .quantized_linear import (
    SUPPORTED_GPU_PACKED_FORMATS,
    DevicePackedGGUFWeight,
    PackedExpertFFNInference,
    packed_to_device,
    quantized_linear,
    quantized_swiglu,
    supports_packed_gpu_type,
)

__all__ = [
    "BLOCK_FORMATS", "PackedGGUFWeight", "SUPPORTED_GPU_PACKED_FORMATS", "DevicePackedGGUFWeight",
    "PackedExpertFFNInference", "packed_to_device", "quantized_linear", "quantized_swiglu",
    "supports_packed_gpu_type",
]
