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

from .router_inference import RouterInference, expert_topk_forward, try_normalized_topk
from .experts_inference import (ExpertsInference, PackedExpertBank, ResidentExpertExecutor,
                                routed_experts_forward, synthetic_bank)
from .grouped_quantized_experts import (grouped_quantized_experts_forward,
                                        supports_grouped_quantized_experts)
from .moe_layer import PackedMoELayer, RMSNormInference
from .gguf_index import GGUFPackedIndex, project_gguf_linear, project_gguf_swiglu, resolve_gguf_weight

__all__ = [
    "RouterInference", "expert_topk_forward", "try_normalized_topk", "ExpertsInference", "PackedExpertBank",
    "ResidentExpertExecutor", "routed_experts_forward", "synthetic_bank", "grouped_quantized_experts_forward",
    "supports_grouped_quantized_experts", "PackedMoELayer", "RMSNormInference",
    "BLOCK_FORMATS", "PackedGGUFWeight", "SUPPORTED_GPU_PACKED_FORMATS", "DevicePackedGGUFWeight",
    "PackedExpertFFNInference", "packed_to_device", "quantized_linear", "quantized_swiglu",
    "supports_packed_gpu_type", "GGUFPackedIndex", "project_gguf_linear", "project_gguf_swiglu",
    "resolve_gguf_weight",
]
