"""ctypes binding of ``libb200q.so`` (the C ABI declared in ``include/b200q.h``).

The library is the only compute back end of this package: there is no Triton path, no
PyTorch-eager path and no CPU fallback. If the shared object is missing the loader tries one
in-tree nvcc build and otherwise raises; nothing silently degrades.
"""

import ctypes
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# B200Q_LIBRARY points the loader at another build of the same ABI (A/B measurements).
LIB_PATH = Path(os.environ.get("B200Q_LIBRARY") or _PKG / "libb200q.so")

FORMAT_ID = {"Q8_0": 0, "Q4_0": 1, "Q4_K": 2, "Q3_K": 3, "Q5_K": 4, "Q6_K": 5, "Q6_K_TILED": 21, "Q4_K_TILED": 22, "Q8_0_TILED": 23, "Q5_K_TILED": 24}
DTYPE_ID = {"float32": 0, "float16": 1, "bfloat16": 2}

_c_int, _c_i64, _c_f32, _ptr = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p

# name -> argument types (all return int unless noted); mirrors include/b200q.h
SIGNATURES = {
    "b200q_abi_version": [],
    "b200q_device_status": [_ptr],
    "b200q_device_status_clear": [],
    "b200q_dequantize": [_ptr, _c_int, _c_i64, _c_int, _ptr, _ptr],
    "b200q_gemv": [_ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr, _c_int, _ptr],
    "b200q_quantize_q8_1": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr],
    "b200q_gemv_q8_1": [_ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr, _c_int, _ptr],
    "b200q_gemm": [_ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr, _c_int, _ptr],
    "b200q_gemm_supported": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "b200q_gemv_norm_supported": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "b200q_gemv_norm": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _c_f32, _ptr, _c_int, _c_f32, _c_int, _ptr, _ptr,
                        _c_int, _ptr],
    "b200q_gemm_workspace_bytes": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "b200q_gemm_ws": [_ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr, _c_int, _ptr, _c_i64, _ptr],
    "b200q_swiglu": [_ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr, _c_int, _ptr],
    "b200q_expert_ffn_static": [_ptr, _c_int, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr,
                                _c_int, _ptr],
    "b200q_rmsnorm": [_ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _c_f32, _ptr, _c_int, _ptr],
    "b200q_residual_rmsnorm": [_ptr, _ptr, _c_int, _c_f32, _ptr, _c_int, _c_int, _c_int, _c_f32, _ptr, _ptr,
                               _c_int, _ptr],
    "b200q_router_logits": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_router_logits_t": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_router_topk_ex": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr],
    "b200q_shared_gate": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr],
    "b200q_router_topk_plan_row": [_ptr, _c_int, _c_int, _c_int, _c_f32, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr,
                                   _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_router_topk": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_f32, _ptr, _ptr, _ptr],
    "b200q_moe_plan": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                       _ptr, _c_int, _ptr, _ptr],
    "b200q_moe_gate_up": [_ptr, _c_i64, _c_int, _ptr, _c_i64, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr,
                          _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_moe_decode_stack_workspace": [_c_int, _c_int, _c_int, _c_int],
    "b200q_moe_decode_stack": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f32, _c_int, _c_int, _ptr, _c_int,
                               _c_f32, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "b200q_q5k_retile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_q5k_untile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_moe_token_image_bytes": [_c_int, _c_int],
    "b200q_moe_token_images": [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr],
    "b200q_moe_gate_up_images": [_ptr, _c_i64, _c_int, _ptr, _c_i64, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr,
                                 _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_moe_plan_ex": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                          _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_moe_combine_ids": [_ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr],
    "b200q_moe_plan_ep": [_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr],
    "b200q_moe_down_peer": [_ptr, _c_i64, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                            _ptr, _c_int, _ptr, _c_int, _ptr],
    "b200q_q4k_retile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_q4k_untile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_rope_kv_store": [_ptr, _ptr, _ptr, _c_i64, _c_i64, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr],
    "b200q_silu_mul": [_ptr, _c_int, _c_int, _ptr, _c_int, _ptr],
    "b200q_decode_attention": [_ptr, _c_i64, _ptr, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f32,
                               _ptr, _c_int, _ptr],
    "b200q_gemv_silu_supported": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "b200q_gemv_silu": [_ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _c_int, _ptr, _c_int, _ptr],
    "b200q_rope_attention": [_ptr, _ptr, _ptr, _c_i64, _c_i64, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int,
                             _c_int, _c_int, _ptr, _ptr, _c_int, _c_f32, _ptr, _c_int, _ptr],
    "b200q_q8_0_retile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_q8_0_untile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_q6k_retile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_q6k_untile": [_ptr, _ptr, _c_i64, _c_int, _ptr],
    "b200q_peer_alloc": [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), _ptr],
    "b200q_peer_open": [_ptr, ctypes.POINTER(ctypes.c_void_p)],
    "b200q_peer_close": [_ptr],
    "b200q_peer_free": [_ptr],
    "b200q_peer_barrier": [_ptr, _c_int, _c_int, _c_int, _ptr],
    "b200q_peer_push3": [_ptr, ctypes.c_size_t, ctypes.c_size_t, _ptr, ctypes.c_size_t, ctypes.c_size_t, _ptr,
                         ctypes.c_size_t, ctypes.c_size_t, _ptr, _c_int, _ptr],
    "b200q_peer_push_rows": [_ptr, ctypes.c_size_t, _ptr, ctypes.c_size_t, _c_int, _ptr],
    "b200q_moe_down": [_ptr, _c_i64, _c_int, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                       _c_int, _ptr, _ptr],
    "b200q_moe_combine": [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr],
    "b200q_moe_combine_norm": [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr, _c_f32, _ptr, _c_int,
                               _c_f32, _ptr, _ptr, _c_int, _ptr],
}

_LOCK = threading.Lock()
_LIB = None


class B200QError(RuntimeError):
    """A b200q entry point returned a non-zero code."""


def load():
    """Load (building once if absent) and return the ctypes library handle."""
    global _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not LIB_PATH.exists():
            from . import build as _build
            _build.build()
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_i64 if name in ("b200q_moe_decode_stack_workspace", "b200q_gemm_workspace_bytes") else _c_int
        lib.b200q_last_error.argtypes = []
        lib.b200q_last_error.restype = ctypes.c_char_p
        _LIB = lib
        return lib


def last_error():
    return (load().b200q_last_error() or b"").decode("utf-8", "replace")


def call(name, *args):
    """Call an entry point; map its return code to the reference's exception types."""
    rc = getattr(load(), name)(*args)
    if rc == 0:
        return
    message = f"{name}: {last_error()}"
    if rc == 1:
        raise ValueError(message)
    if rc == 3:
        raise NotImplementedError(message)
    raise B200QError(message)


def current_stream():
    """Raw handle of the framework's current CUDA stream (the launch stream of every call)."""
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def clear_device_status():
    call("b200q_device_status_clear")


def device_status():
    """Blocking read of the device status word (0 = no kernel gave up on a wait)."""
    value = ctypes.c_int(0)
    call("b200q_device_status", ctypes.byref(value))
    return value.value
