"""CPU-side checks: the C ABI library loads and exports what include/b200q.h declares, host
validation raises the reference's exception types before any launch, quantisers emit valid
blocks. No compute call is made here (there is no GPU in this test tier)."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import (BLOCK_FORMATS, PackedExpertFFNInference, PackedGGUFWeight, packed_to_device,
                              quantized_linear, quantized_swiglu, supports_packed_gpu_type, _lib)
from mylocal_llm_b200.quantize import quantize, random_packed

ROOT = Path(__file__).resolve().parent.parent
FORMATS = ("Q8_0", "Q4_K", "Q5_K", "Q6_K")


def declared_symbols():
    text = (ROOT / "include" / "b200q.h").read_text()
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert "b200q_gemv" in names and "b200q_moe_gate_up" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200q.h but not exported"
    assert lib.b200q_abi_version() >= 1
    # every binding in the Python table is declared in the header
    for name in _lib.SIGNATURES:
        assert name in names


def test_entry_points_validate_before_launching():
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    assert lib.b200q_gemv(null, 2, 8, 256, one, 0, 1, one, 0, null) == 1
    assert lib.b200q_gemv(one, 9, 8, 256, one, 0, 1, one, 0, null) == 1          # unknown format
    assert lib.b200q_gemv(one, 2, 8, 255, one, 0, 1, one, 0, null) == 1          # K not block aligned
    assert lib.b200q_gemv(one, 2, 8, 256, one, 7, 1, one, 0, null) == 1          # bad dtype
    assert b"gemv" in lib.b200q_last_error()
    assert lib.b200q_router_topk(one, 1, 5000, 4, 1, 1e-4, one, one, null) == 1   # n > 4096
    assert lib.b200q_router_topk(one, 1, 16, 33, 1, 1e-4, one, one, null) == 1    # k > 32
    assert lib.b200q_dequantize(one, 2, 4, 100, one, null) == 1
    with pytest.raises(ValueError):
        _lib.call("b200q_rmsnorm", null, 0, null, 0, 1, 8, 1e-5, null, 0, null)


def test_block_formats_and_support_table():
    # the six FP32-lane formats of the reference's packed GPU path (mini_llm/ops/quantized_linear.py:34)
    assert BLOCK_FORMATS == {"Q8_0": (32, 34), "Q4_0": (32, 18), "Q3_K": (256, 110), "Q4_K": (256, 144),
                             "Q5_K": (256, 176), "Q6_K": (256, 210)}
    assert all(supports_packed_gpu_type(f) for f in BLOCK_FORMATS)
    assert not supports_packed_gpu_type("IQ2_S")


def test_packed_weight_validation_and_zero_copy_slices():
    for fmt, (block, nbytes) in BLOCK_FORMATS.items():
        with pytest.raises(ValueError, match="innermost"):
            PackedGGUFWeight(np.zeros(nbytes, np.uint8), (2, block // 2), fmt)
        with pytest.raises(ValueError, match="expected"):
            PackedGGUFWeight(np.zeros(nbytes - 1, np.uint8), (1, block), fmt)
    with pytest.raises(ValueError, match="Unsupported"):
        PackedGGUFWeight(np.zeros(1, np.uint8), (1, 32), "IQ1_S")
    bank = random_packed("Q5_K", (3, 4, 512), seed=49)
    one = bank.select_outer(1)
    assert one.shape == (4, 512) and one.nbytes == 4 * 2 * 176
    assert np.shares_memory(one.data, bank.data)
    with pytest.raises(IndexError):
        bank.select_outer(3)
    with pytest.raises(ValueError):
        bank.select_outer(0).matvec_reference(np.zeros(3))


def test_operator_argument_errors_match_the_reference_types():
    w = random_packed("Q4_K", (2, 256), seed=1)
    with pytest.raises(ValueError, match="Input K"):
        quantized_linear(np.zeros((2, 128), np.float32), w)
    with pytest.raises(ValueError, match="Expected x"):
        quantized_linear(np.zeros((256,), np.float32), w)
    with pytest.raises(TypeError, match="NumPy"):
        quantized_linear([[0] * 256], w)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        quantized_linear(np.zeros((1, 256), np.float32), w)
    with pytest.raises(TypeError, match="packed"):
        quantized_swiglu(np.zeros((1, 256), np.float32), np.zeros((2, 256)), w)
    with pytest.raises(ValueError, match="gate/up"):
        quantized_swiglu(np.zeros((1, 256), np.float32), w, random_packed("Q4_K", (3, 256), seed=2))
    with pytest.raises(ValueError, match="K"):
        quantized_swiglu(np.zeros((1, 512), np.float32), w, w)
    with pytest.raises(TypeError):
        packed_to_device(np.zeros(4))
    with pytest.raises(ValueError, match="identical"):
        PackedExpertFFNInference(w, random_packed("Q4_K", (3, 256), seed=2), w)
    with pytest.raises(ValueError, match="transposed"):
        PackedExpertFFNInference(w, w, w)


@pytest.mark.parametrize("fmt", FORMATS)
def test_quantisers_emit_valid_blocks_close_to_the_source(fmt):
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (6, 1024)).astype(np.float32)
    packed = quantize(w, fmt)
    assert packed.nbytes == 6 * 1024 // BLOCK_FORMATS[fmt][0] * BLOCK_FORMATS[fmt][1]
    dense = po.dequantize(packed.data, packed.shape, fmt)
    bound = {"Q8_0": 0.005, "Q4_K": 0.08, "Q5_K": 0.04, "Q6_K": 0.03}[fmt]
    assert np.abs(dense - w).max() <= bound * np.abs(w).max()
    zeros = quantize(np.zeros((1, 256), np.float32), fmt)
    np.testing.assert_array_equal(po.dequantize(zeros.data, zeros.shape, fmt), np.zeros((1, 256), np.float32))
