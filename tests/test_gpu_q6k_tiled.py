"""Q6_K tile layout: lossless re-ordering, and the tensor-core GEMV that reads it, against the oracle."""

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import PackedExpertBank, packed_to_device, quantized_linear
from mylocal_llm_b200 import moe_ops
from mylocal_llm_b200.experts_inference import routed_experts_forward, synthetic_bank
from mylocal_llm_b200.quantize import quantize, random_packed
from mylocal_llm_b200.quantized_linear import (DevicePackedGGUFWeight, dequantize_device, retile_q6k, retile_weight,
                                               untile_q6k)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,k", [(16, 256), (48, 512), (2048, 512), (32, 2048)])
def test_retile_then_untile_restores_the_gguf_bytes(cuda, rows, k):
    raw = np.random.default_rng(rows + k).integers(0, 256, rows * k // 256 * 210, dtype=np.uint8)
    native = cuda.from_numpy(raw).cuda()
    tiled = retile_q6k(native, rows, k)
    assert tiled.shape == native.shape and not cuda.equal(tiled, native)
    assert cuda.equal(untile_q6k(tiled, rows, k), native)


def test_tiled_weight_dequantizes_to_the_same_values(cuda):
    w = random_packed("Q6_K", (64, 512), seed=3, d=0.01)
    dev = packed_to_device(w)
    tiled = retile_weight(dev)
    assert tiled.quant_type == "Q6_K_TILED" and tiled.nbytes == dev.nbytes
    want = po.dequantize(w.data, w.shape, "Q6_K")
    got = dequantize_device(tiled.data, 64, 512, "Q6_K_TILED").cpu().numpy()
    np.testing.assert_array_equal(got, want)


def test_retile_rejects_bad_shapes(cuda):
    buf = cuda.zeros(24 * 210, dtype=cuda.uint8, device="cuda")
    with pytest.raises(ValueError):
        retile_q6k(buf, 24, 256)                     # rows not a multiple of 16
    small = packed_to_device(random_packed("Q6_K", (24, 256), seed=1))
    assert retile_weight(small) is small             # kept native
    q4 = packed_to_device(random_packed("Q4_K", (32, 256), seed=1))
    assert retile_weight(q4) is q4


@pytest.mark.parametrize("n,k", [(2048, 512), (512, 2048), (8192, 2048), (2048, 4096), (2048, 8192), (16, 256)])
@pytest.mark.parametrize("m", [1, 3, 8, 11])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiled_gemv_matches_the_oracle(cuda, n, k, m, dtype):
    if n * k > 2048 * 8192 // 2 and m not in (1, 8):
        pytest.skip("large shapes: two batch sizes are enough")
    rng = np.random.default_rng(n + k + m)
    w = quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), "Q6_K")
    dev = packed_to_device(w)
    tiled = retile_weight(dev)
    if k > 4096:                                     # activation fragments would not fit: stays native
        assert tiled is dev
        return
    assert tiled.quant_type == "Q6_K_TILED"
    x = cuda.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(getattr(cuda, dtype))
    got = quantized_linear(x, tiled).float().cpu().numpy()
    ref = po.linear_fp64(x.float().cpu().numpy(), w.data, w.shape, "Q6_K")
    if dtype == "float32":
        np.testing.assert_allclose(got, ref, rtol=2e-4, atol=2e-5 * np.sqrt(k / 256))
    else:
        np.testing.assert_allclose(got, ref, rtol=1.6e-2, atol=2e-2)       # bf16 output rounding
    # and it agrees with the kernels that read the native bytes
    native = quantized_linear(x, packed_to_device(w)).float().cpu().numpy()
    np.testing.assert_allclose(got, native, rtol=1.6e-2 if dtype == "bfloat16" else 2e-4, atol=2e-2 if dtype == "bfloat16" else 2e-5 * np.sqrt(k / 256))


def test_tiled_identity_columns_are_exact(cuda):
    """One-hot activations pick single weights: the product must be the dequantized value itself."""
    n, k = 32, 256
    w = random_packed("Q6_K", (n, k), seed=9, d=0.01)
    tiled = retile_weight(packed_to_device(w))
    deq = po.dequantize(w.data, w.shape, "Q6_K")
    for start in (0, 100, 248):
        x = np.zeros((8, k), np.float32)
        for t in range(8):
            x[t, start + t] = 1.0
        got = quantized_linear(cuda.from_numpy(x).cuda(), tiled).cpu().numpy()
        np.testing.assert_array_equal(got, deq[:, start:start + 8].T)


@pytest.mark.parametrize("tokens", [1, 5, 40])
def test_grouped_down_on_a_tiled_bank_equals_the_native_bank_closely(cuda, tokens):
    e, d, f, k = 12, 512, 256, 3
    bank = synthetic_bank(e, d, f, ("Q4_K", "Q4_K", "Q6_K"), seed=2)
    tiled = bank.retiled()
    assert tiled.down_type == "Q6_K_TILED" and tiled.gate is bank.gate
    rng = np.random.default_rng(tokens)
    x = cuda.from_numpy(rng.normal(0, 1, (tokens, d)).astype(np.float32)).cuda()
    ids = cuda.from_numpy(np.stack([rng.choice(e, k, replace=False) for _ in range(tokens)])).cuda()
    weights = cuda.from_numpy(rng.random((tokens, k)).astype(np.float32)).cuda()
    a = routed_experts_forward(x, weights, ids, bank).cpu().numpy()
    b = routed_experts_forward(x, weights, ids, tiled).cpu().numpy()
    np.testing.assert_allclose(b, a, rtol=2e-4, atol=1e-5)
    tables, aligned = tiled.pointer_tables()
    c = routed_experts_forward(x, weights, ids, tiled, tables=tables, tables_aligned16=aligned).cpu().numpy()
    np.testing.assert_array_equal(c, b)
