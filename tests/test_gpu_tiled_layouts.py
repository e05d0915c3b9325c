"""Device tile layouts of Q6_K, Q4_K, Q5_K and Q8_0: lossless re-ordering, and the kernels that read them, against
the oracle and against the kernels that read the GGUF bytes."""

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import PackedExpertBank, packed_to_device, quantized_linear
from mylocal_llm_b200 import moe_ops
from mylocal_llm_b200.experts_inference import routed_experts_forward, synthetic_bank
from mylocal_llm_b200.quantize import quantize, random_packed
from mylocal_llm_b200 import quantized_swiglu
from mylocal_llm_b200.quantized_linear import (DevicePackedGGUFWeight, dequantize_device, retile_bytes, retile_q6k,
                                               retile_weight, untile_bytes, untile_q6k)

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
    q3 = packed_to_device(random_packed("Q3_K", (32, 256), seed=1))
    assert retile_weight(q3) is q3                   # no tile layout for this type
    wide = packed_to_device(random_packed("Q4_K", (16, 8192), seed=1))
    assert retile_weight(wide) is wide               # K above the limit stays native unless forced


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
    assert tiled.down_type == "Q6_K_TILED" and tiled.gate_type == "Q4_K_TILED"
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


# ----------------------------------------------------------------------------------- Q4_K, Q5_K
BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176}
K_FORMATS = pytest.mark.parametrize("fmt", ["Q4_K", "Q5_K"])


@K_FORMATS
@pytest.mark.parametrize("rows,k", [(16, 256), (48, 512), (512, 2048), (32, 8192)])
def test_q4k_retile_then_untile_restores_the_gguf_bytes(cuda, fmt, rows, k):
    raw = np.random.default_rng(rows + k).integers(0, 256, rows * k // 256 * BLOCK_BYTES[fmt], dtype=np.uint8)
    native = cuda.from_numpy(raw).cuda()
    tiled = retile_bytes(native, rows, k, fmt)
    assert tiled.shape == native.shape and not cuda.equal(tiled, native)
    assert cuda.equal(untile_bytes(tiled, rows, k, fmt + "_TILED"), native)
    # every byte only moved: same multiset
    assert cuda.equal(tiled.sort().values, native.sort().values)


@K_FORMATS
def test_q4k_tiled_weight_dequantizes_to_the_same_values(cuda, fmt):
    w = random_packed(fmt, (64, 512), seed=3, d=0.01, dmin=0.005)
    tiled = retile_weight(packed_to_device(w))
    assert tiled.quant_type == fmt + "_TILED"
    got = dequantize_device(tiled.data, 64, 512, fmt + "_TILED").cpu().numpy()
    np.testing.assert_array_equal(got, po.dequantize(w.data, w.shape, fmt))


@pytest.mark.parametrize("n,k", [(8192, 2048), (512, 2048), (2048, 512), (16, 256), (2048, 8192)])
@pytest.mark.parametrize("m", [1, 5, 8, 13])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@K_FORMATS
def test_q4k_tiled_gemv_equals_the_native_direct_kernel_and_the_oracle(cuda, monkeypatch, fmt, n, k, m, dtype):
    if n * k >= 8192 * 2048 and m not in (1, 8):
        pytest.skip("large shapes: two batch sizes are enough")
    monkeypatch.setenv("B200Q_GEMM", "0")        # the two GEMV kernels are compared: 13 BF16 tokens on the GGUF layout would go to the GEMM
    rng = np.random.default_rng(n + k + m)
    w = quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    dev = packed_to_device(w)
    force = k > 4096 and dtype != "float32"
    tiled = retile_weight(dev, force=force)
    if k > 4096 and not force:
        assert tiled is dev
        return
    assert tiled.quant_type == fmt + "_TILED"
    x = cuda.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(getattr(cuda, dtype))
    got = quantized_linear(x, tiled)
    assert cuda.equal(got, quantized_linear(x, dev))             # same arithmetic, other addresses
    ref = po.linear_fp64(x.float().cpu().numpy(), w.data, w.shape, fmt)
    if dtype == "float32":
        np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=2e-4, atol=2e-5 * np.sqrt(k / 256))
    else:
        np.testing.assert_allclose(got.float().cpu().numpy(), ref, rtol=1.6e-2, atol=2e-2)


def test_q4k_tiled_k8192_with_fp32_activations_is_refused(cuda):
    w = retile_weight(packed_to_device(random_packed("Q4_K", (32, 8192), seed=2, d=0.01, dmin=0.005)), force=True)
    x = cuda.zeros((1, 8192), dtype=cuda.float32, device="cuda")
    with pytest.raises(NotImplementedError):
        quantized_linear(x, w)


@K_FORMATS
@pytest.mark.parametrize("m", [1, 8, 9])
def test_q4k_tiled_swiglu_equals_the_native_kernel(cuda, fmt, m):
    f, k = 512, 2048
    rng = np.random.default_rng(m)
    gate = packed_to_device(quantize(rng.normal(0, 0.02, (f, k)).astype(np.float32), fmt))
    up = packed_to_device(quantize(rng.normal(0, 0.02, (f, k)).astype(np.float32), fmt))
    x = cuda.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(cuda.bfloat16)
    want = quantized_swiglu(x, gate, up, out_dtype=cuda.float32)
    got = quantized_swiglu(x, retile_weight(gate), retile_weight(up), out_dtype=cuda.float32)
    assert cuda.equal(got, want)
    with pytest.raises(ValueError):
        quantized_swiglu(x, retile_weight(gate), up)             # mixed layouts


@K_FORMATS
@pytest.mark.parametrize("tokens", [1, 7, 33])
def test_fully_tiled_bank_matches_the_native_bank(cuda, fmt, tokens):
    e, d, f, k = 10, 512, 256, 3
    bank = synthetic_bank(e, d, f, (fmt, fmt, "Q6_K"), seed=4)
    tiled = bank.retiled()
    assert (tiled.gate_type, tiled.up_type, tiled.down_type) == (fmt + "_TILED", fmt + "_TILED", "Q6_K_TILED")
    rng = np.random.default_rng(tokens)
    x = cuda.from_numpy(rng.normal(0, 1, (tokens, d)).astype(np.float32)).cuda().to(cuda.bfloat16)
    ids = cuda.from_numpy(np.stack([rng.choice(e, k, replace=False) for _ in range(tokens)])).cuda()
    weights = cuda.from_numpy(rng.random((tokens, k)).astype(np.float32)).cuda()
    a = routed_experts_forward(x, weights, ids, bank, out_dtype=cuda.float32).cpu().numpy()
    b = routed_experts_forward(x, weights, ids, tiled, out_dtype=cuda.float32).cpu().numpy()
    np.testing.assert_allclose(b, a, rtol=2e-4, atol=1e-5)
    one = tiled.expert(3).forward(x)                              # per-expert handles see whole tiles
    # (from 9 BF16 tokens on the GGUF-layout handle runs its projections on the tensor-core GEMM, whose weights carry
    # one BF16 rounding, and the BF16 outputs of magnitude ~100 have an ulp of 0.5: the band is relative to the
    # output scale, not to each element)
    want = bank.expert(3).forward(x).float().cpu().numpy()
    np.testing.assert_allclose(one.float().cpu().numpy(), want, rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(want).max())))


# ------------------------------------------------------------------------------------------ Q8_0
@pytest.mark.parametrize("rows,k", [(16, 256), (48, 512), (4096, 4096)])
def test_q8_0_retile_then_untile_restores_the_gguf_bytes(cuda, rows, k):
    raw = np.random.default_rng(rows + k).integers(0, 256, rows * k // 32 * 34, dtype=np.uint8)
    native = cuda.from_numpy(raw).cuda()
    tiled = retile_bytes(native, rows, k, "Q8_0")
    assert tiled.shape == native.shape and not cuda.equal(tiled, native)
    assert cuda.equal(untile_bytes(tiled, rows, k, "Q8_0_TILED"), native)


@pytest.mark.parametrize("n,k", [(4096, 4096), (2048, 8192), (8192, 2048), (16, 256), (48, 288)])
@pytest.mark.parametrize("m", [1, 8, 11])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_q8_0_tiled_gemv_matches_the_oracle(cuda, n, k, m, dtype):
    if n * k >= 4096 * 4096 and m == 11:
        pytest.skip("large shapes: two batch sizes are enough")
    rng = np.random.default_rng(n + k + m)
    w = quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), "Q8_0")
    dev = packed_to_device(w)
    force = k > 4096 and dtype != "float32"
    tiled = retile_weight(dev, force=force)
    if k % 256 or (k > 4096 and not force):
        assert tiled is dev                          # K not a multiple of 256, or too wide for FP32 inputs
        return
    assert tiled.quant_type == "Q8_0_TILED"
    x = cuda.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(getattr(cuda, dtype))
    got = quantized_linear(x, tiled).float().cpu().numpy()
    ref = po.linear_fp64(x.float().cpu().numpy(), w.data, w.shape, "Q8_0")
    if dtype == "float32":
        np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-3)
    else:
        np.testing.assert_allclose(got, ref, rtol=1.6e-2, atol=2e-2)
    dq = dequantize_device(tiled.data, n, k, "Q8_0_TILED").cpu().numpy()
    np.testing.assert_array_equal(dq, po.dequantize(w.data, w.shape, "Q8_0"))


def test_q8_0_tiled_identity_columns_are_exact(cuda):
    n, k = 32, 256
    w = random_packed("Q8_0", (n, k), seed=9, d=0.01)
    tiled = retile_weight(packed_to_device(w))
    deq = po.dequantize(w.data, w.shape, "Q8_0")
    for start in (0, 31, 248):
        x = np.zeros((8, k), np.float32)
        for t in range(8):
            x[t, start + t] = 1.0
        got = quantized_linear(cuda.from_numpy(x).cuda(), tiled).cpu().numpy()
        np.testing.assert_array_equal(got, deq[:, start:start + 8].T)
