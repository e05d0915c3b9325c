"""Batches of 9..16 tokens share one pass over the weights (two 8-token tiles per launch).

The arithmetic of a token must not depend on how many tokens travel with it: a 13- or 16-token
call has to return, bit for bit, what the same rows give in calls of at most 8 tokens, and the
whole batch has to match the CPU oracle within the band of the packed linear tests
(tests/test_0106b_quantized_linear.py:119-121 of the reference: rtol 2e-5 / atol 2e-3 vs FP64).
"""

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import packed_to_device, quantized_linear, quantized_swiglu
from mylocal_llm_b200.quantize import quantize
from mylocal_llm_b200.quantized_linear import retile_weight

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def gemv_passes_only(monkeypatch):
    """This file is about the GEMV kernels' token tiles; more than 8 BF16 tokens on a GGUF-layout weight would otherwise go to the GEMM."""
    monkeypatch.setenv("B200Q_GEMM", "0")


def weights(fmt, n, k, seed, tile):
    rng = np.random.default_rng(seed)
    w = quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    dev = packed_to_device(w)
    return w, (retile_weight(dev) if tile else dev)


@pytest.mark.parametrize("fmt,tile", [("Q8_0", True), ("Q6_K", True), ("Q4_K", True), ("Q4_K", False), ("Q5_K", False)])
@pytest.mark.parametrize("n,k", [(512, 2048), (4096, 1024), (48, 256), (2048, 4096)])
@pytest.mark.parametrize("m", [9, 13, 16, 21, 35])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_batches_equal_their_eight_token_slices(cuda, fmt, tile, n, k, m, dtype):
    if n * k >= 2048 * 4096 and m not in (13, 16):
        pytest.skip("large shape: two batch sizes are enough")
    w, dev = weights(fmt, n, k, seed=n + k + m, tile=tile)
    if tile:
        assert dev.quant_type == fmt + "_TILED"
    rng = np.random.default_rng(7 * m + k)
    x_host = (rng.normal(0, 1, (m, k)) * rng.uniform(0.01, 30.0, (m, 1))).astype(np.float32)   # per-token scales differ
    x = cuda.from_numpy(x_host).cuda().to(getattr(cuda, dtype))
    whole = quantized_linear(x, dev, out_dtype=cuda.float32)
    for t0 in range(0, m, 8):
        part = quantized_linear(x[t0:t0 + 8].contiguous(), dev, out_dtype=cuda.float32)
        assert cuda.equal(whole[t0:t0 + 8], part), f"rows {t0}..{t0 + 8} differ from the 8-token call"
    # the reference's band for unit-scale activations (rtol 2e-5 / atol 2e-3 vs FP64), applied after undoing
    # the per-token scale of the inputs; 16-bit activations: the band of the packed linear tests for them
    scale = np.abs(x.float().cpu().numpy()).std(axis=1, keepdims=True).astype(np.float64)
    ref = po.linear_fp64(x.float().cpu().numpy(), w.data, w.shape, fmt) / scale
    np.testing.assert_allclose(whole.double().cpu().numpy() / scale, ref, rtol=2e-5, atol=2e-3)


@pytest.mark.parametrize("fmt,tile", [("Q4_K", True), ("Q4_K", False), ("Q5_K", False)])
@pytest.mark.parametrize("f,k", [(512, 2048), (80, 512), (1408, 4096)])
@pytest.mark.parametrize("m", [9, 16, 27])
@pytest.mark.parametrize("dtype", ["float32", "float16"])
def test_wide_swiglu_batches_equal_their_eight_token_slices(cuda, fmt, tile, f, k, m, dtype):
    gate_w, gate = weights(fmt, f, k, seed=f + k + m, tile=tile)
    up_w, up = weights(fmt, f, k, seed=f + k + m + 1, tile=tile)
    rng = np.random.default_rng(3 * m + f)
    x = cuda.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(getattr(cuda, dtype))
    whole = quantized_swiglu(x, gate, up, out_dtype=cuda.float32)
    for t0 in range(0, m, 8):
        part = quantized_swiglu(x[t0:t0 + 8].contiguous(), gate, up, out_dtype=cuda.float32)
        assert cuda.equal(whole[t0:t0 + 8], part)
    ref = po.swiglu_fp64(x.float().cpu().numpy(), (gate_w.data, gate_w.shape, fmt), (up_w.data, up_w.shape, fmt))
    np.testing.assert_allclose(whole.cpu().numpy(), ref, rtol=3e-4, atol=2e-4)


def test_unused_token_tile_columns_do_not_leak(cuda):
    """Columns of a token tile are independent: NaN rows travelling in the same pass (and through the
    same per-tile scaling step) must not change the finite rows beside them."""
    w, dev = weights("Q8_0", 256, 1024, seed=5, tile=True)
    rng = np.random.default_rng(11)
    x16 = cuda.from_numpy(rng.normal(0, 1, (16, 1024)).astype(np.float32)).cuda()
    x16[9:] = float("nan")
    poisoned = quantized_linear(x16, dev)
    clean = quantized_linear(x16[:9].contiguous(), dev)
    assert cuda.equal(poisoned[:9], clean)
    assert bool(cuda.isnan(poisoned[9:]).all())
