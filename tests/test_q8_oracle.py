"""CPU checks of the Q8_1 oracle (oracle/q8_oracle.py): the codec against its definition
(mini_llm/ops/q8_1_gpu.py:30-58 of the reference) and the integer-dot linear against the FP64 product of the
pinned dequantised weights with the dequantised activations (the two are the same sum regrouped)."""

import numpy as np
import pytest

from oracle import packed_oracle as po
from oracle import q8_oracle as qo
from mylocal_llm_b200.quantize import random_packed


def test_codec_follows_its_definition():
    rng = np.random.default_rng(0)
    x = rng.normal(0, 3, (5, 256)).astype(np.float32)
    x[1, 32:64] = 0                                             # an all-zero block
    x[2, 0:32] = np.linspace(-127, 127, 32)                     # exact codes
    x[3, 0] = 1e9                                               # scale beyond the FP16 range is bounded
    blocks = qo.quantize_q8_1(x)
    assert blocks.shape == (5, 8, 36) and blocks.dtype == np.uint8
    codes = blocks[..., 4:].view(np.int8)
    d = blocks[..., 0:2].copy().view("<f2").astype(np.float32)[..., 0]
    assert codes.min() >= -127 and codes.max() <= 127
    assert not codes[1, 1].any() and d[1, 1] == 0
    np.testing.assert_array_equal(codes[2, 0].astype(np.float32), np.round(np.linspace(-127, 127, 32)).astype(np.float32))
    amax = np.abs(x.reshape(5, 8, 32)).max(axis=2)
    ok = amax / 127 <= 65504
    np.testing.assert_array_equal(d[ok], (amax / np.float32(127))[ok].astype("<f2").astype(np.float32))
    assert d[3, 0] == np.float32(65504)
    # every block's largest magnitude maps to +-127, and dequantisation is within half a step elsewhere
    deq = qo.dequantize_q8_1(blocks).reshape(5, 8, 32)
    err = np.abs(deq - x.reshape(5, 8, 32))
    assert (err[ok] <= 0.5 * d[ok][:, None] * 1.001 + 1e-3 * amax[ok][:, None]).all()
    # ties round away from zero: 0.5 steps of a block whose scale is exactly 1
    t = np.zeros((1, 32), np.float32)
    t[0, :5] = [127, 0.5, -0.5, 1.5, -2.5]
    np.testing.assert_array_equal(qo.quantize_q8_1(t)[0, 0, 4:9].view(np.int8), [127, 1, -1, 2, -3])
    # the stored sum is the butterfly sum of the inputs
    s = blocks[..., 2:4].copy().view("<f2").astype(np.float32)[..., 0]
    np.testing.assert_allclose(s[0], x[0].reshape(8, 32).sum(axis=1), rtol=2e-3, atol=2e-2)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q5_K"])
def test_integer_dot_formula_equals_the_dequantised_product(fmt):
    w = random_packed(fmt, (11, 512), seed=4, d=0.01, dmin=0.005)
    x = np.random.default_rng(1).normal(0, 1, (3, 512)).astype(np.float32)
    blocks = qo.quantize_q8_1(x)
    got = qo.q4k_q8_1_linear(blocks, w.data, w.shape, fmt)
    ref = qo.dequantize_q8_1(blocks) @ po.dequantize(w.data, w.shape, fmt).astype(np.float64).T
    np.testing.assert_allclose(got, ref, rtol=1e-9, atol=1e-9)
    # and the mode's distance from FP32 activations: int8 rounding of x, well inside 2 % of the output scale
    exact = po.linear_fp64(x, w.data, w.shape, fmt)
    assert np.abs(got - exact).max() <= 0.02 * np.abs(exact).max()
