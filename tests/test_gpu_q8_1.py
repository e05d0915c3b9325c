"""Integer-dot mode on the GPU: the Q8_1 quantiser bit for bit against the oracle's IEEE restatement, and the
Q4_K x Q8_1 GEMV against the oracle's integer formula (exact integers, FP64 combination): what separates the
two is FP32 accumulation only, so the band is the packed linear's (rtol 2e-5, absolute part scaled by the
output RMS; tests/test_0106b_quantized_linear.py:119-121 of the reference). The distance of the mode from
the FP32-activation result (int8 rounding of the activations) is stated and bounded separately."""

import numpy as np
import pytest

from oracle import packed_oracle as po
from oracle import q8_oracle as qo
from mylocal_llm_b200 import packed_to_device
from mylocal_llm_b200.q8_1 import q8_1_linear, quantize_q8_1, quantized_linear_q8_1
from mylocal_llm_b200.quantize import quantize, random_packed
from mylocal_llm_b200.quantized_linear import retile_weight

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,k", [(1, 256), (3, 2048), (8, 4096)])
def test_quantiser_matches_the_oracle_bit_for_bit(cuda, rows, k):
    rng = np.random.default_rng(rows + k)
    x = (rng.normal(0, 1, (rows, k)) * rng.uniform(0.01, 50, (rows, 1))).astype(np.float32)
    x[0, 32:64] = 0
    x[-1, 0] = 3e6                                              # block scale beyond the FP16 range
    got = quantize_q8_1(cuda.from_numpy(x).cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, qo.quantize_q8_1(x))
    # BF16 input: the codes of the BF16-rounded values
    xb = cuda.from_numpy(x).cuda().to(cuda.bfloat16)
    np.testing.assert_array_equal(quantize_q8_1(xb).cpu().numpy(), qo.quantize_q8_1(xb.float().cpu().numpy()))


@pytest.mark.parametrize("fmt", ["Q4_K", "Q5_K"])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("n,k,m", [(16, 256, 1), (48, 512, 2), (80, 2048, 3), (512, 2048, 4), (96, 4096, 5), (32, 8192, 8),
                                   (2048, 1024, 1)])
def test_gemv_matches_the_integer_formula(cuda, fmt, tiled, n, k, m):
    w = random_packed(fmt, (n, k), seed=n + k + m, d=0.01, dmin=0.005)
    dev = packed_to_device(w)
    if tiled:
        dev = retile_weight(dev, force=True)
        assert dev.quant_type == fmt + "_TILED"
    x = np.random.default_rng(m).normal(0, 1, (m, k)).astype(np.float32)
    blocks = quantize_q8_1(cuda.from_numpy(x).cuda())
    y = q8_1_linear(blocks, dev).cpu().numpy()
    ref = qo.q4k_q8_1_linear(blocks.cpu().numpy(), w.data, w.shape, fmt)
    rms = float(np.sqrt((ref ** 2).mean()))
    np.testing.assert_allclose(y, ref, rtol=2e-5, atol=2e-5 * rms)


def test_unaligned_row_count_in_the_gguf_layout_and_output_types(cuda):
    w = quantize(np.random.default_rng(2).normal(0, 0.02, (37, 1024)).astype(np.float32), "Q4_K")
    dev = packed_to_device(w)
    x = cuda.randn((2, 3, 1024), device="cuda")
    y = quantized_linear_q8_1(x, dev)
    assert y.shape == (2, 3, 37) and y.dtype == cuda.float32
    ref = po.linear_fp64(x.reshape(6, 1024).cpu().numpy(), w.data, w.shape, "Q4_K")
    # the mode's own distance from FP32 activations: int8 rounding, about 0.4 % of a block's largest value per element
    assert np.abs(y.reshape(6, 37).cpu().numpy() - ref).max() <= 0.02 * np.abs(ref).max()
    yb = quantized_linear_q8_1(x.to(cuda.bfloat16), dev)
    assert yb.dtype == cuda.bfloat16
    with pytest.raises(NotImplementedError):
        q8_1_linear(quantize_q8_1(x), packed_to_device(quantize(np.zeros((16, 1024), np.float32), "Q6_K")))
    with pytest.raises(ValueError):
        q8_1_linear(quantize_q8_1(x[..., :512].contiguous()), dev)
