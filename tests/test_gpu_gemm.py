"""The tensor-core GEMM for many tokens (``b200q_gemm``: tcgen05.mma, accumulator in tensor memory,
activations by TMA) against the FP64 oracle.

Two bars per case. (1) Against the oracle product taken with the weights rounded to BF16 exactly as
the kernel rounds them: what is left is FP32 accumulation, so the band is the packed linear's
(rtol 2e-5 of tests/test_0106b_quantized_linear.py:119-121, absolute part scaled by the output RMS, plus 2^-24 of
the RMS per K = 16 step of the tensor core's accumulator, whose additions do not round to nearest) -
this bar finds every layout, swizzle, descriptor or tile-edge mistake. (2) Against the oracle product
with the exact dequantised weights, element by element: rounding a weight to BF16 moves it by at most
2^-9 relative (uniform, variance (2^-9)^2 / 3), so output (t, r) may differ by twelve standard deviations
of the independent-error model, 12 * 2^-9 / sqrt(3) * sqrt(sum_i (w_ri x_ti)^2) - twelve rather than the
usual six or seven because equal codes of one sub-block round by the same amount, so the errors of a row
are positively correlated - plus the FP32 slack of bar (1); BF16 outputs add their own rounding (2^-8
relative).
"""

import ctypes

import numpy as np
import pytest

from oracle import build_oracle as bo
from mylocal_llm_b200 import _lib, packed_to_device, quantized_linear
from mylocal_llm_b200.quantize import quantize, random_packed

pytestmark = pytest.mark.gpu

FORMATS = ("Q8_0", "Q4_K", "Q5_K", "Q6_K")


def bf16_round(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def run_gemm(torch, w, x_bf16, out_dtype, split=False):
    n, k = w.shape
    m = x_bf16.shape[0]
    dev = packed_to_device(w)
    y = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    fmt, bf16 = _lib.FORMAT_ID[w.quant_type], _lib.DTYPE_ID["bfloat16"]
    if split:
        nbytes = int(_lib.load().b200q_gemm_workspace_bytes(fmt, n, k, bf16, m))
        assert nbytes > 0 and nbytes % (m * n * 4) == 0, "this shape was expected to split K"
        scratch = torch.full((nbytes // 4,), float("nan"), dtype=torch.float32, device="cuda")
        _lib.call("b200q_gemm_ws", ptr(dev.data), fmt, n, k, ptr(x_bf16), bf16, m, ptr(y),
                  _lib.DTYPE_ID[str(out_dtype).replace("torch.", "")], ptr(scratch), nbytes, _lib.current_stream())
    else:
        _lib.call("b200q_gemm", ptr(dev.data), fmt, n, k, ptr(x_bf16), bf16, m,
                  ptr(y), _lib.DTYPE_ID[str(out_dtype).replace("torch.", "")], _lib.current_stream())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return y


def check(torch, w, m, seed, out_dtype=None, split=False):
    out_dtype = out_dtype or torch.float32
    n, k = w.shape
    x = np.random.default_rng(seed).normal(0, 1, (m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda().to(torch.bfloat16)
    y = run_gemm(torch, w, xd, out_dtype, split).double().cpu().numpy()
    assert np.isfinite(y).all(), "some outputs were never written"
    dense = bo.port_dequantize(w.data, w.shape, w.quant_type)
    x64 = xd.double().cpu().numpy()
    ref_rounded = x64 @ bf16_round(torch, dense).T
    ref_exact = x64 @ dense.astype(np.float64).T
    rms = float(np.sqrt((ref_exact ** 2).mean())) or 1.0
    # FP32 slack: the packed linear's 2e-5, plus one unit of 2^-24 per K = 16 step of the tensor core's accumulator -
    # its additions are not round-to-nearest (the measured error is biased toward zero and grows with the number of
    # steps: 2.2e-3 on outputs of RMS 67 at K = 8192 in one CTA, four times less with K split over four CTAs)
    fp32_slack = (2e-5 + (k / 16) * 2.0 ** -24) * rms
    if out_dtype == torch.float32:
        np.testing.assert_allclose(y, ref_rounded, rtol=2e-5, atol=fp32_slack)
    sigma = 2.0 ** -9 / np.sqrt(3.0) * np.sqrt((x64 ** 2) @ (dense.astype(np.float64) ** 2).T)
    slack = 12.0 * sigma + fp32_slack + (2.0 ** -8 if out_dtype != torch.float32 else 2e-5) * np.abs(ref_exact)
    worst = float((np.abs(y - ref_exact) / slack).max())
    assert worst <= 1.0, f"BF16-weight bar exceeded: ratio {worst:.2f}"


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n,k,m", [(64, 256, 17), (128, 256, 128), (64, 512, 33), (192, 1024, 129), (80, 256, 40),
                                   (1024, 2048, 300), (192, 512, 600), (136, 256, 257), (100, 256, 40)])
def test_gemm_small_shapes_all_formats(cuda, fmt, n, k, m):
    # (100 rows: output rows that are not 16-byte aligned leave the staged epilogue for the direct stores)
    w = quantize(np.random.default_rng(n + k).normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    check(cuda, w, m, seed=m)
    if n == 100:
        check(cuda, w, m, seed=m, out_dtype=cuda.bfloat16)


@pytest.mark.parametrize("fmt", FORMATS)
def test_gemm_random_bytes_exercise_every_code_bit(cuda, fmt):
    w = random_packed(fmt, (256, 1024), seed=5, d=0.01, dmin=0.005)
    check(cuda, w, 70, seed=1)
    check(cuda, w, 70, seed=1, out_dtype=cuda.bfloat16)
    check(cuda, w, 70, seed=1, out_dtype=cuda.float16)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("shape", [(8192, 2048), (2048, 8192)])
@pytest.mark.parametrize("m", [32, 512])
def test_gemm_second_configuration(cuda, fmt, shape, m):
    w = random_packed(fmt, shape, seed=shape[0], d=0.01, dmin=0.005)
    check(cuda, w, m, seed=m)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0"])
def test_gemm_benchmarked_shape_at_2048_tokens(cuda, fmt):
    # the shape of the gemm_*_m2048 workloads: CTA pairs by default, two token tiles per pair
    w = random_packed(fmt, (8192, 2048), seed=7, d=0.01, dmin=0.005)
    check(cuda, w, 2048, seed=5, out_dtype=cuda.bfloat16)


def test_quantized_linear_routes_many_bf16_tokens_to_the_gemm(cuda, monkeypatch):
    torch = cuda
    w = quantize(np.random.default_rng(3).normal(0, 0.02, (512, 1024)).astype(np.float32), "Q4_K")
    dev = packed_to_device(w)
    calls = []
    real = _lib.call
    monkeypatch.setattr(_lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    x = torch.randn((2, 40, 1024), device="cuda").to(torch.bfloat16)
    y = quantized_linear(x, dev)
    assert calls == ["b200q_gemm"] and y.shape == (2, 40, 512) and y.dtype == torch.bfloat16
    calls.clear()
    quantized_linear(x[:, :4].contiguous(), dev)                       # 8 tokens (one tile): the GEMV kernel
    quantized_linear(x.float(), dev)                                   # FP32 activations keep the exact-product path
    monkeypatch.setenv("B200Q_GEMM", "0")
    y_gemv = quantized_linear(x, dev)
    assert calls == ["b200q_gemv"] * 3
    ref = y_gemv.float()
    assert float((y.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_gemm_rejects_what_it_does_not_cover(cuda):
    torch = cuda
    w = quantize(np.random.default_rng(3).normal(0, 0.02, (64, 256)).astype(np.float32), "Q4_K")
    dev = packed_to_device(w)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    x32 = torch.randn((32, 256), device="cuda")
    y = torch.empty((32, 64), device="cuda")
    with pytest.raises(NotImplementedError):
        _lib.call("b200q_gemm", ptr(dev.data), 2, 64, 256, ptr(x32), 0, 32, ptr(y), 0, _lib.current_stream())
    with pytest.raises(ValueError):
        _lib.call("b200q_gemm", ptr(dev.data), 22, 64, 256, ptr(x32), 2, 32, ptr(y), 0, _lib.current_stream())
    assert _lib.load().b200q_gemm_supported(2, 64, 256, 2, 32) == 1
    assert _lib.load().b200q_gemm_supported(2, 64, 256, 0, 32) == 0
    assert _lib.load().b200q_gemm_supported(0, 64, 96, 2, 32) == 0


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n,k,m,out", [(256, 8192, 64, "float32"), (128, 4096, 300, "bfloat16"), (2048, 8192, 512, "bfloat16"),
                                       (200, 4352, 33, "float32")])
def test_gemm_split_k_sums_partial_tiles_in_order(cuda, fmt, n, k, m, out):
    # few weight-row tiles: K is split over 2-8 CTAs, FP32 partial tiles added in ascending order by a second kernel;
    # same bars as the one-CTA-per-tile product, rows and tokens off the tile grid included
    if fmt != "Q4_K" and n * k >= 2048 * 8192:
        pytest.skip("the large shape once")
    w = random_packed(fmt, (n, k), seed=n + m, d=0.01, dmin=0.005) if n * k >= 2048 * 8192 else quantize(
        np.random.default_rng(n + k).normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    check(cuda, w, m, seed=m, out_dtype=getattr(cuda, out), split=True)


def test_gemm_split_k_is_used_by_the_linear_and_can_be_turned_off(cuda, monkeypatch):
    torch = cuda
    w = packed_to_device(quantize(np.random.default_rng(1).normal(0, 0.02, (256, 8192)).astype(np.float32), "Q4_K"))
    x = torch.randn((64, 8192), device="cuda").to(torch.bfloat16)
    calls = []
    real = _lib.call
    monkeypatch.setattr(_lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    split = quantized_linear(x, w, out_dtype=torch.float32)
    monkeypatch.setenv("B200Q_GEMM_SPLITK", "0")
    whole = quantized_linear(x, w, out_dtype=torch.float32)
    assert calls == ["b200q_gemm_ws", "b200q_gemm"]
    # the same products added in another order
    torch.testing.assert_close(split, whole, rtol=2e-5, atol=2e-5 * float(whole.abs().max()))
    assert _lib.load().b200q_gemm_workspace_bytes(2, 8192, 2048, 2, 512) == 0          # enough tiles: no split


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n,k,m", [(64, 256, 17), (320, 512, 33), (192, 1024, 129), (1024, 2048, 300), (136, 256, 600),
                                   (256, 512, 1100)])
def test_gemm_cta_pairs(cuda, monkeypatch, fmt, n, k, m):
    # two CTAs of a cluster as one tensor-core unit (each decodes 128 rows and stages half of the tokens), forced at
    # every size: an odd number of weight-row tiles, token tiles cut by m, a single 8-token half, two accumulators
    monkeypatch.setenv("B200Q_GEMM_PAIR", "2")
    w = quantize(np.random.default_rng(n + k).normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    check(cuda, w, m, seed=m)
    check(cuda, w, m, seed=m + 1, out_dtype=cuda.bfloat16)


@pytest.mark.parametrize("n,k,m", [(256, 8192, 64), (200, 4352, 33)])
def test_gemm_cta_pairs_with_split_k(cuda, monkeypatch, n, k, m):
    monkeypatch.setenv("B200Q_GEMM_PAIR", "2")
    w = quantize(np.random.default_rng(n + k).normal(0, 0.02, (n, k)).astype(np.float32), "Q6_K")
    check(cuda, w, m, seed=m, split=True)


def test_gemm_pairs_ctas_from_a_thousand_tokens_on(cuda, monkeypatch):
    # the default: one-CTA tiles below four token tiles, pairs from there on; both kernels give the same product
    torch = cuda
    w = random_packed("Q4_K", (2048, 2048), seed=11, d=0.01, dmin=0.005)
    check(torch, w, 1100, seed=3)
    x = torch.randn((1100, 2048), device="cuda").to(torch.bfloat16)
    paired = run_gemm(torch, w, x, torch.float32)
    monkeypatch.setenv("B200Q_GEMM_PAIR", "0")
    single = run_gemm(torch, w, x, torch.float32)
    torch.testing.assert_close(paired, single, rtol=2e-5, atol=2e-5 * float(single.abs().max()))


@pytest.mark.parametrize("fmt", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("m", [40, 300])
def test_swiglu_of_many_bf16_tokens_runs_its_projections_on_the_gemm(cuda, monkeypatch, fmt, m):
    from mylocal_llm_b200 import quantized_swiglu
    from oracle import packed_oracle as po
    torch = cuda
    f, k = 384, 1024
    rng = np.random.default_rng(m)
    gate_w = quantize(rng.normal(0, 0.03, (f, k)).astype(np.float32), fmt)
    up_w = quantize(rng.normal(0, 0.03, (f, k)).astype(np.float32), fmt)
    gate, up = packed_to_device(gate_w), packed_to_device(up_w)
    x = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    calls = []
    real = _lib.call
    monkeypatch.setattr(_lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    h = quantized_swiglu(x, gate, up, out_dtype=torch.float32)
    assert calls == ["b200q_gemm", "b200q_gemm", "b200q_silu_mul"]
    calls.clear()
    monkeypatch.setenv("B200Q_GEMM", "0")
    h_gemv = quantized_swiglu(x, gate, up, out_dtype=torch.float32)
    assert calls == ["b200q_swiglu"]
    ref = po.swiglu_fp64(x.float().cpu().numpy(), (gate_w.data, gate_w.shape, fmt), (up_w.data, up_w.shape, fmt))
    scale = float(np.abs(ref).max())
    np.testing.assert_allclose(h_gemv.cpu().numpy(), ref, rtol=3e-4, atol=2e-4)             # the exact-product path
    # the GEMM route: BF16-rounded weights in both projections (2^-9 relative each) before the product of the two
    assert float(np.abs(h.cpu().numpy() - ref).max()) <= 1e-2 * scale
