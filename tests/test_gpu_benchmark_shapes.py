"""Parity at the shapes the benchmark runs: the packed MoE layer of the fourth baseline configuration
(hidden 2048, 512 experts of width 512, top-10 renormalised routing, always-on shared expert, Q4_K
gate/up + Q6_K down in the device tile layouts, BF16 hidden states) for 1, 16, 64 and 256 tokens, and
the norm -> layer -> residual chain of the 48-layer stack on two of its layers, against the FP64
layer oracle (tests/test_0106o_qwen3next_decoder.py:103-127 of the reference, restated in
oracle/packed_oracle.py). The launch heuristics of the grouped kernels (K split, row groups, segment
lists of several hundred entries, 513-entry pointer tables) only take their benchmark values here.

Tolerances. FP32 hidden states: the reference's grouped-expert band (rtol 4e-4 / atol 8e-6,
tests/test_0106t_grouped_dispatch.py:172) with the absolute part scaled by the largest output, since
these outputs are O(10..100) where the reference's fixtures are O(0.1). BF16 hidden states are not
covered by any reference test; they get the FP16 band of tests/test_0106c:99-100 (rtol 2e-2 /
atol 6e-3) with the absolute part scaled by the output's RMS. Routing: the device routes in FP32, the
oracle in FP64; a row whose k-th and (k+1)-th logits differ by less than 1e-5 may legitimately pick
another expert and is left out (at most two such rows are tolerated per case).
"""

import numpy as np
import pytest

from oracle import build_oracle as bo
from oracle import packed_oracle as po
from mylocal_llm_b200.experts_inference import synthetic_bank
from mylocal_llm_b200.moe_stack import PackedMoEStack
from mylocal_llm_b200.quantize import random_packed

pytestmark = pytest.mark.gpu

D, F, E, K, FLOOR = 2048, 512, 512, 10, 2.0 ** -14
TYPES = ("Q4_K", "Q4_K", "Q6_K")


def host_layer(torch, stack, seed, index):
    """Host copies of what PackedMoEStack.synthetic(seed=seed) generated for layer `index`: native GGUF
    bytes of the expert bank (the layer itself holds the tile layouts), shared expert, router weight."""
    bank = synthetic_bank(E, D, F, TYPES, seed=seed * 1000 + index)
    raw = [b.cpu().numpy() for b in (bank.gate, bank.up, bank.down)]
    strides = (bank.gate_stride, bank.up_stride, bank.down_stride)
    shapes = ((F, D), (F, D), (D, F))
    del bank
    torch.cuda.empty_cache()

    def expert_of(e):
        return tuple((raw[j][e * strides[j]:(e + 1) * strides[j]], shapes[j], TYPES[j]) for j in range(3))

    shared = tuple((w.data, w.shape, w.quant_type) for w in (
        random_packed(fmt, shape, seed=seed * 7919 + 3 * index + j, d=1.0 / 2048, dmin=1.0 / 4096)
        for j, (fmt, shape) in enumerate(zip(TYPES, shapes))))
    router = stack.layers[index].router.W_router.cpu().numpy()
    return expert_of, shared, router


def tie_free_rows(h64, router, ids_device):
    """Rows whose FP64 top-k set equals the device's; the others must be near ties."""
    logits = h64 @ router.astype(np.float64)
    _, ids64 = po.router_topk(logits, K, FLOOR)
    keep = []
    for r in range(h64.shape[0]):
        if set(ids64[r]) == set(int(v) for v in ids_device[r]):
            keep.append(r)
            continue
        ordered = np.sort(logits[r])[::-1]
        assert ordered[K - 1] - ordered[K] < 1e-5, f"row {r}: device top-k differs from FP64 without a near tie"
    assert len(keep) >= h64.shape[0] - 2
    return np.asarray(keep)


def check_layer(torch, layer, host, x, dtype_name):
    expert_of, shared, router = host
    out = layer.forward(x)[0].float().cpu().numpy()
    h64 = x[0].double().cpu().numpy()
    _, ids_dev = layer.router.forward(x)
    rows = tie_free_rows(h64, router, ids_dev[0].cpu().numpy())
    ref, _, _ = po.moe_layer_fp64_grouped(h64, router, K, FLOOR, expert_of, shared, rows=rows,
                                          dequant=bo.port_dequantize)
    got = out[rows]
    if dtype_name == "float32":
        rtol, atol = 4e-4, 8e-6 * max(1.0, float(np.abs(ref).max()))
    else:
        rtol, atol = 2e-2, 6e-3 * float(np.sqrt((ref ** 2).mean()))
    ratio = np.abs(got - ref) / (atol + rtol * np.abs(ref))
    assert ratio.max() <= 1.0, f"tolerance ratio {ratio.max():.3f} at {np.unravel_index(ratio.argmax(), ratio.shape)}"
    return float(ratio.max())


@pytest.fixture(scope="module")
def one_layer(cuda):
    stack = PackedMoEStack.synthetic(1, seed=3)
    layer = stack.layers[0]
    assert (layer.bank.gate_type, layer.bank.up_type, layer.bank.down_type) == ("Q4_K_TILED", "Q4_K_TILED", "Q6_K_TILED")
    assert layer._tables is not None, "the shared expert must run through the grouped kernels as expert 512"
    return layer, host_layer(cuda, stack, 3, 0)


@pytest.mark.parametrize("tokens,dtype_name", [(1, "bfloat16"), (16, "bfloat16"), (64, "bfloat16"), (256, "bfloat16"),
                                               (1, "float32"), (16, "float32"), (64, "float32")])
def test_benchmark_moe_layer_matches_the_fp64_layer_oracle(cuda, one_layer, tokens, dtype_name):
    torch = cuda
    layer, host = one_layer
    rng = np.random.default_rng(1000 + tokens)
    x = torch.from_numpy(rng.normal(0, 1, (1, tokens, D)).astype(np.float32)).cuda().to(getattr(torch, dtype_name))
    check_layer(torch, layer, host, x, dtype_name)
    from mylocal_llm_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("tokens", [1, 16])
def test_two_layers_of_the_benchmark_stack_match_the_fp64_chain(cuda, tokens):
    """RMSNorm -> MoE layer -> residual add, twice, as bench.py's stack chains them: every layer's output
    is checked against the FP64 layer oracle fed with that layer's own input, and the residual stream
    and the normalised activations against the FP64 residual-add RMSNorm fed with the device's branch."""
    torch = cuda
    seed = 5
    stack = PackedMoEStack.synthetic(2, seed=seed)
    rng = np.random.default_rng(77 + tokens)
    residual = torch.from_numpy(rng.normal(0, 1, (1, tokens, D)).astype(np.float32)).cuda()
    trace = []
    res_out, hidden_out = stack.forward(residual, trace=trace)
    plain_res, plain_hidden = stack.forward(residual)                # the path bench.py times
    assert torch.equal(plain_res, res_out) and torch.equal(plain_hidden, hidden_out)
    assert len(trace) == 2
    gamma = np.ones(D)
    res64 = residual[0].double().cpu().numpy()
    first_in = po.rmsnorm_fp64(res64, gamma, 1e-5)
    np.testing.assert_allclose(trace[0][0][0].float().cpu().numpy(), first_in, rtol=2 ** -8, atol=1e-6)
    for index, (layer_in, branch) in enumerate(trace):
        host = host_layer(torch, stack, seed, index)
        check_layer(torch, stack.layers[index], host, layer_in, "bfloat16")
        res_ref, y_ref = po.residual_rmsnorm_fp64(res64, branch[0].double().cpu().numpy(), gamma, 1e-5)
        res64 = res_ref.astype(np.float64)
        nxt = trace[index + 1][0] if index + 1 < len(trace) else hidden_out
        np.testing.assert_allclose(nxt[0].float().cpu().numpy(), y_ref, rtol=2 ** -8, atol=1e-6)
    np.testing.assert_allclose(res_out[0].cpu().numpy(), res64, rtol=1e-6, atol=1e-6)
