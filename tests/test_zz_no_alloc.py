"""The allocation-free expert FFN entry point (collected last on purpose).

``b200q_expert_ffn_static`` serves callers that have no way to allocate device memory: a host that
binds the C ABI without a tensor framework, or a serving loop in which cudaMalloc is off limits. It
keeps the hidden activations in an array built into the library instead of a caller buffer. The
check: called through the C ABI twice in a row (the second call reuses the array with the first
call's contents still in it), its output must equal the two-call path (b200q_swiglu into a
caller-allocated buffer, then b200q_gemv) bit for bit, and oversized requests are refused. The second
test runs the formats and layouts the MoE layers use by default (Q4_K gate/up and Q6_K down, both in the
device tile layouts), whose kernels start early behind their predecessor on the stream: two calls back to
back, so the second call's first kernel may become resident while the first call's last kernel still
reads the shared array; results are checked against the two-call path and against the FP64 oracle.
"""

import ctypes

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import _lib, packed_to_device
from mylocal_llm_b200.quantize import quantize
from mylocal_llm_b200.quantized_linear import retile_gate_up, retile_weight

pytestmark = pytest.mark.gpu


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_scratch_expert_matches_two_call_path_twice(cuda):
    d, f = 512, 768
    rng = np.random.default_rng(2024)
    packs = [quantize(rng.normal(0, 0.05, s).astype(np.float32), q)
             for s, q in (((f, d), "Q4_K"), ((f, d), "Q5_K"), ((d, f), "Q6_K"))]
    dev = [cuda.from_numpy(p.data.copy()).cuda() for p in packs]
    fmt = [_lib.FORMAT_ID[p.quant_type] for p in packs]
    stream = _lib.current_stream()
    for call, m in enumerate((3, 8)):                       # two calls in a row, different batch sizes
        x = cuda.from_numpy(rng.normal(0, 1, (m, d)).astype(np.float32)).cuda()
        hidden = cuda.empty((m, f), dtype=cuda.float32, device="cuda")
        expect = cuda.empty((m, d), dtype=cuda.float32, device="cuda")
        _lib.call("b200q_swiglu", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], f, d, ptr(x), 0, m, ptr(hidden), 0, stream)
        _lib.call("b200q_gemv", ptr(dev[2]), fmt[2], d, f, ptr(hidden), 0, m, ptr(expect), 0, stream)
        got = cuda.full((m, d), float("nan"), dtype=cuda.float32, device="cuda")
        _lib.call("b200q_expert_ffn_static", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], ptr(dev[2]), fmt[2], d, f,
                  ptr(x), 0, m, ptr(got), 0, stream)
        cuda.cuda.synchronize()
        assert cuda.equal(got, expect), f"call {call}: static-scratch path differs from the two-call path"
    # beyond the built-in scratch: refused with a clear message, nothing launched
    with pytest.raises(NotImplementedError, match="exceeds the built-in scratch"):
        _lib.call("b200q_expert_ffn_static", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], ptr(dev[2]), fmt[2], d,
                  131072 + 256, ptr(x), 0, 1, ptr(got), 0, stream)


def test_static_scratch_expert_on_the_default_tile_layouts_back_to_back(cuda):
    d, f = 2048, 512                                          # the routed experts' shape in the benchmark
    rng = np.random.default_rng(7)
    packs = [quantize(rng.normal(0, 0.05, s).astype(np.float32), q)
             for s, q in (((f, d), "Q4_K"), ((f, d), "Q4_K"), ((d, f), "Q6_K"))]
    gate, up = retile_gate_up(packed_to_device(packs[0]), packed_to_device(packs[1]))
    down = retile_weight(packed_to_device(packs[2]))
    assert (gate.quant_type, up.quant_type, down.quant_type) == ("Q4_K_TILED", "Q4_K_TILED", "Q6_K_TILED")
    fmt = [_lib.FORMAT_ID[w.quant_type] for w in (gate, up, down)]
    dev = [w.data for w in (gate, up, down)]
    stream = _lib.current_stream()
    xs = [cuda.from_numpy(rng.normal(0, 1, (m, d)).astype(np.float32)).cuda() for m in (8, 1, 5)]
    gots = [cuda.full((x.shape[0], d), float("nan"), dtype=cuda.float32, device="cuda") for x in xs]
    for x, got in zip(xs, gots):                              # no synchronisation between the calls
        _lib.call("b200q_expert_ffn_static", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], ptr(dev[2]), fmt[2], d, f,
                  ptr(x), 0, x.shape[0], ptr(got), 0, stream)
    cuda.cuda.synchronize()
    trip = tuple((p.data, p.shape, p.quant_type) for p in packs)
    for x, got in zip(xs, gots):
        m = x.shape[0]
        hidden = cuda.empty((m, f), dtype=cuda.float32, device="cuda")
        expect = cuda.empty((m, d), dtype=cuda.float32, device="cuda")
        _lib.call("b200q_swiglu", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], f, d, ptr(x), 0, m, ptr(hidden), 0, stream)
        _lib.call("b200q_gemv", ptr(dev[2]), fmt[2], d, f, ptr(hidden), 0, m, ptr(expect), 0, stream)
        cuda.cuda.synchronize()
        assert cuda.equal(got, expect), f"m={m}: static-scratch path differs from the two-call path"
        # the reference's expert band (tests/test_0106l_q6k_packed.py:95): rtol 2e-4 / atol 2e-5
        np.testing.assert_allclose(got.cpu().numpy(), po.expert_ffn_fp64(x.cpu().numpy(), *trip), rtol=2e-4, atol=2e-5)
    # arguments the inner calls would refuse are refused before anything is launched
    with pytest.raises(ValueError):
        _lib.call("b200q_expert_ffn_static", ptr(dev[0]), fmt[0], ptr(dev[1]), fmt[1], ptr(dev[2]), 99, d, f,
                  ptr(xs[0]), 0, 1, ptr(gots[0]), 0, stream)
    with pytest.raises(ValueError):
        _lib.call("b200q_expert_ffn_static", ptr(dev[0]), fmt[0], ptr(dev[1]), _lib.FORMAT_ID["Q4_K"], ptr(dev[2]),
                  fmt[2], d, f, ptr(xs[0]), 0, 1, ptr(gots[0]), 0, stream)
