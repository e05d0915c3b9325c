"""The allocation-free expert FFN entry point (collected last on purpose).

``b200q_expert_ffn_static`` serves callers that have no way to allocate device memory: a host that
binds the C ABI without a tensor framework, or a serving loop in which cudaMalloc is off limits. It
keeps the hidden activations in an array built into the library instead of a caller buffer. The
check: called through the C ABI twice in a row (the second call reuses the array with the first
call's contents still in it), its output must equal the two-call path (b200q_swiglu into a
caller-allocated buffer, then b200q_gemv) bit for bit, and oversized requests are refused.
"""

import ctypes

import numpy as np
import pytest

from mylocal_llm_b200 import _lib
from mylocal_llm_b200.quantize import quantize

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
