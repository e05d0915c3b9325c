"""The one-token step of an MoE stack as one persistent kernel must return the bits of the chain of launches.

``b200q_moe_decode_stack`` walks router, top-k + plan, grouped gate/up, grouped down and combine + norm of every
layer inside one cooperative grid; ``PackedMoEStack.forward`` uses it for a single row. The stages are the device
functions the separate kernels are made of, so residual stream and activations must be bit-identical - eagerly,
captured in a CUDA graph, and replayed back to back - and no wait may have run out (device status 0).
"""

import numpy as np
import pytest

from mylocal_llm_b200 import _lib
from mylocal_llm_b200.moe_stack import PackedMoEStack

pytestmark = pytest.mark.gpu

SHAPES = {
    "small": dict(n_layers=3, d_model=512, d_ff=256, n_experts=32, top_k=4, shared_d_ff=256),
    "bench": dict(n_layers=2, d_model=2048, d_ff=512, n_experts=512, top_k=10, shared_d_ff=512),
    "wide-k": dict(n_layers=2, d_model=1024, d_ff=256, n_experts=64, top_k=15, shared_d_ff=256),
}


def logged(fn):
    calls = []
    real = _lib.call
    _lib.call = lambda name, *a: (calls.append(name), real(name, *a))[1]
    try:
        out = fn()
    finally:
        _lib.call = real
    return out, calls


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_persistent_step_matches_the_chain_of_launches(cuda, shape):
    cfg = dict(SHAPES[shape])
    stack = PackedMoEStack.synthetic(cfg.pop("n_layers"), seed=3, **cfg)
    x = cuda.from_numpy(np.random.default_rng(5).normal(0, 1, (1, 1, cfg["d_model"])).astype(np.float32)).cuda()
    stack.persistent_step = False
    (res_chain, hid_chain), calls = logged(lambda: stack.forward(x))
    assert "b200q_moe_decode_stack" not in calls
    stack.persistent_step = True
    (res, hid), calls = logged(lambda: stack.forward(x))
    assert calls == ["b200q_moe_decode_stack"], "the persistent step did not run"
    cuda.cuda.synchronize()
    assert _lib.device_status() == 0
    assert cuda.equal(res, res_chain) and cuda.equal(hid, hid_chain)
    assert bool(cuda.isfinite(res).all())
    # the step changes the stream: not a copy of the input
    assert not cuda.equal(res, x)


def test_persistent_step_in_a_graph_replayed_back_to_back(cuda):
    cfg = dict(SHAPES["small"])
    stack = PackedMoEStack.synthetic(cfg.pop("n_layers"), seed=9, **cfg)
    x = cuda.from_numpy(np.random.default_rng(6).normal(0, 1, (1, 1, cfg["d_model"])).astype(np.float32)).cuda()
    stack.persistent_step = False
    want = stack.forward(x)[0].clone()
    stack.persistent_step = True
    stream = cuda.cuda.Stream()
    with cuda.cuda.stream(stream):
        stack.forward(x)
        stream.synchronize()
        graph = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph, stream=stream):
            res, _ = stack.forward(x)
        outs = []
        for _ in range(4):
            graph.replay()
            outs.append(res.clone())
        stream.synchronize()
    assert _lib.device_status() == 0
    for out in outs:
        assert cuda.equal(out, want)


def test_more_rows_and_unfit_stacks_keep_the_chain(cuda):
    cfg = dict(SHAPES["small"])
    stack = PackedMoEStack.synthetic(cfg.pop("n_layers"), seed=1, **cfg)
    x2 = cuda.from_numpy(np.random.default_rng(7).normal(0, 1, (1, 2, cfg["d_model"])).astype(np.float32)).cuda()
    _, calls = logged(lambda: stack.forward(x2))
    assert "b200q_moe_decode_stack" not in calls
    # a router bias is outside what the persistent step covers: the stack declines, the chain runs
    stack.layers[1].router.b_router = cuda.zeros(cfg["n_experts"], device="cuda")
    x1 = x2[:, :1].contiguous()
    (res, _), calls = logged(lambda: stack.forward(x1))
    assert "b200q_moe_decode_stack" not in calls and bool(cuda.isfinite(res).all())
