"""Llama-family decoder on packed linears: prefill and decode logits against the FP64 oracle."""

import numpy as np
import pytest

from oracle import llama_oracle as lo
from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel
from mylocal_llm_b200.quantize import quantize

pytestmark = pytest.mark.gpu

CFG = dict(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=64, max_position_embeddings=64, rope_theta=10000.0, rms_norm_eps=1e-5)
FORMATS = {"self_attn.q_proj": "Q8_0", "self_attn.k_proj": "Q8_0", "self_attn.v_proj": "Q5_K",
           "self_attn.o_proj": "Q8_0", "mlp.gate_proj": "Q4_K", "mlp.up_proj": "Q4_K", "mlp.down_proj": "Q6_K"}


def make_weights(model, seed=0, uniform=False):
    """Mixed formats by default; ``uniform`` = Q8_0 everywhere (the model then stacks q/k/v and
    gate/up into single matrices)."""
    rng = np.random.default_rng(seed)
    packed, oracle = {}, {}
    for name, shape in model.expected_shapes().items():
        if len(shape) == 1:
            packed[name] = oracle[name] = (1.0 + 0.1 * rng.normal(size=shape)).astype(np.float32)
            continue
        fmt = "Q8_0" if uniform else next((f for key, f in FORMATS.items() if key in name), "Q8_0")
        scale = 0.5 if "embed" in name else 1.0 / np.sqrt(shape[1])
        w = quantize(rng.normal(0, scale, shape).astype(np.float32), fmt)
        packed[name] = w
        oracle[name] = (w.data, w.shape, fmt)
    return packed, oracle


@pytest.mark.parametrize("uniform", [False, True])
@pytest.mark.parametrize("dtype,rtol,atol", [("float32", 2e-3, 2e-3), ("bfloat16", 6e-2, 6e-2)])
def test_prefill_and_decode_logits_match_the_oracle(cuda, dtype, rtol, atol, uniform):
    torch = cuda
    model = ExternalLlamaModel(ExternalLlamaConfig(**CFG), dtype=dtype)
    packed, oracle = make_weights(model, uniform=uniform)
    model.set_weights(packed)
    assert (model.layers[0]["qkv"] is not None) == uniform and (model.layers[0]["gate_up"] is not None) == uniform
    tokens = np.random.default_rng(1).integers(0, CFG["vocab_size"], 12)
    state = model.create_generation_state(1, 32)
    prompt = torch.from_numpy(tokens[:9][None]).cuda()
    logits = model.prefill(prompt, state)
    ref = lo.llama_logits(oracle, CFG, tokens)
    scale = np.abs(ref).max()
    np.testing.assert_allclose(logits[0].cpu().numpy(), ref[8], rtol=rtol, atol=atol * scale)
    for step in range(9, 12):
        logits = model.decode_one(torch.from_numpy(tokens[step:step + 1]).cuda(), state)
        np.testing.assert_allclose(logits[0].cpu().numpy(), ref[step], rtol=rtol, atol=atol * scale)
    assert state.length == 12 and int(state.position.item()) == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fused_decode_kernels_agree_with_the_framework_ops(cuda, dtype):
    """RoPE + cache store and single-query attention as two kernels vs the same step in torch ops."""
    torch = cuda
    model = ExternalLlamaModel(ExternalLlamaConfig(**CFG), dtype=dtype)
    packed, _ = make_weights(model, seed=7, uniform=dtype == "bfloat16")
    model.set_weights(packed)
    tokens = torch.from_numpy(np.random.default_rng(8).integers(0, CFG["vocab_size"], (2, 9))).cuda()
    outs = {}
    for fused in (True, False):
        model.fused_decode = fused
        state = model.create_generation_state(2, 24)
        model.prefill(tokens[:, :5].contiguous(), state)
        outs[fused] = [model.decode_one(tokens[:, i].contiguous(), state).clone() for i in range(5, 9)]
        outs[fused].append(state.k.float().clone())
    tol = 2e-5 if dtype == "float32" else 3e-2
    for a, b in zip(outs[True], outs[False]):
        scale = float(b.abs().max())
        assert float((a - b).abs().max()) <= tol * max(scale, 1.0)


def test_batched_prefill_rows_are_independent(cuda):
    torch = cuda
    model = ExternalLlamaModel(ExternalLlamaConfig(**CFG), dtype="float32")
    packed, _ = make_weights(model, seed=3)
    model.set_weights(packed)
    tokens = torch.from_numpy(np.random.default_rng(2).integers(0, CFG["vocab_size"], (3, 7))).cuda()
    both = model.prefill(tokens, model.create_generation_state(3, 16))
    for row in range(3):
        one = model.prefill(tokens[row:row + 1].contiguous(), model.create_generation_state(1, 16))
        np.testing.assert_allclose(both[row].cpu().numpy(), one[0].cpu().numpy(), rtol=1e-5, atol=1e-5)


def test_decode_step_replays_from_a_cuda_graph(cuda):
    torch = cuda
    model = ExternalLlamaModel(ExternalLlamaConfig(**CFG), dtype="bfloat16")
    packed, _ = make_weights(model, seed=5)
    model.set_weights(packed)
    tokens = torch.from_numpy(np.random.default_rng(4).integers(0, CFG["vocab_size"], 10)).cuda()
    eager_state = model.create_generation_state(1, 32)
    model.prefill(tokens[None, :6].contiguous(), eager_state)
    eager = [model.decode_one(tokens[i:i + 1], eager_state).clone() for i in range(6, 10)]

    state = model.create_generation_state(1, 32)
    model.prefill(tokens[None, :6].contiguous(), state)
    token = tokens[6:7].clone()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        snapshot = (state.k.clone(), state.v.clone(), state.position.clone())
        model.decode_one(token, state)                                   # warm-up outside the graph
        state.k.copy_(snapshot[0]); state.v.copy_(snapshot[1]); state.position.copy_(snapshot[2])
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = model.decode_one(token, state)
        state.k.copy_(snapshot[0]); state.v.copy_(snapshot[1]); state.position.copy_(snapshot[2])
        for i in range(6, 10):
            token.copy_(tokens[i:i + 1])
            graph.replay()
            stream.synchronize()
            assert torch.equal(out, eager[i - 6])


def test_set_weights_rejects_incomplete_or_misshaped_imports(cuda):
    model = ExternalLlamaModel(ExternalLlamaConfig(**CFG))
    packed, _ = make_weights(model)
    missing = dict(packed)
    missing.pop("model.layers.1.mlp.down_proj.weight")
    with pytest.raises(ValueError):
        model.set_weights(missing)
    wrong = dict(packed)
    wrong["model.norm.weight"] = np.ones(7, np.float32)
    with pytest.raises(ValueError):
        model.set_weights(wrong)
    with pytest.raises(RuntimeError):
        model.create_generation_state()
    with pytest.raises(ValueError):
        ExternalLlamaConfig(**{**CFG, "num_key_value_heads": 3}).validate()


def test_one_layer_of_the_third_configuration_prefill_gemm_and_decode(cuda, monkeypatch):
    """The layer shape of the third benchmark configuration (hidden 2048, 32 heads of 64, FFN 8192, Q8_0
    everywhere, BF16 activations) with one layer and a small vocabulary: a 48-token prefill - long enough
    for the projections to run on the tensor-core GEMM from their GGUF-layout copies - and two decode steps
    against the FP64 oracle, and the prefill again with the GEMM switched off (GEMV passes on the tile
    layouts): both must meet the BF16 band, and agree with each other within it."""
    torch = cuda
    cfg = dict(vocab_size=512, hidden_size=2048, intermediate_size=8192, num_hidden_layers=1, num_attention_heads=32,
               num_key_value_heads=32, head_dim=64, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5)
    model = ExternalLlamaModel(ExternalLlamaConfig(**cfg), dtype="bfloat16")
    rng = np.random.default_rng(3)
    packed, oracle = {}, {}
    for name, shape in model.expected_shapes().items():
        if len(shape) == 1:
            packed[name] = oracle[name] = np.ones(shape, np.float32)
            continue
        w = quantize(rng.normal(0, 0.5 if "embed" in name else 0.02, shape).astype(np.float32), "Q8_0")
        packed[name], oracle[name] = w, (w.data, w.shape, "Q8_0")
    model.set_weights(packed)
    assert model.native_of, "no GGUF-layout copies were kept for the prefill GEMM"
    tokens = rng.integers(0, cfg["vocab_size"], 50)
    ref = lo.llama_logits(oracle, cfg, tokens)
    scale = np.abs(ref).max()
    calls = []
    from mylocal_llm_b200 import _lib
    real = _lib.call
    monkeypatch.setattr(_lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    state = model.create_generation_state(1, 64)
    logits = model.prefill(torch.from_numpy(tokens[:48][None]).cuda(), state)
    # qkv, o, gate|up, down of the one layer (a projection with few row tiles takes the split-K entry point)
    assert calls.count("b200q_gemm") + calls.count("b200q_gemm_ws") == 4, calls
    np.testing.assert_allclose(logits[0].cpu().numpy(), ref[47], rtol=6e-2, atol=6e-2 * scale)
    for step in (48, 49):
        logits = model.decode_one(torch.from_numpy(tokens[step:step + 1]).cuda(), state)
        np.testing.assert_allclose(logits[0].cpu().numpy(), ref[step], rtol=6e-2, atol=6e-2 * scale)
    monkeypatch.setenv("B200Q_GEMM", "0")
    calls.clear()
    state2 = model.create_generation_state(1, 64)
    logits2 = model.prefill(torch.from_numpy(tokens[:48][None]).cuda(), state2)
    assert "b200q_gemm" not in calls
    np.testing.assert_allclose(logits2[0].cpu().numpy(), ref[47], rtol=6e-2, atol=6e-2 * scale)
