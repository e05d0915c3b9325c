"""Residual add + RMSNorm fused into the projection that consumes it (``b200q_gemv_norm``) must return the bits of
``b200q_residual_rmsnorm`` followed by ``b200q_gemv``: the same norm arithmetic run by every CTA of the GEMV, the
same GEMV body. Checked on the operator and on the Llama one-token step (eager and in a replayed CUDA graph)."""

import ctypes

import numpy as np
import pytest

from mylocal_llm_b200 import _lib, packed_to_device, quantized_linear
from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel
from mylocal_llm_b200.moe_layer import RMSNormInference
from mylocal_llm_b200.quantize import quantize
from mylocal_llm_b200.quantized_linear import retile_weight

pytestmark = pytest.mark.gpu

ptr = lambda t: ctypes.c_void_p(t.data_ptr())
dtype_id = lambda t: _lib.DTYPE_ID[str(t.dtype).replace("torch.", "")]


def fused(torch, weight, residual, branch, norm, out_dtype):
    rows, k = residual.shape
    n = weight.shape[0]
    res_out = torch.full_like(residual, float("nan"))
    y = torch.full((rows, n), float("nan"), dtype=out_dtype, device="cuda")
    _lib.call("b200q_gemv_norm", ptr(weight.data), _lib.FORMAT_ID[weight.quant_type], n, k, ptr(residual), ptr(branch),
              dtype_id(branch), 1.0, ptr(norm.gamma), dtype_id(norm.gamma), float(norm.eps), rows, ptr(res_out), ptr(y),
              dtype_id(y), _lib.current_stream())
    return res_out, y


@pytest.mark.parametrize("fmt", ["Q8_0", "Q6_K"])
@pytest.mark.parametrize("n,k", [(6144, 2048), (64, 256), (2048, 4096), (49152, 2048)])
@pytest.mark.parametrize("rows", [1, 2, 4])
@pytest.mark.parametrize("act", ["bfloat16", "float16"])
def test_fused_norm_gemv_equals_the_two_launches(cuda, fmt, n, k, rows, act):
    torch = cuda
    if n * k > 2048 * 4096 and (rows != 1 or fmt != "Q8_0" or act != "bfloat16"):
        pytest.skip("the large shape once")
    rng = np.random.default_rng(n + k + rows)
    weight = retile_weight(packed_to_device(quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), fmt)))
    assert weight.quant_type == fmt + "_TILED"
    dt = getattr(torch, act)
    norm = RMSNormInference(k, eps=1e-5)
    norm.set_weights(torch.from_numpy(rng.normal(1, 0.1, k).astype(np.float32)).cuda().to(dt))
    residual = torch.from_numpy(rng.normal(0, 1, (rows, k)).astype(np.float32)).cuda()
    branch = torch.from_numpy(rng.normal(0, 1, (rows, k)).astype(np.float32)).cuda().to(dt)
    res_want, hidden = norm.forward_residual_add(residual, branch)
    for out_dtype in (torch.float32, dt):
        want = quantized_linear(hidden, weight, out_dtype=out_dtype)
        res_got, got = fused(torch, weight, residual, branch, norm, out_dtype)
        torch.cuda.synchronize()
        assert torch.equal(res_got, res_want)
        assert torch.equal(got, want)
    assert _lib.device_status() == 0


def test_fused_norm_gemv_declines_what_it_does_not_cover(cuda):
    torch = cuda
    lib = _lib.load()
    q8, q8t, bf16, f32 = _lib.FORMAT_ID["Q8_0"], _lib.FORMAT_ID["Q8_0_TILED"], _lib.DTYPE_ID["bfloat16"], _lib.DTYPE_ID["float32"]
    assert lib.b200q_gemv_norm_supported(q8t, 2048, 2048, bf16, 1) == 1
    assert lib.b200q_gemv_norm_supported(q8, 2048, 2048, bf16, 1) == 0          # GGUF layout
    assert lib.b200q_gemv_norm_supported(q8t, 2048, 2048, f32, 1) == 0          # FP32 activations
    assert lib.b200q_gemv_norm_supported(q8t, 2048, 2048, bf16, 5) == 0         # too many rows
    assert lib.b200q_gemv_norm_supported(_lib.FORMAT_ID["Q4_K_TILED"], 2048, 2048, bf16, 1) == 0
    w = packed_to_device(quantize(np.random.default_rng(0).normal(0, 0.02, (64, 256)).astype(np.float32), "Q8_0"))
    norm = RMSNormInference(256)
    norm.set_weights(torch.ones(256, dtype=torch.bfloat16, device="cuda"))
    r = torch.zeros((1, 256), device="cuda")
    with pytest.raises(NotImplementedError):
        fused(torch, w, r, r.to(torch.bfloat16), norm, torch.float32)


LLAMA = dict(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
             num_key_value_heads=4, head_dim=64, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5)


@pytest.mark.parametrize("batch", [1, 2, 6])
@pytest.mark.parametrize("graph", [False, True])
def test_llama_one_token_step_with_deferred_norms(cuda, batch, graph):
    torch = cuda
    model = ExternalLlamaModel.synthetic(ExternalLlamaConfig(**LLAMA), seed=4)
    prompt = torch.randint(0, LLAMA["vocab_size"], (batch, 9), device="cuda")

    def run(fuse):
        model.fused_norm_linear = fuse
        state = model.create_generation_state(batch, 32)
        token = model.prefill(prompt, state).argmax(dim=-1)
        outs, calls = [], []
        real = _lib.call
        _lib.call = lambda name, *a: (calls.append(name), real(name, *a))[1]
        try:
            if not graph:
                for _ in range(3):
                    logits = model.decode_one(token, state)
                    outs.append(logits.clone())
                    token = logits.argmax(dim=-1)
            else:
                stream = torch.cuda.Stream()
                with torch.cuda.stream(stream):
                    step = lambda: token.copy_(model.decode_one(token, state).argmax(dim=-1))
                    step()
                    stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        logits = model.decode_one(token, state)
                        token.copy_(logits.argmax(dim=-1))
                    for _ in range(3):
                        g.replay()
                        outs.append(logits.clone())
                    stream.synchronize()
        finally:
            _lib.call = real
        return outs, calls

    want, calls_plain = run(False)
    got, calls_fused = run(True)
    assert "b200q_gemv_norm" not in calls_plain
    if batch == 1:
        assert "b200q_gemv_norm" in calls_fused and "b200q_residual_rmsnorm" not in calls_fused
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("fmt", ["Q8_0", "Q6_K"])
@pytest.mark.parametrize("n,k", [(2048, 8192), (64, 256), (512, 1024)])
@pytest.mark.parametrize("rows", [1, 3])
@pytest.mark.parametrize("act", ["bfloat16", "float16"])
def test_fused_silu_gemv_equals_the_two_launches(cuda, fmt, n, k, rows, act):
    """``b200q_gemv_silu`` (SiLU(gate) * up computed by every CTA of the down projection) against ``b200q_silu_mul``
    followed by ``b200q_gemv``: same bits."""
    torch = cuda
    if n * k > 512 * 1024 and (fmt != "Q8_0" or act != "bfloat16"):
        pytest.skip("the large shape once per row count")
    rng = np.random.default_rng(n + k + rows)
    # (force: K = 8192 is tiled only for callers that pass 16-bit activations, as the Llama model does)
    weight = retile_weight(packed_to_device(quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), fmt)), force=True)
    assert weight.quant_type == fmt + "_TILED"
    dt = getattr(torch, act)
    gu = torch.from_numpy(rng.normal(0, 2, (rows, 2 * k)).astype(np.float32)).cuda()
    gu[0, :4] = torch.tensor([-100.0, 100.0, 0.0, -0.0], device="cuda")          # both branches of the logistic
    act_rows = torch.empty((rows, k), dtype=dt, device="cuda")
    _lib.call("b200q_silu_mul", ptr(gu), rows, k, ptr(act_rows), dtype_id(act_rows), _lib.current_stream())
    fmt_id = _lib.FORMAT_ID[weight.quant_type]
    assert _lib.load().b200q_gemv_silu_supported(fmt_id, n, k, dtype_id(act_rows), rows) == 1
    for out_dtype in (torch.float32, dt):
        want = quantized_linear(act_rows, weight, out_dtype=out_dtype)
        got = torch.full((rows, n), float("nan"), dtype=out_dtype, device="cuda")
        _lib.call("b200q_gemv_silu", ptr(weight.data), fmt_id, n, k, ptr(gu), dtype_id(act_rows), rows, ptr(got),
                  dtype_id(got), _lib.current_stream())
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert _lib.device_status() == 0


def test_llama_one_token_step_fusions_change_no_bit(cuda, monkeypatch):
    """RoPE + cache store inside the attention kernel and SiLU * up inside the down projection: the step's logits and
    its caches are those of the separate launches."""
    torch = cuda
    model = ExternalLlamaModel.synthetic(ExternalLlamaConfig(**LLAMA), seed=4)
    prompt = torch.randint(0, LLAMA["vocab_size"], (1, 9), device="cuda")

    def run():
        state = model.create_generation_state(1, 32)
        token = model.prefill(prompt, state).argmax(dim=-1)
        outs, calls = [], []
        real = _lib.call
        _lib.call = lambda name, *a: (calls.append(name), real(name, *a))[1]
        try:
            for _ in range(3):
                logits = model.decode_one(token, state)
                outs.append(logits.clone())
                token = logits.argmax(dim=-1)
        finally:
            _lib.call = real
        return outs, calls, [k.clone() for k in state.k], [v.clone() for v in state.v]

    monkeypatch.setenv("B200Q_SILU_GEMV", "1")            # off by default (measured slower at the 1.7B shape)
    got, calls_fused, k_got, v_got = run()
    monkeypatch.setenv("B200Q_ROPE_ATTENTION", "0")
    monkeypatch.setenv("B200Q_SILU_GEMV", "0")
    want, calls_plain, k_want, v_want = run()
    assert "b200q_rope_attention" in calls_fused and "b200q_rope_kv_store" not in calls_fused
    assert "b200q_gemv_silu" in calls_fused and "b200q_silu_mul" not in calls_fused
    assert "b200q_rope_kv_store" in calls_plain and "b200q_silu_mul" in calls_plain
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    for a, b in zip(k_got + v_got, k_want + v_want):
        assert torch.equal(a, b)
    assert _lib.device_status() == 0
