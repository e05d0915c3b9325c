"""The Llama oracle against the reference's own model, and (GPU) the packed Llama model against the oracle.

``tests/golden/llama_golden.npz`` holds logits produced by the reference's ``ExternalLlamaModel``
(mini_llm/external/llama_model.py:75-178, NumPy backend, FP32) on Q8_0 weights: the prompt's last
position and three greedy decode steps (``tests/golden/make_golden.py llama``). The FP64 oracle
(``oracle/llama_oracle.py``) must reproduce them from the packed bytes within FP32 rounding; the GPU
model is then held to the oracle."""

import numpy as np
import pytest

from oracle import llama_oracle as lo
from tests.golden_llama import LLAMA_CONFIG, load_llama_golden


def oracle_steps(weights, prompt, tokens):
    """Last-position logits after the prompt and after each appended token (full causal forward each time)."""
    seq = [int(v) for v in prompt[0]]
    steps = [lo.llama_logits(weights, LLAMA_CONFIG, seq)[-1]]
    for token in tokens:
        seq.append(int(token))
        steps.append(lo.llama_logits(weights, LLAMA_CONFIG, seq)[-1])
    return np.stack(steps)


def test_llama_oracle_reproduces_the_reference_logits():
    weights, prompt, tokens, logits = load_llama_golden()
    got = oracle_steps(weights, prompt, tokens)
    # the reference computes in FP32 (NumPy BLAS); logits are O(1)
    np.testing.assert_allclose(got, logits, rtol=2e-4, atol=2e-5)
    assert [int(np.argmax(row)) for row in got[:-1]] == [int(t) for t in tokens]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,rtol,atol", [("float32", 2e-4, 2e-4), ("bfloat16", 6e-2, 6e-2)])
def test_packed_llama_model_matches_reference_logits(cuda, dtype, rtol, atol):
    torch = cuda
    from mylocal_llm_b200 import PackedGGUFWeight
    from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel
    weights, prompt, tokens, logits = load_llama_golden()
    model = ExternalLlamaModel(ExternalLlamaConfig(**LLAMA_CONFIG), dtype=dtype)
    packed = {name: (PackedGGUFWeight(w[0], w[1], w[2]) if isinstance(w, tuple) else w) for name, w in weights.items()}
    model.set_weights(packed)
    state = model.create_generation_state(1, 32)
    got = [model.prefill(torch.from_numpy(prompt).cuda(), state)[0].float().cpu().numpy()]
    for token in tokens:
        got.append(model.decode_one(torch.tensor([int(token)], device="cuda"), state)[0].float().cpu().numpy())
    got = np.stack(got)
    scale = float(np.abs(logits).max())
    np.testing.assert_allclose(got, logits, rtol=rtol, atol=atol * scale)
    if dtype == "float32":
        assert [int(np.argmax(row)) for row in got[:-1]] == [int(t) for t in tokens]
