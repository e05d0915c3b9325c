"""Programmatic dependent launches of the decode chain must not change any result.

The kernels of a decode step are launched so that the next one may become resident while its
predecessor drains; each waits for the predecessor grid before touching memory. ``B200Q_CHAIN=0``
launches the same kernels with the usual full stream serialisation. Both settings have to give
bit-identical outputs, eagerly and when the step is captured in a CUDA graph and replayed
back to back (the case in which a missing wait would show up as a read of stale data).
"""

import numpy as np
import pytest

from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel
from mylocal_llm_b200.moe_stack import PackedMoEStack

pytestmark = pytest.mark.gpu

LLAMA = dict(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
             num_key_value_heads=4, head_dim=64, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5)


def run_stack(torch, stack, x, graph, replays):
    if not graph:
        outs = [stack.forward(x)[0].clone() for _ in range(replays)]
        torch.cuda.synchronize()
        return outs
    stream = torch.cuda.Stream()
    outs = []
    with torch.cuda.stream(stream):
        stack.forward(x)                                   # warm-up outside the capture
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            res, _ = stack.forward(x)
        for _ in range(replays):
            g.replay()
            outs.append(res.clone())
        stream.synchronize()
    return outs


@pytest.mark.parametrize("tokens", [1, 7, 64])
@pytest.mark.parametrize("graph", [False, True])
def test_moe_stack_is_identical_with_and_without_chained_launches(cuda, monkeypatch, tokens, graph):
    torch = cuda
    stack = PackedMoEStack.synthetic(4, d_model=512, d_ff=256, n_experts=32, top_k=4, shared_d_ff=256, seed=3)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(tokens)
    x = torch.randn((1, tokens, 512), device="cuda", generator=gen)
    monkeypatch.setenv("B200Q_CHAIN", "0")
    plain = run_stack(torch, stack, x, graph, 1)[0]
    monkeypatch.setenv("B200Q_CHAIN", "1")
    for out in run_stack(torch, stack, x, graph, 20):
        assert torch.equal(out, plain)
    assert bool(torch.isfinite(plain).all())


@pytest.mark.parametrize("batch", [1, 3])
def test_llama_decode_is_identical_with_and_without_chained_launches(cuda, monkeypatch, batch):
    torch = cuda
    model = ExternalLlamaModel.synthetic(ExternalLlamaConfig(**LLAMA), seed=1)
    prompt = torch.from_numpy(np.random.default_rng(2).integers(0, LLAMA["vocab_size"], (batch, 9))).cuda()

    def generate(chain, graph):
        monkeypatch.setenv("B200Q_CHAIN", chain)
        state = model.create_generation_state(batch, 64)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            token = model.prefill(prompt, state).argmax(dim=-1)
            seen = []
            if graph:
                token.copy_(model.decode_one(token, state).argmax(dim=-1))
                seen.append(token.clone())
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    logits = model.decode_one(token, state)
                    token.copy_(logits.argmax(dim=-1))
                for _ in range(12):
                    g.replay()
                    seen.append(logits.clone())
            else:
                token = model.decode_one(token, state).argmax(dim=-1)
                seen.append(token.clone())
                for _ in range(12):
                    logits = model.decode_one(token, state)
                    token = logits.argmax(dim=-1)
                    seen.append(logits.clone())
            stream.synchronize()
        return seen

    reference = generate("0", graph=False)
    for chain, graph in (("1", False), ("1", True), ("0", True)):
        got = generate(chain, graph)
        assert len(got) == len(reference)
        for a, b in zip(got, reference):
            assert torch.equal(a, b), f"chain={chain} graph={graph}"
