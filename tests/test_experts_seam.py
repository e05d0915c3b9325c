"""``ExpertsInference`` driven through the reference's executor seam (``forward`` / ``try_forward_grouped`` /
``dispatch_scope``, mini_llm/ops/experts_inference.py:188-312, expert_residency.py:539-560,1166-1208) with a
fake executor on CPU tensors: dispatch order, scope handling, the grouped hand-off with routing slots, the
fall-through when the executor declines, repeated ids, and the ``on_cpu_submitted`` callback."""

import contextlib

import numpy as np
import pytest
import torch

from mylocal_llm_b200 import ExpertsInference

D, E = 8, 6


class FakeExecutor:
    """Expert e multiplies its rows by (e + 1); records every call."""

    def __init__(self, grouped=None):
        self.calls, self.depth, self.grouped = [], 0, grouped

    @contextlib.contextmanager
    def dispatch_scope(self, layer_id, expert_ids):
        self.calls.append(("scope", layer_id, tuple(expert_ids)))
        self.depth += 1
        try:
            yield
        finally:
            self.depth -= 1

    def forward(self, layer_id, expert_id, x):
        assert self.depth == 1, "expert calls must happen inside the dispatch scope"
        self.calls.append(("forward", layer_id, int(expert_id), tuple(x.shape)))
        return x * float(expert_id + 1)

    def try_forward_grouped(self, layer_id, expert_ids, x, routing_weights, slots):
        assert self.depth == 1
        self.calls.append(("grouped", layer_id, tuple(expert_ids), tuple(slots)))
        if self.grouped == "decline":
            return None
        out = torch.zeros_like(x)
        for e, s in zip(expert_ids, slots):
            out += routing_weights[s] * x * float(e + 1)
        return out


def expected(x, w, ids):
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        for s in np.argsort(ids[t], kind="stable"):
            out[t] += w[t, s] * x[t] * (ids[t, s] + 1)
    return out


def test_many_rows_run_each_active_expert_once_in_ascending_order():
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (1, 5, D)).astype(np.float32)
    ids = np.array([[4, 1], [1, 3], [0, 4], [3, 1], [5, 0]])
    w = rng.random((5, 2)).astype(np.float32)
    ex = FakeExecutor()
    layer = ExpertsInference(D, 4, E, expert_executor=ex, layer_id=7)
    out = layer.forward(torch.from_numpy(x), torch.from_numpy(w)[None], torch.from_numpy(ids)[None])
    np.testing.assert_allclose(out[0].numpy(), expected(x[0], w, ids), rtol=1e-6, atol=1e-6)
    assert ex.calls[0] == ("scope", 7, (0, 1, 3, 4, 5))
    assert [c[2] for c in ex.calls if c[0] == "forward"] == [0, 1, 3, 4, 5]
    assert [c[3] for c in ex.calls if c[0] == "forward"] == [(2, D), (3, D), (2, D), (2, D), (1, D)]
    assert not any(c[0] == "grouped" for c in ex.calls)          # the grouped hook is a one-row hand-off


@pytest.mark.parametrize("grouped", ["accept", "decline"])
def test_one_row_offers_the_grouped_hook_with_slots_then_falls_through(grouped):
    x = np.arange(D, dtype=np.float32)[None, None] / 10
    ids = np.array([[5, 2, 3]])
    w = np.array([[0.5, 0.25, 0.125]], np.float32)
    ex = FakeExecutor(grouped)
    seen = []
    layer = ExpertsInference(D, 4, E, expert_executor=ex, layer_id=1)
    out = layer.forward(torch.from_numpy(x), torch.from_numpy(w)[None], torch.from_numpy(ids)[None],
                        on_cpu_submitted=lambda: seen.append(1))
    np.testing.assert_allclose(out[0].numpy(), expected(x[0], w, ids), rtol=1e-6, atol=1e-6)
    assert ex.calls[1] == ("grouped", 1, (2, 3, 5), (1, 2, 0))   # ascending ids, slots into the [k] weights
    assert bool([c for c in ex.calls if c[0] == "forward"]) == (grouped == "decline")
    assert seen == [1] and ex.depth == 0


def test_one_row_with_a_repeated_id_takes_the_general_dispatch():
    x = np.ones((1, 1, D), np.float32)
    ids = np.array([[2, 2, 0]])
    w = np.array([[0.5, 0.25, 1.0]], np.float32)
    ex = FakeExecutor()
    layer = ExpertsInference(D, 4, E, expert_executor=ex)
    out = layer.forward(torch.from_numpy(x), torch.from_numpy(w)[None], torch.from_numpy(ids)[None])
    np.testing.assert_allclose(out[0].numpy(), expected(x[0], w, ids), rtol=1e-6, atol=1e-6)
    assert not any(c[0] == "grouped" for c in ex.calls)
    assert [c for c in ex.calls if c[0] == "forward"] == [("forward", 0, 0, (1, D)), ("forward", 0, 2, (2, D))]


def test_ids_outside_the_expert_range_are_rejected_before_any_call():
    ex = FakeExecutor()
    layer = ExpertsInference(D, 4, E, expert_executor=ex)
    with pytest.raises(ValueError):
        layer.forward(torch.ones((1, 1, D)), torch.ones((1, 1, 1)), torch.tensor([[[E]]]))
    assert ex.calls == []
