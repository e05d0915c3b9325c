"""Host logic of the expert-parallel MoE layer on CPU: two gloo ranks, NumPy experts.

The device steps are replaced by a NumPy engine with the oracle's routing and summation rules, so
what is under test is the partitioning, the row gather, the term exchange and the home-rank combine
of ``mylocal_llm_b200.expert_parallel`` - the result must equal the single-process layer bit for bit.
"""

import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mylocal_llm_b200.expert_parallel import (CollectiveComm, ExpertParallelMoELayer, LocalComm, expert_partition)
from oracle import packed_oracle as po

D, F, K, FLOOR = 32, 16, 2, 2.0 ** -14


def test_expert_partition_is_contiguous_and_balanced():
    assert expert_partition(512, 8) == [(64 * r, 64) for r in range(8)]
    assert expert_partition(7, 2) == [(0, 4), (4, 3)]
    assert expert_partition(5, 5) == [(r, 1) for r in range(5)]
    parts = expert_partition(513, 4)
    assert parts[0][0] == 0 and sum(c for _, c in parts) == 513
    assert all(parts[i][0] + parts[i][1] == parts[i + 1][0] for i in range(3))
    with pytest.raises(ValueError):
        expert_partition(3, 4)


def _model(n_experts, seed=5):
    rng = np.random.default_rng(seed)
    experts = [(rng.normal(0, 0.2, (F, D)), rng.normal(0, 0.2, (F, D)), rng.normal(0, 0.2, (D, F)))
               for _ in range(n_experts + 1)]                      # last one = shared expert
    router = rng.normal(0, 0.5, (D, n_experts)).astype(np.float32)
    return experts, router


def _ffn(experts, e, rows):
    gate, up, down = experts[e]
    x = rows.astype(np.float64)
    hidden = (po.silu64(x @ gate.T) * (x @ up.T)).astype(np.float32).astype(np.float64)
    return hidden @ down.T


class NumpyEngine:
    """Same interface as DeviceExpertEngine; tensors are CPU torch tensors."""

    def __init__(self, experts, router, first, count, n_global):
        self.experts, self.router = experts, router
        self.first, self.count, self.n_global = first, count, n_global
        self.k_out = K + 1
        self.pad_id = n_global + 1          # padding entries of a partly filled slot: nobody executes them

    def route(self, x_all):
        x = x_all.float().numpy()
        logits = (x.astype(np.float64) @ self.router.astype(np.float64)).astype(np.float32)
        weights, ids = po.router_topk_rows_fp32(logits, K, FLOOR)
        t = x.shape[0]
        weights = np.concatenate([weights, np.ones((t, 1), np.float32)], axis=1)
        ids = np.concatenate([ids.astype(np.int64), np.full((t, 1), self.n_global, np.int64)], axis=1)
        return torch.from_numpy(weights), torch.from_numpy(ids)

    def local_terms(self, x_all, weights, ids, home_lo, home_hi, *, peer=None, total_rows=None):
        assert peer is None
        x, w, idn = x_all.float().numpy(), weights.numpy(), ids.numpy()
        terms = np.zeros((idn.size, D), np.float32)
        for row in range(idn.shape[0]):
            for slot in range(idn.shape[1]):
                g = int(idn[row, slot])
                mine = self.first <= g < self.first + self.count or (g == self.n_global and home_lo <= row < home_hi)
                if mine:
                    out = _ffn(self.experts, g, x[row:row + 1])[0].astype(np.float32)
                    terms[row * idn.shape[1] + slot] = (out * w[row, slot]).astype(np.float32)
        return torch.from_numpy(terms)

    def combine(self, terms_home, ids_home, x_home, out_dtype):
        terms, idn = terms_home.numpy(), ids_home.numpy()
        rows, k_out = idn.shape
        out = np.zeros((rows, D), np.float32)
        for row in range(rows):
            for slot in sorted(range(k_out), key=lambda s: (idn[row, s], s)):
                out[row] = (out[row] + terms[row * k_out + slot]).astype(np.float32)
        return torch.from_numpy(out).to(out_dtype)


def _single_process(experts, router, n_experts, x_all):
    engine = NumpyEngine(experts, router, 0, n_experts, n_experts)
    layer = ExpertParallelMoELayer(engine, LocalComm(), D)
    return layer.forward(torch.from_numpy(x_all)[None])[0].numpy()


def _inputs(world, rows, seed=3):
    return np.random.default_rng(seed).normal(0, 1, (world * rows, D)).astype(np.float32)


def test_world_of_one_matches_the_oracle_dispatch():
    n_experts = 6
    experts, router = _model(n_experts)
    x = _inputs(1, 5)
    got = _single_process(experts, router, n_experts, x)
    engine = NumpyEngine(experts, router, 0, n_experts, n_experts)
    weights, ids = engine.route(torch.from_numpy(x))
    want = po.experts_forward_fp32sum(x, weights.numpy(), ids.numpy(), lambda e, r: _ffn(experts, e, r),
                                      n_experts + 1)
    assert np.array_equal(got, want)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# experts, rows of (rank 0, rank 1), dtype; consecutive cases change the row count on purpose, and the
# unequal ones (a batch that does not divide by the ranks, a rank without rows) use padded slots
CASES = [(6, (3, 3), "float32"), (7, (1, 1), "float32"), (6, (4, 4), "bfloat16"), (6, (2, 1), "float32"),
         (7, (1, 0), "float32"), (6, (0, 3), "bfloat16"), (6, (3, 3), "float32")]


def _rank_main(rank, world, port, queue):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        comm = CollectiveComm()
        for case, (n_experts, counts, dtype_name) in enumerate(CASES):
            experts, router = _model(n_experts)
            first, count = expert_partition(n_experts, world)[rank]
            layer = ExpertParallelMoELayer(NumpyEngine(experts, router, first, count, n_experts), comm, D)
            x_all = torch.from_numpy(_inputs(1, sum(counts))).to(getattr(torch, dtype_name))
            lo = sum(counts[:rank])
            mine = x_all[lo:lo + counts[rank]].reshape(1, counts[rank], D)
            out = layer.forward(mine.contiguous(), slot_rows=max(counts))[0]
            queue.put((case, rank, out.float().numpy()))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_process_layer():
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world * len(CASES)):
            case, rank, out = queue.get(timeout=180)
            results[case, rank] = out
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
    assert all(p.exitcode == 0 for p in procs)
    for case, (n_experts, counts, dtype_name) in enumerate(CASES):
        experts, router = _model(n_experts)
        x_all = torch.from_numpy(_inputs(1, sum(counts))).to(getattr(torch, dtype_name)).float().numpy()
        want = _single_process(experts, router, n_experts, x_all)
        if dtype_name == "bfloat16":
            want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
        got = np.concatenate([results[case, r].reshape(-1, D) for r in range(world)], axis=0)
        assert got.shape == want.shape and np.array_equal(got, want), CASES[case]
