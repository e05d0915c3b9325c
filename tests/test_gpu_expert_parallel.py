"""Expert-parallel MoE on the GPU: whatever the number of ranks, the result must be the single-GPU
layer's, bit for bit.

One GPU is enough for most of it: the ranks' device steps run one after the other on the same GPU
(no kernel waits on another rank there), and the exchange is done by hand. The real two-process runs
(NCCL collectives, and peer-memory stores with the device barrier) need two GPUs and are skipped
otherwise.
"""

import os
import socket

import numpy as np
import pytest

from mylocal_llm_b200 import PackedMoELayer, packed_to_device
from mylocal_llm_b200 import _lib
from mylocal_llm_b200.expert_parallel import (CollectiveComm, DeviceExpertEngine, ExpertParallelMoELayer, LocalComm,
                                              PeerComm, expert_partition, shard_bank)
from mylocal_llm_b200.experts_inference import synthetic_bank
from mylocal_llm_b200.quantize import random_packed

pytestmark = pytest.mark.gpu

D, F, E, K = 512, 256, 16, 4
TYPES = ("Q4_K", "Q4_K", "Q6_K")


@pytest.fixture(autouse=True, params=["tensor", "lanes"])
def kernel_family(request, monkeypatch):
    monkeypatch.setenv("B200Q_KERNEL", {"tensor": "auto", "lanes": "lanes"}[request.param])
    monkeypatch.setenv("B200Q_RETILE", "1" if request.param == "tensor" else "0")
    return request.param


def build_model(torch, *, shared_ff=F, with_gate=False, seed=0):
    bank = synthetic_bank(E, D, F, TYPES, seed=seed)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(100 + seed)
    w_router = torch.empty((D, E), dtype=torch.float32, device="cuda").normal_(0.0, 0.3, generator=gen)
    shared = None
    if shared_ff:
        shapes = ((shared_ff, D), (shared_ff, D), (D, shared_ff))
        shared = tuple(packed_to_device(random_packed(fmt, shape, seed=50 + seed + j, d=1.0 / 2048, dmin=1.0 / 4096))
                       for j, (fmt, shape) in enumerate(zip(TYPES, shapes)))
    gate = None
    if with_gate:
        gate = torch.empty(D, dtype=torch.float32, device="cuda").normal_(0.0, 0.1, generator=gen)
    return bank, w_router, shared, gate


def make_rows(torch, rows, dtype, seed=1):
    x = np.random.default_rng(seed).normal(0, 1, (rows, D)).astype(np.float32)
    return torch.from_numpy(x).cuda().to(dtype)


def engines_for(world, bank, w_router, shared, gate):
    out = []
    for rank in range(world):
        first, local = shard_bank(bank, rank, world)
        out.append(DeviceExpertEngine(local, w_router, K, first_expert=first, n_experts_global=E, shared=shared,
                                      shared_gate=gate))
    return out


@pytest.mark.parametrize("world,rows", [(1, 5), (2, 1), (2, 16), (4, 3)])
@pytest.mark.parametrize("variant", ["folded", "folded_gate", "separate_shared", "no_shared"])
def test_emulated_ranks_with_summed_terms_equal_the_single_gpu_layer(cuda, world, rows, variant):
    torch = cuda
    bank, w_router, shared, gate = build_model(
        torch, shared_ff={"separate_shared": 512, "no_shared": 0}.get(variant, F), with_gate=variant == "folded_gate")
    if variant == "separate_shared":
        gate = torch.full((D,), 0.01, dtype=torch.float32, device="cuda")
    x_all = make_rows(torch, world * rows, torch.bfloat16)
    want = PackedMoELayer(bank, w_router, K, shared=shared, shared_gate=gate).forward(x_all[None])[0]
    engines = engines_for(world, bank, w_router, shared, gate)
    weights, ids = engines[0].route(x_all)
    total = None
    for rank, engine in enumerate(engines):
        w_r, ids_r = engine.route(x_all)
        assert torch.equal(ids_r, ids) and torch.equal(w_r, weights)
        terms = engine.local_terms(x_all, weights, ids, rank * rows, (rank + 1) * rows)
        if total is not None:                       # every row has exactly one producer
            assert not bool(((total != 0) & (terms != 0)).any())
        total = terms if total is None else total + terms
    k_out = engines[0].k_out
    got = []
    for rank, engine in enumerate(engines):
        lo, hi = rank * rows, (rank + 1) * rows
        got.append(engine.combine(total[lo * k_out:hi * k_out], ids[lo:hi].contiguous(), x_all[lo:hi],
                                  torch.bfloat16))
    assert torch.equal(torch.cat(got), want)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("world,rows", [(2, 4), (4, 1)])
def test_emulated_ranks_storing_into_home_buffers_equal_the_single_gpu_layer(cuda, world, rows):
    torch = cuda
    bank, w_router, shared, gate = build_model(torch, with_gate=True, seed=3)
    x_all = make_rows(torch, world * rows, torch.float32, seed=4)
    want = PackedMoELayer(bank, w_router, K, shared=shared, shared_gate=gate).forward(x_all[None])[0]
    engines = engines_for(world, bank, w_router, shared, gate)
    k_out = engines[0].k_out
    homes = [torch.full((rows * k_out, D), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
    table = torch.tensor([h.data_ptr() for h in homes], dtype=torch.int64, device="cuda")
    weights, ids = engines[0].route(x_all)
    for rank, engine in enumerate(engines):
        engine.local_terms(x_all, weights, ids, rank * rows, (rank + 1) * rows, peer=(table, rows * k_out))
    got = []
    for rank, engine in enumerate(engines):
        assert not bool(torch.isnan(homes[rank]).any())        # every term row was written by someone
        lo, hi = rank * rows, (rank + 1) * rows
        got.append(engine.combine(homes[rank], ids[lo:hi].contiguous(), x_all[lo:hi], torch.float32))
    assert torch.equal(torch.cat(got), want)
    assert _lib.device_status() == 0


def test_plan_ep_reports_ids_outside_the_global_range(cuda):
    from mylocal_llm_b200 import moe_ops
    ids = cuda.tensor([[0, 3], [18, 1]], dtype=cuda.int64, device="cuda")
    plan = moe_ops.moe_plan_ep(ids, e_global=17, first_expert=0, n_local=8, shared_id=16, home_lo=0, home_hi=2)
    assert int(plan.status.item()) == 1
    plan = moe_ops.moe_plan_ep(ids.clamp(max=16), e_global=17, first_expert=0, n_local=8, shared_id=16, home_lo=0,
                               home_hi=1)
    assert int(plan.status.item()) == 0
    # rows: [0, 3] local; [16 -> not home (row 1) -> skipped, 1 local]
    assert plan.counts.cpu().tolist() == [1, 1, 0, 1, 0, 0, 0, 0, 0, 1]
    # the id e_global marks padding entries of a partly filled slot: legal, never executed, even on the home rank
    padded = cuda.tensor([[2, 16], [17, 17]], dtype=cuda.int64, device="cuda")
    plan = moe_ops.moe_plan_ep(padded, e_global=17, first_expert=0, n_local=8, shared_id=16, home_lo=0, home_hi=2)
    assert int(plan.status.item()) == 0
    assert plan.counts.cpu().tolist() == [0, 0, 1, 0, 0, 0, 0, 0, 1, 2]
    assert int(plan.num_segments.item()) == 2
    with pytest.raises(ValueError):
        moe_ops.moe_plan_ep(ids, e_global=4, first_expert=0, n_local=8, shared_id=-1, home_lo=0, home_hi=2)


@pytest.mark.parametrize("world,row_counts", [(2, (2, 1)), (4, (1, 0, 0, 0)), (4, (3, 3, 2, 2))])
@pytest.mark.parametrize("variant", ["folded_gate", "no_shared"])
def test_emulated_ranks_with_partly_filled_slots_equal_the_single_gpu_layer(cuda, world, row_counts, variant):
    """A batch that does not divide by the number of ranks: every rank reserves the same slot, ranks with
    fewer rows (or none) pad theirs with entries nobody executes."""
    torch = cuda
    bank, w_router, shared, gate = build_model(torch, shared_ff={"no_shared": 0}.get(variant, F),
                                               with_gate=variant == "folded_gate", seed=5)
    total_rows, slot = sum(row_counts), max(row_counts)
    x_real = make_rows(torch, total_rows, torch.bfloat16, seed=9)
    want = PackedMoELayer(bank, w_router, K, shared=shared, shared_gate=gate).forward(x_real[None])[0]
    engines = engines_for(world, bank, w_router, shared, gate)
    k_out = engines[0].k_out
    starts = np.concatenate(([0], np.cumsum(row_counts)))
    slots, routed = [], []
    for rank, engine in enumerate(engines):
        x_home = x_real[starts[rank]:starts[rank + 1]]
        layer = ExpertParallelMoELayer(engine, LocalComm(), D)
        w_r = ids_r = None
        if row_counts[rank]:
            w_r, ids_r = engine.route(x_home)
        routed.append((x_home, ids_r))
        slots.append(layer._fill_slot(x_home, w_r, ids_r, row_counts[rank], slot))
    x_all, w_all, ids_all = (torch.cat([s[j] for s in slots]) for j in range(3))
    total = None
    for rank, engine in enumerate(engines):
        terms = engine.local_terms(x_all, w_all, ids_all, rank * slot, rank * slot + row_counts[rank],
                                   total_rows=total_rows)
        if total is not None:
            assert not bool(((total != 0) & (terms != 0)).any())
        total = terms if total is None else total + terms
    got = []
    for rank, engine in enumerate(engines):
        x_home, ids_r = routed[rank]
        if row_counts[rank]:
            lo = rank * slot * k_out
            got.append(engine.combine(total[lo:lo + row_counts[rank] * k_out], ids_r, x_home, torch.bfloat16))
    assert torch.equal(torch.cat(got), want)
    assert _lib.device_status() == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_peer_comm_in_a_world_of_one(cuda):
    """Arena allocation, push, barrier and peer-table stores with a single rank (nothing to wait for)."""
    import torch.distributed as dist
    torch = cuda
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{_free_port()}", rank=0, world_size=1)
    try:
        bank, w_router, shared, gate = build_model(torch, seed=6)
        comm = PeerComm(None, max_rows=8, d_model=D, k_out=K + 1)
        layer = ExpertParallelMoELayer(DeviceExpertEngine(bank, w_router, K, first_expert=0, n_experts_global=E,
                                                          shared=shared), comm, D)
        for rows in (8, 2):
            x = make_rows(torch, rows, torch.bfloat16, seed=rows)
            want = PackedMoELayer(bank, w_router, K, shared=shared).forward(x[None])
            assert torch.equal(layer.forward(x[None]), want)
        with pytest.raises(ValueError):
            layer.forward(make_rows(torch, 9, torch.bfloat16)[None])
        assert _lib.device_status() == 0
        comm.close()
    finally:
        dist.destroy_process_group()


def test_barrier_gives_up_after_its_limit_and_reports_it(cuda):
    """A peer that never arrives: the barrier returns after its time limit with status 201, the
    context stays usable, and the host can clear the word. (The absent peer is a second pad on the
    same GPU that nothing ever signals - no second kernel is involved.)"""
    import ctypes
    import time
    torch = cuda
    assert _lib.device_status() == 0
    pads = torch.zeros(2, 64, dtype=torch.int32, device="cuda")            # two signal pads of 256 bytes
    table = torch.tensor([pads[0].data_ptr(), pads[1].data_ptr()], dtype=torch.int64, device="cuda")
    t0 = time.perf_counter()
    _lib.call("b200q_peer_barrier", ctypes.c_void_p(table.data_ptr()), 0, 2, 50, _lib.current_stream())
    assert _lib.device_status() == 201
    assert time.perf_counter() - t0 < 5.0
    assert int(pads[1, 0].item()) == 1                                     # rank 0 did signal its peer
    _lib.clear_device_status()
    assert _lib.device_status() == 0
    # the context is intact: a normal kernel still runs
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
    with pytest.raises(ValueError):
        _lib.call("b200q_peer_barrier", ctypes.c_void_p(table.data_ptr()), 2, 2, 50, _lib.current_stream())


def test_local_comm_layer_equals_packed_layer(cuda):
    torch = cuda
    bank, w_router, shared, gate = build_model(torch, with_gate=True, seed=8)
    layer = ExpertParallelMoELayer(DeviceExpertEngine(bank, w_router, K, first_expert=0, n_experts_global=E,
                                                      shared=shared, shared_gate=gate), LocalComm(), D)
    x = make_rows(torch, 7, torch.float32)[None]
    assert torch.equal(layer.forward(x), PackedMoELayer(bank, w_router, K, shared=shared, shared_gate=gate).forward(x))


# ---------------------------------------------------------------------------- two real processes
def _rank_main(rank, world, port, family, queue):
    import torch
    import torch.distributed as dist
    os.environ["B200Q_KERNEL"] = family
    os.environ["B200Q_RETILE"] = "1" if family == "auto" else "0"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    ok, note = True, ""
    try:
        bank, w_router, shared, gate = build_model(torch, with_gate=True, seed=11)
        first, local = shard_bank(bank, rank, world)
        engine = DeviceExpertEngine(local, w_router, K, first_expert=first, n_experts_global=E, shared=shared,
                                    shared_gate=gate)
        reference = PackedMoELayer(bank, w_router, K, shared=shared, shared_gate=gate)
        comms = [("collective", CollectiveComm()), ("peer", PeerComm(None, max_rows=16, d_model=D, k_out=K + 1))]
        for name, comm in comms:
            layer = ExpertParallelMoELayer(engine, comm, D)
            for rows, dtype in ((16, torch.bfloat16), (1, torch.float32), (5, torch.bfloat16)):
                x_all = make_rows(torch, world * rows, dtype, seed=rows)
                want = reference.forward(x_all[None])[0][rank * rows:(rank + 1) * rows]
                for _ in range(3):                                    # repeated calls reuse the arenas
                    got = layer.forward(x_all[rank * rows:(rank + 1) * rows][None].contiguous())[0]
                    if not torch.equal(got, want):
                        ok, note = False, f"{name} rows={rows} differs"
            # batches that do not divide by the number of ranks: (rows of rank 0, rows of rank 1), one slot size
            for counts in ((2, 1), (1, 0), (5, 5), (0, 3)):
                slot = max(counts)
                x_real = make_rows(torch, sum(counts), torch.bfloat16, seed=40 + sum(counts))
                lo = sum(counts[:rank])
                mine = x_real[lo:lo + counts[rank]]
                want = reference.forward(x_real[None])[0][lo:lo + counts[rank]]
                for _ in range(2):
                    got = layer.forward(mine.reshape(1, counts[rank], D).contiguous(), slot_rows=slot,
                                        total_rows=sum(counts))[0]
                    if tuple(got.shape) != (counts[rank], D) or not torch.equal(got, want):
                        ok, note = False, f"{name} row counts {counts} differ"
            torch.cuda.synchronize()
            comm.close()
        if _lib.device_status() != 0:
            ok, note = False, f"device status {_lib.device_status()}"
    except Exception as exc:                                          # reported to the parent
        ok, note = False, repr(exc)
    finally:
        queue.put((rank, ok, note))
        dist.destroy_process_group()


def test_two_gpus_collective_and_peer_exchange(cuda, kernel_family):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    family = {"tensor": "auto", "lanes": "lanes"}[kernel_family]
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, family, queue)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as queue_module
    results = []
    try:
        for _ in range(world):
            results.append(queue.get(timeout=300))
    except queue_module.Empty:
        pass                                   # a rank died or blocked: reported below, children ended in `finally`
    finally:
        for p in procs:
            p.join(timeout=60 if len(results) == world else 5)
        for p in procs:
            if p.is_alive():                   # never leave a child holding a GPU of a shared machine
                p.terminate()
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()
    assert len(results) == world, f"only {len(results)} of {world} ranks reported: {results}"
    assert all(ok for _, ok, _ in results), results
