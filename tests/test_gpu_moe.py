"""GPU parity of the router / routing-plan / grouped-expert kernels against the oracle.

Tolerances are the reference's: router weights 2e-7 with exact ids
(tests/test_0106v_router_decode.py:37-38), grouped experts rtol 4e-4 / atol 8e-6
(tests/test_0106t_grouped_quantized_experts.py:172), MoE layer rtol 3e-5 / atol 2e-6 against
FP64 where stated (tests/test_0106o_qwen3next_decoder.py:192).
"""

import numpy as np
import pytest

from oracle import packed_oracle as po
from mylocal_llm_b200 import moe_ops
from mylocal_llm_b200.quantize import quantize

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["tensor", "staged", "lanes"])
def kernel_family(request, monkeypatch):
    """Run every case on all kernel families: "tensor" is the default selection (direct-load
    tensor-core kernel where it applies), "staged" the bulk-copy staged tensor-core kernel,
    "lanes" the FP32-lane kernel."""
    monkeypatch.setenv("B200Q_KERNEL", {"tensor": "auto", "staged": "staged", "lanes": "lanes"}[request.param])
    return request.param


def to_cuda(torch, a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


# ------------------------------------------------------------------------------------ router
def test_router_topk_matches_reference_golden(cuda, golden):
    logits, k = golden["router_logits"], int(golden["router_k"])
    w, ids = moe_ops.router_topk(to_cuda(cuda, logits), k, renormalize=False)
    np.testing.assert_array_equal(ids.cpu().numpy(), golden["router_ids"])
    np.testing.assert_allclose(w.cpu().numpy(), golden["router_w_raw"], rtol=0, atol=2e-7)


def test_router_projection_and_renormalisation_match_reference_golden(cuda, golden):
    k = int(golden["router_k"])
    logits = moe_ops.router_logits(to_cuda(cuda, golden["router_fw_x"]), to_cuda(cuda, golden["router_fw_W"]))
    ref_logits = golden["router_fw_x"].astype(np.float64) @ golden["router_fw_W"].astype(np.float64)
    np.testing.assert_allclose(logits.cpu().numpy(), ref_logits, rtol=1e-5, atol=1e-5)
    w, ids = moe_ops.router_topk(logits, k, renormalize=True, floor=2.0 ** -14)
    np.testing.assert_array_equal(ids.cpu().numpy(), golden["router_fw_ids"])
    np.testing.assert_allclose(w.cpu().numpy(), golden["router_fw_w"], rtol=0, atol=2e-7)


def test_router_ties_infinities_and_nans(cuda):
    rows = np.array([[1, 1, 1, 1], [0, np.inf, -np.inf, 5], [np.nan, 2, 2, 1], [3, np.nan, np.nan, 3]], np.float32)
    w, ids = moe_ops.router_topk(to_cuda(cuda, rows), 3, renormalize=True, floor=2.0 ** -14)
    np.testing.assert_array_equal(ids.cpu().numpy(), [[0, 1, 2], [1, 3, 0], [1, 2, 3], [0, 3, 1]])
    w_ref, ids_ref = po.router_topk_rows_fp32(rows, 3, 2.0 ** -14)
    got = w.cpu().numpy()
    np.testing.assert_array_equal(np.isnan(got), np.isnan(w_ref))
    np.testing.assert_allclose(np.nan_to_num(got), np.nan_to_num(w_ref), rtol=0, atol=2e-7)


@pytest.mark.parametrize("rows,n,k", [(1, 512, 10), (16, 512, 10), (256, 512, 10), (3, 4096, 32), (5, 7, 7)])
def test_router_topk_shapes_against_oracle(cuda, rows, n, k):
    logits = np.random.default_rng(rows + n).normal(0, 1.5, (rows, n)).astype(np.float32)
    w, ids = moe_ops.router_topk(to_cuda(cuda, logits), k, renormalize=True, floor=2.0 ** -14)
    w_ref, ids_ref = po.router_topk(logits, k, 2.0 ** -14)
    np.testing.assert_array_equal(ids.cpu().numpy(), ids_ref)
    np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=0, atol=2e-7)


# -------------------------------------------------------------------------------------- plan
# (7, 6, 4): more routes than experts, so rows repeat experts and the kernel takes its ordered pass;
# (600, 3, 4096): the per-expert row bitmasks would not fit in shared memory, ordered pass as well
@pytest.mark.parametrize("rows,k,e,dtype", [(1, 10, 512, "int64"), (11, 3, 9, "int64"), (256, 10, 512, "int32"),
                                            (700, 4, 33, "int64"), (5, 2, 4096, "int32"), (7, 6, 4, "int64"),
                                            (600, 3, 4096, "int32"), (2048, 11, 513, "int64")])
def test_routing_plan_is_the_stable_sort_by_expert(cuda, rows, k, e, dtype):
    rng = np.random.default_rng(rows * k + e)
    ids = np.stack([rng.choice(e, size=k, replace=k > e) for _ in range(rows)]).astype(dtype)
    plan = moe_ops.moe_plan(to_cuda(cuda, ids), e)
    order, counts, offsets = po.routing_plan(ids, e)
    np.testing.assert_array_equal(plan.counts.cpu().numpy(), counts)
    np.testing.assert_array_equal(plan.offsets.cpu().numpy(), offsets)
    np.testing.assert_array_equal(plan.order.cpu().numpy(), order)
    inv = np.empty_like(order)
    inv[order] = np.arange(order.size)
    np.testing.assert_array_equal(plan.inv.cpu().numpy(), inv)
    assert int(plan.status.item()) == 0
    nseg = int(plan.num_segments.item())
    seg_e = plan.seg_expert.cpu().numpy()[:nseg]
    seg_b = plan.seg_begin.cpu().numpy()[:nseg]
    seg_c = plan.seg_count.cpu().numpy()[:nseg]
    expect = [(ex, offsets[ex] + r, min(moe_ops.SEGMENT_CAP, counts[ex] - r))
              for ex in range(e) for r in range(0, counts[ex], moe_ops.SEGMENT_CAP)]
    assert [(int(a), int(b), int(c)) for a, b, c in zip(seg_e, seg_b, seg_c)] == expect


def test_routing_plan_skips_one_expert(cuda):
    rng = np.random.default_rng(3)
    rows, k, e, skip = 40, 3, 12, 5
    ids = np.stack([rng.choice(e, size=k, replace=False) for _ in range(rows)]).astype(np.int64)
    plan = moe_ops.moe_plan(to_cuda(cuda, ids), e, skip_expert=skip)
    order, counts, offsets = po.routing_plan(ids, e)
    np.testing.assert_array_equal(plan.counts.cpu().numpy(), counts)
    got_order = plan.order.cpu().numpy()
    lo, hi = offsets[skip], offsets[skip + 1]
    np.testing.assert_array_equal(got_order[:lo], order[:lo])                    # executed experts: stable order
    np.testing.assert_array_equal(got_order[hi:], order[hi:])
    assert sorted(got_order[lo:hi]) == sorted(order[lo:hi])                      # skipped: any order, all present
    nseg = int(plan.num_segments.item())
    assert skip not in plan.seg_expert.cpu().numpy()[:nseg].tolist()
    assert nseg == sum(-(-int(c) // moe_ops.SEGMENT_CAP) for ex, c in enumerate(counts) if ex != skip)


def test_routing_plan_flags_out_of_range_ids(cuda):
    ids = np.array([[0, 9], [2, 1]], np.int64)
    plan = moe_ops.moe_plan(to_cuda(cuda, ids), 4)
    assert int(plan.status.item()) == 1


def test_routing_plan_golden_counts(cuda, golden):
    plan = moe_ops.moe_plan(to_cuda(cuda, golden["plan_ids"]), 9)
    np.testing.assert_array_equal(plan.counts.cpu().numpy(), golden["plan_sizes"])
    np.testing.assert_array_equal(plan.offsets.cpu().numpy(), golden["plan_offsets"])
    sorted_experts = golden["plan_ids"].reshape(-1)[plan.order.cpu().numpy()]
    np.testing.assert_array_equal(sorted_experts, golden["plan_expert_sorted"])


# ----------------------------------------------------------------------------------- combine
def test_combine_adds_in_ascending_expert_order_without_fma_or_tree(cuda):
    # terms [1e8, 1, -1e8, 3] summed left to right give 3; any tree or reordering gives 4 or 0
    k, d = 4, 8
    ids = np.array([[3, 0, 2, 1]], np.int64)          # slot -> expert
    per_expert = {0: 1e8, 1: 1.0, 2: -1e8, 3: 3.0}
    plan = moe_ops.moe_plan(to_cuda(cuda, ids), 4)
    terms = np.zeros((k, d), np.float32)
    for pos, flat in enumerate(plan.order.cpu().numpy()):
        terms[pos] = per_expert[int(ids[0, flat])]
    out = moe_ops.moe_combine(to_cuda(cuda, terms), plan, d).cpu().numpy()
    np.testing.assert_array_equal(out, np.full((1, d), 3.0, np.float32))


# -------------------------------------------------------------------------- grouped experts
def run_routed(torch, hidden, weights, ids, gate_bank, up_bank, down_bank, d, f, e, fmts, x_dtype=None):
    x = to_cuda(torch, hidden, x_dtype)
    plan = moe_ops.moe_plan(to_cuda(torch, ids), e)
    gs, us, ds = (bank.shape[1] for bank in (gate_bank, up_bank, down_bank))
    gb, ub, db = (to_cuda(torch, bank.reshape(-1)) for bank in (gate_bank, up_bank, down_bank))
    hbuf = moe_ops.moe_gate_up(x, plan, gb, ub, fmts[0], fmts[1], f, d, gs, us)
    terms = moe_ops.moe_down(hbuf, to_cuda(torch, weights.astype(np.float32)), plan, db, fmts[2], d, f, ds)
    return moe_ops.moe_combine(terms, plan, d)


@pytest.mark.parametrize("tag", ["moe", "moe1"])
def test_grouped_experts_match_reference_golden(cuda, golden, tag):
    d, f, e, k = (int(v) for v in golden["moe_dims"])
    out = run_routed(cuda, golden[f"{tag}_hidden"], golden[f"{tag}_weights"], golden[f"{tag}_ids"],
                     golden["moe_gate_bytes"], golden["moe_up_bytes"], golden["moe_down_bytes"], d, f, e,
                     ("Q4_K", "Q4_K", "Q6_K"))
    np.testing.assert_allclose(out.cpu().numpy(), golden[f"{tag}_routed"], rtol=4e-4, atol=8e-6)


@pytest.mark.parametrize("tokens", [1, 16, 40])
def test_grouped_experts_against_fp64_oracle_with_crowded_experts(cuda, tokens):
    # few experts and many tokens: segments longer than the per-pass cap, repeated experts per pass
    d, f, e, k = 512, 256, 5, 2
    rng = np.random.default_rng(tokens)
    packs = [[quantize(rng.normal(0, 0.05, s).astype(np.float32), q) for _ in range(e)]
             for s, q in (((f, d), "Q4_K"), ((f, d), "Q5_K"), ((d, f), "Q6_K"))]
    banks = [np.stack([p.data for p in group]) for group in packs]
    hidden = rng.normal(0, 1, (tokens, d)).astype(np.float32)
    logits = rng.normal(0, 1, (tokens, e))
    w, ids = po.router_topk(logits, k, 2.0 ** -14)
    out = run_routed(cuda, hidden, w.astype(np.float32), ids, *banks, d, f, e, ("Q4_K", "Q5_K", "Q6_K"))
    experts = [tuple((packs[j][i].data, packs[j][i].shape, q) for j, q in enumerate(("Q4_K", "Q5_K", "Q6_K")))
               for i in range(e)]
    ref = po.experts_forward_fp32sum(hidden, w.astype(np.float32), ids,
                                     lambda ex, rows: po.expert_ffn_fp64(rows, *experts[ex]), e)
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=4e-4, atol=8e-6)


@pytest.mark.parametrize("fmt,x_dtype", [("Q4_K", "bfloat16"), ("Q4_K", "float32"), ("Q5_K", "float16"),
                                         ("Q4_K_TILED", "bfloat16"), ("Q4_K_TILED", "float32")])
@pytest.mark.parametrize("tokens,e,k", [(40, 5, 2), (64, 96, 6), (9, 33, 4)])
def test_gate_up_with_token_images_is_bit_identical(cuda, kernel_family, fmt, x_dtype, tokens, e, k):
    # the images are what the kernel would have prepared per token: same bits with them, without them, and
    # when the caller makes them once and passes them in; crowded experts give segments of 8 and re-used tokens
    from mylocal_llm_b200.quantized_linear import retile_bytes
    if kernel_family != "tensor":
        pytest.skip("only the direct-load kernel gathers images; the other families ignore the buffer")
    d, f = 768, 64
    base = "Q4_K" if fmt == "Q4_K_TILED" else fmt
    rng = np.random.default_rng(tokens + e)
    packs = [[quantize(rng.normal(0, 0.05, (f, d)).astype(np.float32), base) for _ in range(e)] for _ in range(2)]
    banks = [to_cuda(cuda, np.stack([p.data for p in group]).reshape(-1)) for group in packs]
    stride = packs[0][0].data.size
    if fmt == "Q4_K_TILED":
        banks = [retile_bytes(b, e * f, d, "Q4_K") for b in banks]
    x = to_cuda(cuda, rng.normal(0, 1, (tokens, d)).astype(np.float32), getattr(cuda, x_dtype))
    _, ids = po.router_topk(rng.normal(0, 1, (tokens, e)), k, 2.0 ** -14)
    plan = moe_ops.moe_plan(to_cuda(cuda, ids), e)
    run = lambda **kw: moe_ops.moe_gate_up(x, plan, banks[0], banks[1], fmt, fmt, f, d, stride, stride, **kw)
    import os
    os.environ["B200Q_TOKEN_IMAGES"] = "0"
    try:
        plain = run()
    finally:
        del os.environ["B200Q_TOKEN_IMAGES"]
    images = moe_ops.token_images(x)
    assert images is not None and images.shape[0] == tokens
    assert cuda.equal(run(), plain)
    assert cuda.equal(run(images=images), plain)
