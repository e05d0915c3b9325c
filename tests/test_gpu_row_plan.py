"""Top-k and routing plan of a single token row in one launch (``b200q_router_topk_plan_row``).

For one row the plan is a sort of k distinct expert ids, so the one-token decode step lets the
top-k kernel write it. Weights, ids and every plan array have to equal what ``b200q_router_topk_ex``
followed by ``b200q_moe_plan`` produce (``RoutingPlan.from_router_outputs``,
mini_llm/ops/routing_plan.py:52-118 of the reference), and a layer has to return the same bits
either way.
"""

import pytest

from mylocal_llm_b200 import moe_ops
from mylocal_llm_b200.moe_stack import PackedMoEStack

pytestmark = pytest.mark.gpu

PLAN_FIELDS = ("counts", "offsets", "order", "inv", "num_segments", "status")


@pytest.mark.parametrize("n,k,extra", [(512, 10, True), (512, 10, False), (64, 8, True), (33, 31, True), (8, 1, False),
                                       (1024, 4, True)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_row_plan_equals_topk_then_plan(cuda, n, k, extra, seed):
    torch = cuda
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed * 7919 + n + k)
    logits = torch.randn((1, n), device="cuda", generator=gen) * 3
    if seed == 2:
        logits[0, :: max(1, n // 7)] = logits[0, 0]                    # ties: the lower id wins
    extra_id = n if extra else -1
    scale = torch.rand(1, device="cuda", generator=gen) if extra else None
    e_plan = n + (1 if extra else 0)
    w_ref, i_ref = moe_ops.router_topk(logits, k, renormalize=True, extra_id=extra_id, extra_weight=scale)
    plan_ref = moe_ops.moe_plan(i_ref, e_plan)
    w, i, plan = moe_ops.router_topk_plan_row(logits, k, e_plan, renormalize=True, extra_id=extra_id, extra_weight=scale)
    assert torch.equal(w, w_ref) and torch.equal(i, i_ref)
    assert (plan.rows, plan.k, plan.n_experts, plan.max_segments) == (plan_ref.rows, plan_ref.k, plan_ref.n_experts,
                                                                      plan_ref.max_segments)
    for name in PLAN_FIELDS:
        assert torch.equal(getattr(plan, name), getattr(plan_ref, name)), name
    segs = int(plan_ref.num_segments.item())
    assert segs == plan.k
    for name in ("seg_expert", "seg_begin", "seg_count"):
        assert torch.equal(getattr(plan, name)[:segs], getattr(plan_ref, name)[:segs]), name


def test_row_plan_rejects_what_it_cannot_do(cuda):
    torch = cuda
    with pytest.raises(ValueError):
        moe_ops.router_topk_plan_row(torch.zeros((2, 64), device="cuda"), 4, 64)
    with pytest.raises(ValueError):          # the plan must cover the appended id
        moe_ops.router_topk_plan_row(torch.zeros((1, 64), device="cuda"), 4, 64, extra_id=64)
    with pytest.raises(ValueError):          # an appended id inside the routed range would not be distinct
        moe_ops.router_topk_plan_row(torch.zeros((1, 64), device="cuda"), 4, 65, extra_id=3)


@pytest.mark.parametrize("act", ["bfloat16", "float32"])
def test_one_token_stack_is_identical_with_and_without_the_fused_plan(cuda, act):
    torch = cuda
    stack = PackedMoEStack.synthetic(3, d_model=512, d_ff=256, n_experts=32, top_k=4, shared_d_ff=256, seed=9,
                                     act_dtype=getattr(torch, act))
    x = torch.randn((1, 1, 512), device="cuda")
    for layer in stack.layers:
        layer.fuse_row_plan = False
    res_ref, hid_ref = stack.forward(x)
    for layer in stack.layers:
        layer.fuse_row_plan = True
    res, hid = stack.forward(x)
    assert torch.equal(res, res_ref) and torch.equal(hid, hid_ref)
