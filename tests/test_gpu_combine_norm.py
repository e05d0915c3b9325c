"""Ordered combine fused with the residual add and RMSNorm that follow a MoE layer.

``b200q_moe_combine_norm`` has to return the bits of ``b200q_moe_combine`` followed by
``b200q_residual_rmsnorm`` (the reference's ``_ordered_reduce`` /
``RMSNormInference.forward_residual_add`` pair, mini_llm/ops/grouped_quantized_experts.py:70-79 and
mini_llm/ops/rmsnorm_inference.py:228-252), for every branch dtype, with and without the
shared-expert term, and through the layer and stack front ends.
"""

import numpy as np
import pytest

from mylocal_llm_b200 import moe_ops
from mylocal_llm_b200.moe_layer import RMSNormInference
from mylocal_llm_b200.moe_stack import PackedMoEStack

pytestmark = pytest.mark.gpu


def make_norm(torch, d, dtype, seed):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    norm = RMSNormInference(d, eps=1e-5)
    norm.set_weights((1.0 + 0.1 * torch.randn(d, device="cuda", generator=gen)).to(dtype))
    return norm


@pytest.mark.parametrize("rows,k,d", [(1, 11, 2048), (5, 4, 512), (64, 11, 2048), (3, 16, 768), (7, 1, 300)])
@pytest.mark.parametrize("branch_dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("with_extra", [False, True])
def test_fused_combine_norm_equals_the_two_kernels(cuda, rows, k, d, branch_dtype, with_extra):
    torch = cuda
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rows * 131 + k * 7 + d)
    e = max(k, 24)
    ids = torch.stack([torch.randperm(e, device="cuda", generator=gen)[:k] for _ in range(rows)]).to(torch.int64)
    plan = moe_ops.moe_plan(ids.contiguous(), e)
    terms = torch.randn((rows * k, d), device="cuda", generator=gen) * 0.3
    residual = torch.randn((rows, d), device="cuda", generator=gen)
    extra = torch.randn((rows, d), device="cuda", generator=gen) if with_extra else None
    extra_scale = torch.rand(rows, device="cuda", generator=gen) if with_extra else None
    bdt = getattr(torch, branch_dtype)
    norm = make_norm(torch, d, torch.bfloat16 if branch_dtype != "float32" else torch.float32, seed=k)
    branch = moe_ops.moe_combine(terms, plan, d, extra=extra, extra_scale=extra_scale, out_dtype=bdt)
    res_ref, y_ref = norm.forward_residual_add(residual, branch)
    res, y = moe_ops.moe_combine_norm(terms, plan, d, norm, residual, extra=extra, extra_scale=extra_scale,
                                      branch_dtype=bdt)
    assert torch.equal(res, res_ref)
    assert torch.equal(y, y_ref)
    assert y.dtype == norm.gamma.dtype and res.dtype == torch.float32


def test_fused_combine_norm_rejects_what_it_cannot_do(cuda):
    torch = cuda
    ids = torch.arange(17, device="cuda", dtype=torch.int64).reshape(1, 17)
    plan = moe_ops.moe_plan(ids, 32)
    norm = make_norm(torch, 256, torch.float32, seed=1)
    terms = torch.zeros((17, 256), device="cuda")
    with pytest.raises(NotImplementedError):
        moe_ops.moe_combine_norm(terms, plan, 256, norm, torch.zeros((1, 256), device="cuda"))
    plan4 = moe_ops.moe_plan(ids[:, :4].contiguous(), 32)
    with pytest.raises(ValueError):
        moe_ops.moe_combine_norm(terms[:4], plan4, 256, norm, torch.zeros((1, 256), device="cuda", dtype=torch.float16))


@pytest.mark.parametrize("tokens", [1, 6, 40])
@pytest.mark.parametrize("act", ["bfloat16", "float32"])
def test_stack_with_and_without_the_fused_epilogue(cuda, tokens, act):
    torch = cuda
    stack = PackedMoEStack.synthetic(3, d_model=512, d_ff=256, n_experts=32, top_k=4, shared_d_ff=256, seed=5,
                                     act_dtype=getattr(torch, act))
    assert all(layer.can_fuse_residual_norm() for layer in stack.layers)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(tokens)
    x = torch.randn((1, tokens, 512), device="cuda", generator=gen)
    stack.fuse_residual_norm = False
    res_ref, hid_ref = stack.forward(x)
    stack.fuse_residual_norm = True
    res, hid = stack.forward(x)
    assert torch.equal(res, res_ref) and torch.equal(hid, hid_ref)
    assert bool(torch.isfinite(res).all())


def test_layer_front_end_checks_the_residual(cuda):
    torch = cuda
    stack = PackedMoEStack.synthetic(1, d_model=512, d_ff=256, n_experts=32, top_k=4, shared_d_ff=256, seed=2)
    layer, norm = stack.layers[0], stack.final_norm
    hidden = torch.randn((1, 3, 512), device="cuda").to(torch.bfloat16)
    with pytest.raises(ValueError):
        layer.forward(hidden, residual_norm=(norm, torch.zeros((1, 2, 512), device="cuda")))
    res, y = layer.forward(hidden, residual_norm=(norm, torch.zeros((1, 3, 512), device="cuda")))
    ref = norm.forward_residual_add(torch.zeros((1, 3, 512), device="cuda"), layer.forward(hidden))
    assert torch.equal(res, ref[0]) and torch.equal(y, ref[1])
