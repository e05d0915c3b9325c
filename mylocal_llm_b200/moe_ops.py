"""Thin torch-tensor wrappers over the MoE entry points of the C ABI.

Each function allocates its outputs with torch, passes raw pointers to ``libb200q.so`` and
returns torch tensors; all work is enqueued on torch's current stream and nothing here
synchronises or reads device memory back.
"""

import os
import ctypes
from dataclasses import dataclass

from . import _lib

SEGMENT_CAP = 8  # tokens of one expert handled per pass of the grouped kernels


def _torch():
    import torch
    return torch


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _dtype_id(t):
    name = str(t.dtype).replace("torch.", "")
    if name not in _lib.DTYPE_ID:
        raise TypeError("activations must be FP16, BF16 or FP32")
    return _lib.DTYPE_ID[name]


def router_logits(x2d, w_router, bias=None):
    """FP32 ``x[T,D] @ W[D,E] (+ bias)``; W and bias are FP32 device tensors."""
    torch = _torch()
    t, d = x2d.shape
    e = w_router.shape[1]
    if w_router.dtype != torch.float32 or not w_router.is_contiguous() or w_router.shape[0] != d:
        raise ValueError("router weight must be a contiguous FP32 [D, E] tensor")
    out = torch.empty((t, e), dtype=torch.float32, device=x2d.device)
    _lib.call("b200q_router_logits", _ptr(x2d), _dtype_id(x2d), t, d, _ptr(w_router), _ptr(bias), e, _ptr(out),
              _lib.current_stream())
    return out


def router_logits_t(x2d, w_router_t, bias=None):
    """FP32 ``x[T,D] @ Wt[E,D].T (+ bias)`` for a router weight stored expert-major."""
    torch = _torch()
    t, d = x2d.shape
    e = w_router_t.shape[0]
    if w_router_t.dtype != torch.float32 or not w_router_t.is_contiguous() or w_router_t.shape[1] != d:
        raise ValueError("router weight must be a contiguous FP32 [E, D] tensor")
    out = torch.empty((t, e), dtype=torch.float32, device=x2d.device)
    _lib.call("b200q_router_logits_t", _ptr(x2d), _dtype_id(x2d), t, d, _ptr(w_router_t), _ptr(bias), e, _ptr(out),
              _lib.current_stream())
    return out


def router_topk(logits2d, k, *, renormalize, floor=1e-30, extra_id=-1, extra_weight=None):
    """(FP32 weights [T,k'], int64 ids [T,k']) from FP32 logits [T,E].

    With ``extra_id >= 0`` one more assignment (that id, weight ``extra_weight[t]`` or 1) is appended
    to every row, so k' = k + 1."""
    torch = _torch()
    if logits2d.dtype != torch.float32 or not logits2d.is_contiguous():
        raise ValueError("logits must be a contiguous FP32 tensor")
    t, e = logits2d.shape
    k_out = int(k) + (1 if extra_id >= 0 else 0)
    weights = torch.empty((t, k_out), dtype=torch.float32, device=logits2d.device)
    ids = torch.empty((t, k_out), dtype=torch.int64, device=logits2d.device)
    _lib.call("b200q_router_topk_ex", _ptr(logits2d), t, e, int(k), 1 if renormalize else 0, float(floor),
              int(extra_id), _ptr(extra_weight), _ptr(weights), _ptr(ids), _lib.current_stream())
    return weights, ids


def shared_gate(x2d, gate_vec):
    """sigmoid(x[T,D] . g[D]) as FP32 [T]."""
    torch = _torch()
    t, d = x2d.shape
    out = torch.empty((t,), dtype=torch.float32, device=x2d.device)
    _lib.call("b200q_shared_gate", _ptr(x2d), _dtype_id(x2d), t, d, _ptr(gate_vec), _ptr(out),
              _lib.current_stream())
    return out


@dataclass
class DeviceRoutingPlan:
    """Device-resident routing plan (all int32 CUDA tensors); see ``b200q_moe_plan``."""

    rows: int
    k: int
    n_experts: int
    counts: object
    offsets: object
    order: object
    inv: object
    seg_expert: object
    seg_begin: object
    seg_count: object
    num_segments: object
    max_segments: int
    status: object


def max_segments_for(rows, k, n_experts, seg_cap=SEGMENT_CAP):
    total = rows * k
    return min(n_experts, total) + total // seg_cap


def moe_plan(ids, n_experts, *, skip_expert=-1):
    """Build the device routing plan for integer ids ``[T,k]`` (int32 or int64).

    Assignments to ``skip_expert`` are sorted and counted but never executed."""
    torch = _torch()
    if ids.dtype not in (torch.int32, torch.int64) or not ids.is_contiguous():
        raise ValueError("expert ids must be a contiguous int32/int64 tensor")
    rows, k = ids.shape
    total = rows * k
    max_seg = max_segments_for(rows, k, n_experts)
    i32 = dict(dtype=torch.int32, device=ids.device)
    plan = DeviceRoutingPlan(
        rows, k, n_experts,
        torch.empty(n_experts, **i32), torch.empty(n_experts + 1, **i32), torch.empty(total, **i32),
        torch.empty(total, **i32), torch.empty(max_seg, **i32), torch.empty(max_seg, **i32),
        torch.empty(max_seg, **i32), torch.empty(1, **i32), max_seg, torch.empty(1, **i32))
    _lib.call("b200q_moe_plan_ex", _ptr(ids), 1 if ids.dtype == torch.int64 else 0, rows, k, n_experts,
              int(skip_expert), SEGMENT_CAP,
              _ptr(plan.counts), _ptr(plan.offsets), _ptr(plan.order), _ptr(plan.inv), _ptr(plan.seg_expert),
              _ptr(plan.seg_begin), _ptr(plan.seg_count), _ptr(plan.num_segments), max_seg, _ptr(plan.status),
              _lib.current_stream())
    return plan


def router_topk_plan_row(logits2d, k, n_experts, *, renormalize=True, floor=2.0 ** -14, extra_id=-1, extra_weight=None):
    """``router_topk`` and ``moe_plan`` of a single token row in one launch: returns ``(weights [1,k'],
    ids [1,k'], plan)`` with the same contents as the two calls (one-token decode step)."""
    torch = _torch()
    if logits2d.dtype != torch.float32 or not logits2d.is_contiguous() or logits2d.shape[0] != 1:
        raise ValueError("logits must be a contiguous FP32 tensor of one row")
    e = logits2d.shape[1]
    k_out = int(k) + (1 if extra_id >= 0 else 0)
    weights = torch.empty((1, k_out), dtype=torch.float32, device=logits2d.device)
    ids = torch.empty((1, k_out), dtype=torch.int64, device=logits2d.device)
    max_seg = max_segments_for(1, k_out, n_experts)
    i32 = dict(dtype=torch.int32, device=logits2d.device)
    plan = DeviceRoutingPlan(
        1, k_out, n_experts,
        torch.empty(n_experts, **i32), torch.empty(n_experts + 1, **i32), torch.empty(k_out, **i32),
        torch.empty(k_out, **i32), torch.empty(max_seg, **i32), torch.empty(max_seg, **i32),
        torch.empty(max_seg, **i32), torch.empty(1, **i32), max_seg, torch.empty(1, **i32))
    _lib.call("b200q_router_topk_plan_row", _ptr(logits2d), e, int(k), 1 if renormalize else 0, float(floor),
              int(extra_id), _ptr(extra_weight), _ptr(weights), _ptr(ids), int(n_experts), _ptr(plan.counts),
              _ptr(plan.offsets), _ptr(plan.order), _ptr(plan.inv), _ptr(plan.seg_expert), _ptr(plan.seg_begin),
              _ptr(plan.seg_count), _ptr(plan.num_segments), max_seg, _ptr(plan.status), _lib.current_stream())
    return weights, ids, plan


# Rows of activations from which the grouped gate/up launch is fed with per-token images (one extra small
# launch that converts every row once; below this the segments convert their few tokens themselves).
TOKEN_IMAGE_MIN_ROWS = 32


def token_images(x2d):
    """Per-token activation images of ``x2d [rows, d]`` for ``moe_gate_up(..., images=...)``, or ``None``
    when this width has none. One image serves every expert segment (and every layer input equal to
    ``x2d``) the token appears in."""
    torch = _torch()
    rows, d = x2d.shape
    per_row = _lib.load().b200q_moe_token_image_bytes(int(d), _dtype_id(x2d))
    if per_row <= 0:
        return None
    images = torch.empty((rows, per_row), dtype=torch.uint8, device=x2d.device)
    _lib.call("b200q_moe_token_images", _ptr(x2d), _dtype_id(x2d), int(rows), int(d), _ptr(images),
              _lib.current_stream())
    return images


def moe_gate_up(x2d, plan, gate_bank, up_bank, gate_fmt, up_fmt, f, d, gate_stride, up_stride, *,
                gate_table=None, up_table=None, tables_aligned16=False, images=None):
    """FP32 hidden activations ``[T*k, F]`` in sorted-assignment order.

    Experts live either in contiguous banks (``*_bank`` + byte stride) or behind device pointer
    tables (int64 tensors with one address per expert). ``images`` = ``token_images(x2d)``; by default they
    are made here when ``x2d`` has at least ``TOKEN_IMAGE_MIN_ROWS`` rows (``B200Q_TOKEN_IMAGES=0`` or
    ``images=False`` turns that off). The results are the same bits either way."""
    torch = _torch()
    hbuf = torch.empty((plan.rows * plan.k, f), dtype=torch.float32, device=x2d.device)
    if images is False:          # the caller knows its plan executes too few of the rows for images to pay
        images = None
    elif images is None and x2d.shape[0] >= TOKEN_IMAGE_MIN_ROWS and os.environ.get("B200Q_TOKEN_IMAGES", "1") != "0" \
            and gate_fmt in ("Q4_K", "Q5_K", "Q4_K_TILED", "Q5_K_TILED") and gate_fmt == up_fmt:
        images = token_images(x2d)
    if images is not None:
        _lib.call("b200q_moe_gate_up_images", _ptr(gate_bank), int(gate_stride), _lib.FORMAT_ID[gate_fmt],
                  _ptr(up_bank), int(up_stride), _lib.FORMAT_ID[up_fmt], _ptr(gate_table), _ptr(up_table),
                  1 if tables_aligned16 else 0, f, d, _ptr(x2d), _dtype_id(x2d), _ptr(images), plan.k,
                  _ptr(plan.order), _ptr(plan.seg_expert), _ptr(plan.seg_begin), _ptr(plan.seg_count),
                  _ptr(plan.num_segments), plan.max_segments, _ptr(hbuf), _lib.current_stream())
        return hbuf
    _lib.call("b200q_moe_gate_up", _ptr(gate_bank), int(gate_stride), _lib.FORMAT_ID[gate_fmt], _ptr(up_bank),
              int(up_stride), _lib.FORMAT_ID[up_fmt], _ptr(gate_table), _ptr(up_table), 1 if tables_aligned16 else 0,
              f, d, _ptr(x2d), _dtype_id(x2d), plan.k, _ptr(plan.order),
              _ptr(plan.seg_expert), _ptr(plan.seg_begin), _ptr(plan.seg_count), _ptr(plan.num_segments),
              plan.max_segments, _ptr(hbuf), _lib.current_stream())
    return hbuf


def moe_down(hbuf, route_weights, plan, down_bank, down_fmt, d, f, down_stride, *, down_table=None,
             tables_aligned16=False, flat_rows=False, out=None):
    """Route-weighted FP32 terms ``[T*k, D]`` in sorted-assignment order, or (``flat_rows``) at the
    flat assignment index ``row*k+slot``; ``out`` lets the caller supply (and pre-zero) the buffer."""
    torch = _torch()
    if route_weights.dtype != torch.float32 or not route_weights.is_contiguous():
        raise ValueError("routing weights must be a contiguous FP32 tensor")
    terms = out if out is not None else torch.empty((plan.rows * plan.k, d), dtype=torch.float32,
                                                     device=hbuf.device)
    _lib.call("b200q_moe_down", _ptr(down_bank), int(down_stride), _lib.FORMAT_ID[down_fmt], _ptr(down_table),
              1 if tables_aligned16 else 0, 1 if flat_rows else 0, d, f, _ptr(hbuf),
              _ptr(route_weights), _ptr(plan.order), _ptr(plan.seg_expert), _ptr(plan.seg_begin),
              _ptr(plan.seg_count), _ptr(plan.num_segments), plan.max_segments, _ptr(terms), _lib.current_stream())
    return terms


def moe_combine(terms, plan, d, *, extra=None, extra_scale=None, out_dtype=None):
    """Ordered per-token sum of the k terms (+ optional shared-expert term) -> ``[T, D]``."""
    torch = _torch()
    out_dtype = out_dtype or torch.float32
    out = torch.empty((plan.rows, d), dtype=out_dtype, device=terms.device)
    _lib.call("b200q_moe_combine", _ptr(terms), _ptr(plan.inv), plan.rows, plan.k, d, _ptr(extra), _ptr(extra_scale),
              _ptr(out), _lib.DTYPE_ID[str(out_dtype).replace("torch.", "")], _lib.current_stream())
    return out


COMBINE_NORM_MAX_K = 16


def moe_combine_norm(terms, plan, d, norm, residual, *, extra=None, extra_scale=None, branch_dtype=None, alpha=1.0):
    """``moe_combine`` fused with ``norm.forward_residual_add(residual, branch, alpha)``: returns
    ``(new residual FP32 [T, D], normalised activations [T, D] in the norm weight's dtype)``, the same
    bits as the two calls. ``branch_dtype`` is the type the combine alone would have produced."""
    torch = _torch()
    if residual.dtype != torch.float32 or not residual.is_contiguous() or residual.numel() != plan.rows * d:
        raise ValueError("the residual stream must be a contiguous FP32 tensor of [rows, d]")
    if plan.k > COMBINE_NORM_MAX_K:
        raise NotImplementedError("fused combine + norm handles at most 16 terms per row")
    branch_dtype = branch_dtype or torch.float32
    res_out = torch.empty_like(residual)
    y = torch.empty(residual.shape, dtype=norm.gamma.dtype, device=residual.device)
    name = lambda dt: _lib.DTYPE_ID[str(dt).replace("torch.", "")]
    _lib.call("b200q_moe_combine_norm", _ptr(terms), _ptr(plan.inv), plan.rows, plan.k, d, _ptr(extra),
              _ptr(extra_scale), name(branch_dtype), _ptr(residual), float(alpha), _ptr(norm.gamma),
              name(norm.gamma.dtype), float(norm.eps), _ptr(res_out), _ptr(y), name(y.dtype), _lib.current_stream())
    return res_out, y


def moe_combine_ids(terms_flat, ids2d, d, *, extra=None, extra_scale=None, out_dtype=None):
    """Ordered per-token sum of terms stored at the flat assignment index; ``ids2d`` [T,k] gives the
    order (ascending expert id, then slot). ``extra`` [T,d] (times ``extra_scale`` [T]) is added last."""
    torch = _torch()
    out_dtype = out_dtype or torch.float32
    rows, k = ids2d.shape
    if not ids2d.is_contiguous():
        raise ValueError("expert ids must be contiguous")
    out = torch.empty((rows, d), dtype=out_dtype, device=terms_flat.device)
    _lib.call("b200q_moe_combine_ids", _ptr(terms_flat), _ptr(ids2d), 1 if ids2d.dtype == torch.int64 else 0, rows, k,
              d, _ptr(extra), _ptr(extra_scale), _ptr(out), _lib.DTYPE_ID[str(out_dtype).replace("torch.", "")],
              _lib.current_stream())
    return out


def moe_plan_ep(ids, *, e_global, first_expert, n_local, shared_id, home_lo, home_hi, max_segments=None):
    """Routing plan of one expert-parallel rank over the gathered ids ``[T_all, k]`` (global ids).

    Local expert ids: 0..n_local-1 routed, n_local = shared expert (home rows only), n_local+1 =
    assignments other ranks execute (sorted last, never run). ``max_segments`` overrides the segment
    bound (never below what this rank's plan can need): the grouped kernels derive their split of K
    over warps from it, so a rank that passes the single-GPU layer's bound sums in the same order."""
    torch = _torch()
    if ids.dtype not in (torch.int32, torch.int64) or not ids.is_contiguous():
        raise ValueError("expert ids must be a contiguous int32/int64 tensor")
    rows, k = ids.shape
    n_plan = n_local + 2
    total = rows * k
    max_seg = max(max_segments_for(rows, k, n_plan), int(max_segments or 0))
    i32 = dict(dtype=torch.int32, device=ids.device)
    plan = DeviceRoutingPlan(
        rows, k, n_plan,
        torch.empty(n_plan, **i32), torch.empty(n_plan + 1, **i32), torch.empty(total, **i32),
        torch.empty(total, **i32), torch.empty(max_seg, **i32), torch.empty(max_seg, **i32),
        torch.empty(max_seg, **i32), torch.empty(1, **i32), max_seg, torch.empty(1, **i32))
    _lib.call("b200q_moe_plan_ep", _ptr(ids), 1 if ids.dtype == torch.int64 else 0, rows, k, int(e_global),
              int(first_expert), int(n_local), int(shared_id), int(home_lo), int(home_hi), SEGMENT_CAP,
              _ptr(plan.counts), _ptr(plan.offsets), _ptr(plan.order), _ptr(plan.inv), _ptr(plan.seg_expert),
              _ptr(plan.seg_begin), _ptr(plan.seg_count), _ptr(plan.num_segments), max_seg, _ptr(plan.status),
              _lib.current_stream())
    return plan


def moe_down_peer(hbuf, route_weights, plan, down_fmt, d, f, *, down_table, tables_aligned16, term_tables,
                  rows_per_rank):
    """Grouped down projection whose route-weighted term rows go straight to their home rank's buffer
    (``term_tables``: int64 device tensor with one base address per rank)."""
    torch = _torch()
    if route_weights.dtype != torch.float32 or not route_weights.is_contiguous():
        raise ValueError("routing weights must be a contiguous FP32 tensor")
    _lib.call("b200q_moe_down_peer", None, 0, _lib.FORMAT_ID[down_fmt], _ptr(down_table),
              1 if tables_aligned16 else 0, d, f, _ptr(hbuf), _ptr(route_weights), _ptr(plan.order),
              _ptr(plan.seg_expert), _ptr(plan.seg_begin), _ptr(plan.seg_count), _ptr(plan.num_segments),
              plan.max_segments, _ptr(term_tables), int(rows_per_rank), _lib.current_stream())
