"""Routed expert execution on device-resident packed banks.

Host-side mirror of the reference's sparse dispatcher ``ExpertsInference.forward``
(``mini_llm/ops/experts_inference.py:160-312``) and of the part of
``HeterogeneousExpertExecutor`` that the dispatcher calls
(``mini_llm/ops/expert_residency.py:1166-1208``: ``forward``, ``try_forward_grouped``,
``dispatch_scope``). Differences that follow from the target: a B200 holds every expert of the
model in HBM, so there is no cache, no eviction and no CPU path; and the dispatch plan is built on
the device (``b200q_moe_plan``), so no expert count or id ever travels to the host - the same code
path serves one token and many, and can be captured in a CUDA graph.

Semantics kept: each token adds ``route_weight * FFN_e(x)`` over its k experts in ascending
expert id, every term rounded to FP32 before the next plain FP32 add.
"""

import contextlib
from dataclasses import dataclass

import numpy as np

from . import moe_ops
from .quantized_linear import DevicePackedGGUFWeight, PackedExpertFFNInference, packed_bytes_to_device
from .quantized_weight import BLOCK_FORMATS, DEVICE_LAYOUTS, PackedGGUFWeight, packed_nbytes


def _torch():
    import torch
    return torch


@dataclass
class PackedExpertBank:
    """All experts of one MoE layer as three contiguous packed banks in HBM.

    ``gate`` / ``up`` hold ``[E, F, D]`` and ``down`` ``[E, D, F]`` packed rows (uint8 CUDA
    tensors); expert ``e`` starts ``e * stride`` bytes into its bank.
    """

    gate: object
    up: object
    down: object
    gate_type: str
    up_type: str
    down_type: str
    n_experts: int
    d_model: int
    d_ff: int

    def __post_init__(self):
        for name, fmt, shape in (("gate", self.gate_type, (self.d_ff, self.d_model)),
                                 ("up", self.up_type, (self.d_ff, self.d_model)),
                                 ("down", self.down_type, (self.d_model, self.d_ff))):
            if fmt not in BLOCK_FORMATS and fmt not in DEVICE_LAYOUTS:
                raise ValueError(f"Unsupported packed GGUF type: {fmt}")
            data = getattr(self, name)
            expect = self.n_experts * packed_nbytes(shape, fmt)
            if int(data.numel()) != expect:
                raise ValueError(f"{name} bank: expected {expect} bytes, got {int(data.numel())}")

    @property
    def gate_stride(self):
        return packed_nbytes((self.d_ff, self.d_model), self.gate_type)

    @property
    def up_stride(self):
        return packed_nbytes((self.d_ff, self.d_model), self.up_type)

    @property
    def down_stride(self):
        return packed_nbytes((self.d_model, self.d_ff), self.down_type)

    @property
    def nbytes(self):
        return int(self.gate.numel() + self.up.numel() + self.down.numel())

    @classmethod
    def from_packed(cls, gate, up, down):
        """Upload three host ``PackedGGUFWeight`` tensors shaped [E,F,D], [E,F,D], [E,D,F]."""
        for w in (gate, up, down):
            if not isinstance(w, PackedGGUFWeight) or len(w.shape) != 3:
                raise TypeError("expected three-dimensional PackedGGUFWeight banks")
        e, f, d = gate.shape
        if up.shape != (e, f, d) or down.shape != (e, d, f):
            raise ValueError("expert bank shapes must be gate/up [E,F,D], down [E,D,F]")
        return cls(packed_bytes_to_device(gate.data), packed_bytes_to_device(up.data),
                   packed_bytes_to_device(down.data), gate.quant_type, up.quant_type, down.quant_type, e, d, f)

    def retiled(self):
        """Bank with its Q4_K / Q5_K / Q6_K / Q8_0 projections in the tile layout (new tensors for the converted
        banks, the others are shared). Gate and up are converted together or not at all; shapes the
        layout does not cover keep the GGUF bytes."""
        from .quantized_linear import can_retile, retile_bytes, _RETILE
        gate, up, down = self.gate, self.up, self.down
        gate_type, up_type, down_type = self.gate_type, self.up_type, self.down_type
        if gate_type == up_type and can_retile(gate_type, self.d_ff, self.d_model) and gate_type in ("Q4_K", "Q5_K"):
            gate = retile_bytes(gate, self.n_experts * self.d_ff, self.d_model, gate_type)
            up = retile_bytes(up, self.n_experts * self.d_ff, self.d_model, up_type)
            gate_type = up_type = _RETILE[gate_type][1]
        if can_retile(down_type, self.d_model, self.d_ff):
            down = retile_bytes(down, self.n_experts * self.d_model, self.d_ff, down_type)
            down_type = _RETILE[down_type][1]
        if (gate_type, down_type) == (self.gate_type, self.down_type):
            return self
        return PackedExpertBank(gate, up, down, gate_type, up_type, down_type, self.n_experts, self.d_model,
                                self.d_ff)

    def pointer_tables(self, extra=None):
        """Device pointer tables (three int64 tensors with one address per expert) and whether every
        address is 16-byte aligned. ``extra`` = optional (gate, up, down) DevicePackedGGUFWeight triple
        appended as expert ``n_experts`` (an always-on shared expert of the same shape and formats)."""
        torch = _torch()
        cols = []
        for bank, stride, w in ((self.gate, self.gate_stride, 0), (self.up, self.up_stride, 1),
                                (self.down, self.down_stride, 2)):
            ptrs = [bank.data_ptr() + e * stride for e in range(self.n_experts)]
            if extra is not None:
                ptrs.append(extra[w].data.data_ptr())
            cols.append(ptrs)
        aligned = all(p % 16 == 0 for col in cols for p in col)
        tables = tuple(torch.tensor(col, dtype=torch.int64, device=self.gate.device) for col in cols)
        return tables, aligned

    def expert(self, index):
        """Zero-copy ``PackedExpertFFNInference`` handle of one expert."""
        if not 0 <= int(index) < self.n_experts:
            raise IndexError(index)
        i = int(index)
        view = lambda bank, stride, shape, fmt: DevicePackedGGUFWeight(bank[i * stride:(i + 1) * stride], shape, fmt)
        return PackedExpertFFNInference(
            view(self.gate, self.gate_stride, (self.d_ff, self.d_model), self.gate_type),
            view(self.up, self.up_stride, (self.d_ff, self.d_model), self.up_type),
            view(self.down, self.down_stride, (self.d_model, self.d_ff), self.down_type))


def routed_experts_forward(x2d, weights2d, ids2d, bank, *, extra=None, extra_scale=None, out_dtype=None,
                           tables=None, tables_aligned16=False, n_experts=None, residual_norm=None, plan=None):
    """plan -> grouped gate/up -> grouped down (route-weighted) -> ordered combine.

    x2d [T,D]; weights2d FP32 [T,k]; ids2d int32/int64 [T,k]; returns [T,D]. With ``tables`` (from
    ``PackedExpertBank.pointer_tables``) experts are addressed through pointer tables and
    ``n_experts`` may exceed the bank (appended shared expert). With ``residual_norm = (norm,
    residual)`` the combine also performs the residual add and RMSNorm that follow the layer and
    the result is ``(new residual, normalised activations)`` (``moe_ops.moe_combine_norm``).
    """
    torch = _torch()
    if plan is None:                      # a caller that routed a single row may bring the plan along
        plan = moe_ops.moe_plan(ids2d, n_experts or bank.n_experts)
    route = weights2d if weights2d.dtype == torch.float32 else weights2d.float()
    if tables is not None:
        hbuf = moe_ops.moe_gate_up(x2d, plan, None, None, bank.gate_type, bank.up_type, bank.d_ff, bank.d_model, 0, 0,
                                   gate_table=tables[0], up_table=tables[1], tables_aligned16=tables_aligned16)
        terms = moe_ops.moe_down(hbuf, route.contiguous().reshape(-1), plan, None, bank.down_type, bank.d_model,
                                 bank.d_ff, 0, down_table=tables[2], tables_aligned16=tables_aligned16)
        return _combine(terms, plan, bank.d_model, extra, extra_scale, out_dtype or x2d.dtype, residual_norm)
    hbuf = moe_ops.moe_gate_up(x2d, plan, bank.gate, bank.up, bank.gate_type, bank.up_type, bank.d_ff,
                               bank.d_model, bank.gate_stride, bank.up_stride)
    terms = moe_ops.moe_down(hbuf, route.contiguous().reshape(-1), plan, bank.down, bank.down_type, bank.d_model,
                             bank.d_ff, bank.down_stride)
    return _combine(terms, plan, bank.d_model, extra, extra_scale, out_dtype or x2d.dtype, residual_norm)


def _combine(terms, plan, d, extra, extra_scale, out_dtype, residual_norm):
    if residual_norm is None:
        return moe_ops.moe_combine(terms, plan, d, extra=extra, extra_scale=extra_scale, out_dtype=out_dtype)
    norm, residual = residual_norm
    return moe_ops.moe_combine_norm(terms, plan, d, norm, residual, extra=extra, extra_scale=extra_scale,
                                    branch_dtype=out_dtype)


class ResidentExpertExecutor:
    """Executor with every expert resident in HBM (the reference's executor API, minus caching).

    ``banks`` maps layer id -> ``PackedExpertBank``.
    """

    overlaps_cpu_gpu = False
    routing_profiler = None

    def __init__(self, banks, *, model_id="model", compute_dtype="float32"):
        if not banks:
            raise ValueError("at least one expert bank is required")
        self.banks = dict(banks)
        first = next(iter(self.banks.values()))
        self.model_id = model_id
        self.d_model, self.d_ff = first.d_model, first.d_ff
        self.compute_dtype = compute_dtype
        self._dispatch_depth = 0
        self.counters = {"gpu_experts": 0, "grouped_gpu_dispatches": 0}

    def bank(self, layer_id):
        return self.banks[int(layer_id)]

    def forward(self, layer_id, expert_id, x):
        """One expert's FFN on a batch of rows ``[M, D]``."""
        return self.bank(layer_id).expert(expert_id).forward(x)

    @contextlib.contextmanager
    def dispatch_scope(self, layer_id, expert_ids):
        """Scope of one layer's dispatch (the reference pins the selected experts against eviction here,
        ``expert_residency.py:539-560``; nothing can be evicted from a resident bank, so only the depth is
        kept: ``try_forward_grouped`` is valid inside a scope only, as in the reference)."""
        self._dispatch_depth += 1
        try:
            yield self
        finally:
            self._dispatch_depth -= 1

    def try_forward_grouped(self, layer_id, expert_ids, x, routing_weights, slots):
        """One-row grouped dispatch over resident experts, or ``None`` when the call is not eligible
        (``expert_residency.py:1166-1193``): needs an open ``dispatch_scope``, a single FP32 row, expert
        ids of this layer's bank and a layout the grouped kernels support. A decline changes no counter."""
        from .grouped_quantized_experts import grouped_quantized_experts_forward, supports_grouped_quantized_experts
        if not self._dispatch_depth or x.shape[0] != 1 or int(layer_id) not in self.banks:
            return None
        bank = self.banks[int(layer_id)]
        ids = [int(e) for e in expert_ids]
        if not ids or any(not 0 <= e < bank.n_experts for e in ids):
            return None
        experts = [bank.expert(e) for e in ids]
        if not supports_grouped_quantized_experts(x, experts, routing_weights, routing_slots=None if slots is None
                                                  else tuple(slots)):
            return None
        out = grouped_quantized_experts_forward(x, experts, routing_weights,
                                                routing_slots=None if slots is None else tuple(slots))
        self.counters["gpu_experts"] += len(experts)
        self.counters["grouped_gpu_dispatches"] += 1
        return out

    def forward_routed(self, layer_id, x2d, weights2d, ids2d, **kwargs):
        """Device-side dispatch of any number of rows (plan, grouped kernels, ordered combine) with no
        host round trip - the fast path ``ExpertsInference`` prefers when an executor offers it."""
        return routed_experts_forward(x2d, weights2d, ids2d, self.bank(layer_id), **kwargs)

    def statistics(self):
        return {"resident_layers": len(self.banks), "resident_bytes": sum(b.nbytes for b in self.banks.values()),
                **self.counters}


class ExpertsInference:
    """Mixture of expert FFNs for inference; evaluates only the selected experts."""

    def __init__(self, d_model, d_ff, n_experts, dtype="float32", *, expert_executor=None, layer_id=0):
        if expert_executor is None:
            raise RuntimeError("ExpertsInference needs an expert_executor holding packed banks "
                               "(dense per-expert weights are not part of this package)")
        self.d_model, self.d_ff, self.n_experts = d_model, d_ff, n_experts
        self.expert_executor = expert_executor
        self.layer_id = int(layer_id)

    def forward(self, x, weights, expert_indices, *, on_cpu_submitted=None):
        """x [B,T,D]; weights [B,T,k]; expert_indices [B,T,k] -> [B,T,D] in x's dtype.

        An executor that offers ``forward_routed`` (``ResidentExpertExecutor``) gets the whole dispatch
        as device work. Any other executor is driven through the reference's own seam
        (``mini_llm/ops/experts_inference.py:188-312``): inside ``dispatch_scope``, one row with
        unique ids first tries ``try_forward_grouped(layer_id, ascending ids, x, weights, slots)``;
        otherwise each active expert, in ascending id, runs ``forward(layer_id, id, rows)`` and its
        route-weighted output is added to the rows' accumulators (FP32, rounded once at the end)."""
        batch, seq, d_model = x.shape
        k = weights.shape[-1]
        n = batch * seq
        x2d = x.reshape(n, d_model)
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        ids = expert_indices.reshape(n, k)
        if not ids.is_contiguous():
            ids = ids.contiguous()
        executor = self.expert_executor
        if hasattr(executor, "forward_routed"):
            out = executor.forward_routed(self.layer_id, x2d, weights.reshape(n, k), ids)
            if on_cpu_submitted is not None:
                on_cpu_submitted()
            return out.reshape(batch, seq, d_model)
        return self._forward_reference_seam(x2d, weights.reshape(n, k), ids, on_cpu_submitted).reshape(batch, seq, d_model)

    def _forward_reference_seam(self, x2d, weights2d, ids2d, on_cpu_submitted):
        torch = _torch()
        executor = self.expert_executor
        n, k = ids2d.shape
        host_ids = ids2d.detach().cpu().numpy().astype(np.int64)         # the reference plans on the host as well
        if host_ids.min(initial=0) < 0 or host_ids.max(initial=0) >= self.n_experts:
            raise ValueError("expert index outside [0, n_experts)")
        active = [int(e) for e in np.unique(host_ids)]
        singleton = n == 1 and len(active) == k                          # one row, no repeated id
        acc = torch.zeros(x2d.shape, dtype=torch.float32, device=x2d.device)
        called = False
        with executor.dispatch_scope(self.layer_id, active):
            grouped = getattr(executor, "try_forward_grouped", None)
            if singleton and grouped is not None:
                slot_of = {int(e): s for s, e in enumerate(host_ids[0])}
                out = grouped(self.layer_id, active, x2d, weights2d.reshape(-1), tuple(slot_of[e] for e in active))
                if out is not None:
                    if on_cpu_submitted is not None:
                        on_cpu_submitted()
                    return out.to(x2d.dtype)
            if on_cpu_submitted is not None:
                on_cpu_submitted()
                called = True
            for e in active:
                rows, slots = np.nonzero(host_ids == e)
                order = np.argsort(rows, kind="stable")
                rows_t = torch.as_tensor(rows[order], device=x2d.device)
                slots_t = torch.as_tensor(slots[order], device=x2d.device)
                out = executor.forward(self.layer_id, e, x2d.index_select(0, rows_t))
                term = out.float() * weights2d[rows_t, slots_t].float()[:, None]
                acc.index_add_(0, rows_t, term)                          # a row names an expert once per slot
        if on_cpu_submitted is not None and not called:
            on_cpu_submitted()
        return acc.to(x2d.dtype)


def synthetic_bank(n_experts, d_model, d_ff, types=("Q4_K", "Q4_K", "Q6_K"), seed=0, device="cuda"):
    """Random-byte expert bank generated on the device (benchmark / smoke input).

    The quant codes and sub-block scales are uniform random bytes; the FP16 super-block scales are
    set to small finite values so that outputs stay O(1). Layout and sizes are exactly those of a
    real bank; the bytes are reproducible for a given seed.
    """
    torch = _torch()
    gen = torch.Generator(device=device)
    banks = []
    for i, (fmt, shape) in enumerate(zip(types, ((d_ff, d_model), (d_ff, d_model), (d_model, d_ff)))):
        gen.manual_seed(seed * 3 + i)
        qk, qb = BLOCK_FORMATS[fmt]
        nblocks = n_experts * shape[0] * shape[1] // qk
        raw = torch.randint(0, 256, (nblocks, qb), dtype=torch.uint8, device=device, generator=gen)
        half = lambda v: torch.tensor(np.frombuffer(np.float16(v).tobytes(), np.uint8).copy(), device=device)
        if fmt == "Q6_K":
            raw[:, 208:210] = half(1.0 / 4096)
        elif fmt in ("Q4_K", "Q5_K"):
            raw[:, 0:2] = half(1.0 / 2048)
            raw[:, 2:4] = half(1.0 / 4096)
        else:
            raw[:, 0:2] = half(1.0 / 2048)
        banks.append(raw.reshape(-1))
    return PackedExpertBank(banks[0], banks[1], banks[2], types[0], types[1], types[2], n_experts, d_model, d_ff)
