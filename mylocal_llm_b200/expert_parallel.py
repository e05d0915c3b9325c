"""Expert-parallel packed MoE over the GPUs of one node (one process per GPU).

The reference is single-process and has no multi-GPU path; this module adds one whose result is,
bit for bit, the single-GPU layer's (``moe_layer.PackedMoELayer``), whatever the number of ranks:

* rank ``r`` of ``G`` owns the contiguous expert range ``expert_partition(E, G)[r]`` of every layer;
  router weights, shared expert and norms are replicated; tokens are data-parallel (every rank
  reserves the same number of row slots per call and may fill fewer, down to none);
* per layer: every rank routes its own rows -> rows, routing weights and expert ids of all ranks are
  gathered on every rank -> each rank runs the assignments that hit its experts (plus the shared
  expert for its own rows) ->
  the route-weighted FP32 term of assignment ``row*k+slot`` travels to the row's home rank -> the
  home rank adds its rows' terms in ascending expert id (the reference's order,
  ``mini_llm/ops/grouped_quantized_experts.py:70-79``).

Every term row has exactly one producer, so the exchange never adds two non-zero numbers and the
result does not depend on ``G``. Two exchanges implement it:

``PeerComm``        the grouped down projection stores each term row directly into the home rank's
                    arena through NVLink peer memory (``b200q_moe_down_peer``), the rows are gathered
                    by peer stores as well, and ranks synchronise with a bounded device barrier -
                    no library collective on the decode path;
``CollectiveComm``  ``torch.distributed``: all-gather of rows, reduce-scatter of a zero-filled term
                    buffer (NCCL on GPUs; gloo in the CPU tests of the host logic).
"""

import ctypes
import os

from . import _lib


def _torch():
    import torch
    return torch


# Optional callable(name): called between the phases of a layer ("route", "push", "plan", "gate_up", "down",
# "barrier", "combine") after the phase's launches are issued. A benchmark sets it to record CUDA events;
# it stays None in normal use.
PHASE_HOOK = None


def _phase(name):
    if PHASE_HOOK is not None:
        PHASE_HOOK(name)


def expert_partition(n_experts, world):
    """[(first, count)] per rank: contiguous, ascending, sizes differing by at most one."""
    if world < 1 or n_experts < world:
        raise ValueError("need at least one expert per rank")
    base, rem = divmod(int(n_experts), int(world))
    out, first = [], 0
    for r in range(world):
        count = base + (1 if r < rem else 0)
        out.append((first, count))
        first += count
    return out


# ------------------------------------------------------------------------------------ exchanges
class LocalComm:
    """World of one rank (also the base class of the real exchanges)."""

    peer = False
    rank, world = 0, 1

    def all_gather_rows(self, x2d):
        return x2d

    def gather_routed(self, x2d, weights, ids):
        """Rows, routing weights and expert ids of all ranks, rank-major."""
        return self.all_gather_rows(x2d), self.all_gather_rows(weights), self.all_gather_rows(ids)

    def exchange_terms(self, terms_all, rows_per_rank):
        return terms_all

    def barrier(self):
        pass

    def close(self):
        pass


class CollectiveComm(LocalComm):
    """``torch.distributed`` exchange (NCCL on CUDA tensors, gloo on CPU tensors)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._gloo = dist.get_backend(group) == "gloo"

    def all_gather_rows(self, x2d):
        torch = _torch()
        if self.world == 1:
            return x2d
        out = torch.empty((self.world * x2d.shape[0],) + tuple(x2d.shape[1:]), dtype=x2d.dtype, device=x2d.device)
        if self._gloo and x2d.dtype == torch.bfloat16:          # gloo has no bf16 all-gather
            raw = x2d.contiguous().view(torch.uint8)
            parts = torch.empty((self.world * raw.shape[0], raw.shape[1]), dtype=torch.uint8)
            self.dist.all_gather_into_tensor(parts, raw, group=self.group)
            return parts.view(torch.bfloat16)
        self.dist.all_gather_into_tensor(out, x2d.contiguous(), group=self.group)
        return out

    def exchange_terms(self, terms_all, rows_per_rank):
        """terms_all [world*rows_per_rank, D], zero where another rank produces the row; returns this
        rank's rows summed over ranks (one non-zero contributor each, hence exact)."""
        torch = _torch()
        if self.world == 1:
            return terms_all
        if self._gloo:                                           # gloo has no reduce-scatter
            self.dist.all_reduce(terms_all, group=self.group)
            return terms_all[self.rank * rows_per_rank:(self.rank + 1) * rows_per_rank].contiguous()
        out = torch.empty((rows_per_rank,) + tuple(terms_all.shape[1:]), dtype=terms_all.dtype,
                          device=terms_all.device)
        self.dist.reduce_scatter_tensor(out, terms_all, group=self.group)
        return out


class _RawDeviceMemory:
    """CUDA array interface over a raw device address, so torch can view it without owning it."""

    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(address), False),
                                         "version": 2, "strides": None}


class PeerComm(LocalComm):
    """Exchange through mapped peer memory (CUDA IPC arenas) with a bounded device-side barrier.

    Arena of each rank: ``[signal pad 256 B | gathered rows | gathered routing weights | gathered
    expert ids | term rows this rank is home of]``,
    sized for ``max_rows`` rows per rank of width ``d_model`` and ``k_out`` terms per row.
    ``group`` is only used at construction, to exchange the 64-byte IPC handles.
    """

    peer = True
    PAD_BYTES = 256

    def __init__(self, group, *, max_rows, d_model, k_out, timeout_ms=None):
        import torch.distributed as dist
        torch = _torch()
        self._dist, self._group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 16:
            raise ValueError("PeerComm supports at most 16 ranks")
        self.max_rows, self.d_model, self.k_out = int(max_rows), int(d_model), int(k_out)
        self.timeout_ms = int(timeout_ms or os.environ.get("B200Q_PEER_TIMEOUT_MS", 5000))
        self.device = torch.device("cuda", torch.cuda.current_device())
        align = lambda v: (v + 255) // 256 * 256
        self.rows_offset = self.PAD_BYTES
        self.weights_offset = align(self.rows_offset + self.world * self.max_rows * self.d_model * 4)
        self.ids_offset = align(self.weights_offset + self.world * self.max_rows * self.k_out * 4)
        self.terms_offset = align(self.ids_offset + self.world * self.max_rows * self.k_out * 8)
        self.nbytes = align(self.terms_offset + self.max_rows * self.k_out * self.d_model * 4)
        base = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        _lib.call("b200q_peer_alloc", self.nbytes, ctypes.byref(base), handle)
        self._own = base.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.bases, self._opened = [], []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self._own)
                continue
            ptr = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            _lib.call("b200q_peer_open", buf, ctypes.byref(ptr))
            self.bases.append(ptr.value)
            self._opened.append(ptr.value)
        table = lambda off: torch.tensor([b + off for b in self.bases], dtype=torch.int64, device=self.device)
        self.pad_table = table(0)
        self.rows_table = table(self.rows_offset)
        self.terms_table = table(self.terms_offset)
        self._local = torch.as_tensor(_RawDeviceMemory(self._own, self.nbytes), device=self.device)
        torch.cuda.synchronize()
        dist.barrier(group=group)          # every arena is mapped and cleared before the first kernel

    def _view(self, offset, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * dtype.itemsize
        return self._local[offset:offset + nbytes].view(dtype).reshape(shape)

    def _check(self, rows, d):
        if rows > self.max_rows or d != self.d_model:
            raise ValueError(f"PeerComm was sized for {self.max_rows} rows of width {self.d_model}")

    def barrier(self):
        _lib.call("b200q_peer_barrier", ctypes.c_void_p(self.pad_table.data_ptr()), self.rank, self.world,
                  self.timeout_ms, _lib.current_stream())

    def all_gather_rows(self, x2d):
        rows, d = x2d.shape
        self._check(rows, d)
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        nbytes = rows * d * x2d.element_size()
        _lib.call("b200q_peer_push_rows", ctypes.c_void_p(x2d.data_ptr()), nbytes,
                  ctypes.c_void_p(self.rows_table.data_ptr()), self.rank * nbytes, self.world, _lib.current_stream())
        self.barrier()
        return self._view(self.rows_offset, (self.world * rows, d), x2d.dtype)

    def gather_routed(self, x2d, weights, ids):
        """One store kernel for the three buffers, one barrier; returns views of the local arena."""
        torch = _torch()
        rows, d = x2d.shape
        self._check(rows, d)
        k_out = weights.shape[1]
        if k_out > self.k_out or tuple(ids.shape) != (rows, k_out):
            raise ValueError(f"PeerComm was sized for {self.k_out} routes per row")
        if weights.dtype != torch.float32 or ids.dtype != torch.int64:
            raise TypeError("routing weights must be FP32 and expert ids int64")
        x2d, weights, ids = x2d.contiguous(), weights.contiguous(), ids.contiguous()
        xb, wb, ib = rows * d * x2d.element_size(), rows * k_out * 4, rows * k_out * 8
        _lib.call("b200q_peer_push3", ctypes.c_void_p(x2d.data_ptr()), xb, self.rows_offset + self.rank * xb,
                  ctypes.c_void_p(weights.data_ptr()), wb, self.weights_offset + self.rank * wb,
                  ctypes.c_void_p(ids.data_ptr()), ib, self.ids_offset + self.rank * ib,
                  ctypes.c_void_p(self.pad_table.data_ptr()), self.world, _lib.current_stream())
        self.barrier()
        n = self.world * rows
        return (self._view(self.rows_offset, (n, d), x2d.dtype),
                self._view(self.weights_offset, (n, k_out), torch.float32),
                self._view(self.ids_offset, (n, k_out), torch.int64))

    def term_buffers(self, rows, k_out, d):
        """(device table of the ranks' term buffers, this rank's own buffer [rows*k_out, d])."""
        self._check(rows, d)
        if k_out > self.k_out:
            raise ValueError(f"PeerComm was sized for {self.k_out} terms per row")
        return self.terms_table, self._view(self.terms_offset, (rows * k_out, d), _torch().float32)

    def close(self):
        """Collective: every rank stops using the arenas before any of them is unmapped or freed."""
        _torch().cuda.synchronize()
        self._dist.barrier(group=self._group)
        for ptr in self._opened:
            _lib.call("b200q_peer_close", ctypes.c_void_p(ptr))
        self._opened = []
        if self._own:
            self._local = None
            _lib.call("b200q_peer_free", ctypes.c_void_p(self._own))
            self._own = None


# ------------------------------------------------------------------------------------ device engine
class DeviceExpertEngine:
    """The three device steps of one rank: route all rows, run the local assignments, combine.

    ``bank`` holds this rank's experts (``first_expert`` .. ``first_expert + bank.n_experts - 1`` of
    ``n_experts_global``). A shared expert with the routed experts' shape and formats is folded in
    as global id ``n_experts_global`` (added last, as in the single-GPU layer); any other shared
    expert is evaluated on the home rank's own rows and handed to the combine as ``extra``.
    """

    def __init__(self, bank, router_weight, top_k, *, first_expert, n_experts_global, shared=None, shared_gate=None,
                 normalization_floor=2.0 ** -14):
        from .quantized_linear import retile_enabled, retile_gate_up, retile_weight
        from .router_inference import RouterInference
        if retile_enabled():
            bank = bank.retiled()
            if shared is not None:
                gate_t, up_t = retile_gate_up(shared[0], shared[1])
                shared = (gate_t, up_t, retile_weight(shared[2]))
        self.bank = bank
        self.first_expert, self.n_global = int(first_expert), int(n_experts_global)
        self.router = RouterInference(bank.d_model, self.n_global, top_k, renormalize_selected=True,
                                      normalization_floor=normalization_floor)
        self.router.W_router = router_weight
        self.router.b_router = None
        self.shared, self.shared_gate = shared, shared_gate
        same = shared is not None and all(
            w.shape == shape and w.quant_type == fmt for w, shape, fmt in zip(
                shared, ((bank.d_ff, bank.d_model), (bank.d_ff, bank.d_model), (bank.d_model, bank.d_ff)),
                (bank.gate_type, bank.up_type, bank.down_type)))
        self.folded = bool(same)
        self.tables, self.aligned = bank.pointer_tables(extra=shared if self.folded else None)
        self.k_out = int(top_k) + (1 if self.folded else 0)
        # one past the last global id (the folded shared expert included): padding entry of the exchange
        self.pad_id = self.n_global + (1 if self.folded else 0)

    def route(self, x_all):
        from . import moe_ops
        logits = self.router.logits(x_all)
        scale = None
        if self.folded and self.shared_gate is not None:
            scale = moe_ops.shared_gate(x_all, self.shared_gate)
        return moe_ops.router_topk(logits, self.router.k, renormalize=True, floor=self.router.normalization_floor,
                                   extra_id=self.n_global if self.folded else -1, extra_weight=scale)

    def local_terms(self, x_all, weights, ids, home_lo, home_hi, *, peer=None, total_rows=None):
        """Run this rank's assignments. ``peer`` = (term table, rows_per_rank): rows go to their home
        ranks' buffers and nothing is returned; otherwise returns the zero-filled flat term buffer.
        ``total_rows`` = real rows of all ranks (default: every gathered row is real); the plan then
        carries the segment bound of the single-GPU layer for that batch, which makes the grouped
        kernels split K as they would there - the condition for bit-identical sums."""
        from . import moe_ops
        torch = _torch()
        bank = self.bank
        e_global = self.n_global + (1 if self.folded else 0)
        bound = moe_ops.max_segments_for(int(total_rows or ids.shape[0]), ids.shape[1], e_global)
        plan = moe_ops.moe_plan_ep(ids, e_global=e_global, first_expert=self.first_expert, n_local=bank.n_experts,
                                   shared_id=self.n_global if self.folded else -1, home_lo=home_lo, home_hi=home_hi,
                                   max_segments=bound)
        _phase("plan")
        hbuf = moe_ops.moe_gate_up(x_all, plan, None, None, bank.gate_type, bank.up_type, bank.d_ff, bank.d_model, 0, 0,
                                   gate_table=self.tables[0], up_table=self.tables[1], tables_aligned16=self.aligned)
        _phase("gate_up")
        route = (weights if weights.dtype == torch.float32 else weights.float()).contiguous().reshape(-1)
        if peer is not None:
            moe_ops.moe_down_peer(hbuf, route, plan, bank.down_type, bank.d_model, bank.d_ff,
                                  down_table=self.tables[2], tables_aligned16=self.aligned, term_tables=peer[0],
                                  rows_per_rank=peer[1])
            _phase("down")
            return None
        terms = torch.zeros((ids.shape[0] * ids.shape[1], bank.d_model), dtype=torch.float32, device=x_all.device)
        moe_ops.moe_down(hbuf, route, plan, None, bank.down_type, bank.d_model, bank.d_ff, 0,
                         down_table=self.tables[2], tables_aligned16=self.aligned, flat_rows=True, out=terms)
        _phase("down")
        return terms

    def combine(self, terms_home, ids_home, x_home, out_dtype):
        from . import moe_ops
        from .quantized_linear import quantized_linear, quantized_swiglu
        torch = _torch()
        extra = extra_scale = None
        if self.shared is not None and not self.folded:
            gate, up, down = self.shared
            extra = quantized_linear(quantized_swiglu(x_home, gate, up, out_dtype=torch.float32, allow_gemm=False), down,
                                     allow_gemm=False)
            if self.shared_gate is not None:
                extra_scale = moe_ops.shared_gate(x_home, self.shared_gate)
        return moe_ops.moe_combine_ids(terms_home, ids_home, self.bank.d_model, extra=extra, extra_scale=extra_scale,
                                       out_dtype=out_dtype)


# ------------------------------------------------------------------------------------ layer / stack
class ExpertParallelMoELayer:
    """One MoE layer whose routed experts are spread over the ranks of ``comm``.

    ``engine`` is a ``DeviceExpertEngine`` (or, in host-logic tests, any object with the same
    ``route`` / ``local_terms`` / ``combine`` / ``k_out`` interface).
    """

    def __init__(self, engine, comm, d_model):
        self.engine, self.comm, self.d_model = engine, comm, int(d_model)
        self._empty_slots = {}

    def forward(self, hidden, slot_rows=None, total_rows=None):
        """hidden [B, T, D] (this rank's rows) -> [B, T, D].

        ``slot_rows`` = rows every rank reserves in the exchange, the same number on every rank and at
        least this rank's ``B*T`` (default: ``B*T``, i.e. every rank brings the same number of rows).
        A rank with fewer rows - none at all is allowed, as ``[1, 0, D]`` - fills the rest of its slot
        with padding entries that no rank executes, so a batch that does not divide by the number of
        ranks (one token on eight GPUs) costs only the experts its real rows select. ``total_rows`` =
        real rows of all ranks together (default ``world * slot_rows``); give it when slots are partly
        filled and the result has to equal the single-GPU layer's bit for bit."""
        if hidden.ndim != 3 or hidden.shape[-1] != self.d_model:
            raise ValueError("hidden must have shape [batch,time,d_model]")
        batch, seq, d = hidden.shape
        rows = batch * seq
        slot = rows if slot_rows is None else int(slot_rows)
        if slot < rows:
            raise ValueError("slot_rows must cover this rank's rows")
        if slot == 0:
            return hidden.clone()
        x2d = hidden.reshape(rows, d)
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        comm, engine = self.comm, self.engine
        weights = ids = None
        if rows:
            weights, ids = engine.route(x2d)
        _phase("route")
        x_slot, w_slot, ids_slot = self._fill_slot(x2d, weights, ids, rows, slot)
        x_all, w_all, ids_all = comm.gather_routed(x_slot, w_slot, ids_slot)
        _phase("push")
        home_lo, home_hi = comm.rank * slot, comm.rank * slot + rows
        rows_per_rank = slot * engine.k_out
        if comm.peer:
            table, terms_home = comm.term_buffers(slot, engine.k_out, d)
            engine.local_terms(x_all, w_all, ids_all, home_lo, home_hi, peer=(table, rows_per_rank),
                               total_rows=total_rows)
            comm.barrier()
        else:
            terms_all = engine.local_terms(x_all, w_all, ids_all, home_lo, home_hi, total_rows=total_rows)
            terms_home = comm.exchange_terms(terms_all, rows_per_rank)
        _phase("barrier")
        if not rows:
            return hidden.clone()
        # the ids this rank routed itself, not the gathered copy: peers may already be writing the next
        # call's entries into the arena while this combine runs
        out = engine.combine(terms_home[:rows * engine.k_out], ids, x2d, hidden.dtype)
        _phase("combine")
        return out.reshape(batch, seq, d)

    def _fill_slot(self, x2d, weights, ids, rows, slot):
        """This rank's slot of the exchange: its rows, then padding (zero rows, zero weights, the id
        ``engine.pad_id`` that no rank executes)."""
        if rows == slot:
            return x2d, weights, ids
        torch = _torch()
        key = (slot, x2d.dtype, x2d.device)
        if rows == 0 and key in self._empty_slots:
            return self._empty_slots[key]
        k_out, d = self.engine.k_out, self.d_model
        x_slot = torch.zeros((slot, d), dtype=x2d.dtype, device=x2d.device)
        w_slot = torch.zeros((slot, k_out), dtype=torch.float32, device=x2d.device)
        ids_slot = torch.full((slot, k_out), self.engine.pad_id, dtype=torch.int64, device=x2d.device)
        if rows:
            x_slot[:rows] = x2d
            w_slot[:rows] = weights
            ids_slot[:rows] = ids
        else:
            self._empty_slots[key] = (x_slot, w_slot, ids_slot)
        return x_slot, w_slot, ids_slot


def shard_bank(bank, rank, world):
    """This rank's contiguous slice of a full ``PackedExpertBank`` (views, no copy)."""
    from .experts_inference import PackedExpertBank
    first, count = expert_partition(bank.n_experts, world)[rank]
    cut = lambda data, stride: data[first * stride:(first + count) * stride]
    return first, PackedExpertBank(cut(bank.gate, bank.gate_stride), cut(bank.up, bank.up_stride),
                                   cut(bank.down, bank.down_stride), bank.gate_type, bank.up_type, bank.down_type,
                                   count, bank.d_model, bank.d_ff)


class ExpertParallelMoEStack:
    """``x -> x + MoE(RMSNorm(x))`` per layer with expert-parallel MoE layers; the residual stream and
    the norms stay on the home rank (same chaining as ``moe_stack.PackedMoEStack``)."""

    def __init__(self, layers, norms, final_norm):
        if len(layers) != len(norms) or not layers:
            raise ValueError("one RMSNorm per MoE layer is required")
        self.layers, self.norms, self.final_norm = list(layers), list(norms), final_norm

    @property
    def packed_bytes(self):
        total = 0
        for layer in self.layers:
            total += layer.engine.bank.nbytes
            if layer.engine.shared is not None:
                total += sum(w.nbytes for w in layer.engine.shared)
        return total

    def forward(self, residual, slot_rows=None, total_rows=None):
        """residual FP32 [B, T, D] (this rank's rows, possibly none) -> (new residual, normalised
        activations); ``slot_rows`` and ``total_rows`` as in ``ExpertParallelMoELayer.forward``."""
        res = residual
        hidden = self.norms[0].forward_residual(res)
        for i, layer in enumerate(self.layers):
            branch = layer.forward(hidden, slot_rows, total_rows)
            norm = self.norms[i + 1] if i + 1 < len(self.layers) else self.final_norm
            res, hidden = norm.forward_residual_add(res, branch)
        return res, hidden

    @classmethod
    def sharded_from(cls, stack, native_banks, comm):
        """Expert-parallel twin of a single-GPU ``PackedMoEStack``: the same router weights, shared
        experts and norms, and this rank's slice of every layer's full bank (``native_banks``: the
        banks in GGUF layout the stack was built from). Its outputs equal the stack's bit for bit."""
        layers = []
        for layer, bank in zip(stack.layers, native_banks):
            first, local = shard_bank(bank, comm.rank, comm.world)
            engine = DeviceExpertEngine(local, layer.router.W_router, layer.router.k, first_expert=first,
                                        n_experts_global=bank.n_experts, shared=layer.shared_native,
                                        shared_gate=layer.shared_gate,
                                        normalization_floor=layer.router.normalization_floor)
            layers.append(ExpertParallelMoELayer(engine, comm, bank.d_model))
        return cls(layers, stack.norms, stack.final_norm)

    @classmethod
    def synthetic(cls, n_layers, comm, *, d_model=2048, d_ff=512, n_experts=512, top_k=10, shared_d_ff=512,
                  types=("Q4_K", "Q4_K", "Q6_K"), act_dtype=None, seed=0, eps=1e-5, device="cuda"):
        """Random-init stack; each rank generates only its own experts (router weights and the shared
        expert depend on the layer alone, so they are identical on every rank)."""
        from .experts_inference import synthetic_bank
        from .moe_layer import RMSNormInference
        from .quantize import random_packed
        from .quantized_linear import packed_to_device
        torch = _torch()
        act_dtype = act_dtype or torch.bfloat16
        first, count = expert_partition(n_experts, comm.world)[comm.rank]
        gen = torch.Generator(device=device)
        layers, norms = [], []
        for i in range(n_layers):
            bank = synthetic_bank(count, d_model, d_ff, types, seed=(seed * 1000 + i) * 64 + comm.rank, device=device)
            gen.manual_seed(seed * 1000 + i)
            w_router = torch.empty((d_model, n_experts), dtype=torch.float32, device=device)
            w_router.normal_(0.0, 0.02, generator=gen)
            shared = None
            if shared_d_ff:
                shared = tuple(packed_to_device(random_packed(fmt, shape, seed=seed * 7919 + 3 * i + j,
                                                              d=1.0 / 2048, dmin=1.0 / 4096))
                               for j, (fmt, shape) in enumerate(zip(types, ((shared_d_ff, d_model),
                                                                             (shared_d_ff, d_model),
                                                                             (d_model, shared_d_ff)))))
            engine = DeviceExpertEngine(bank, w_router, top_k, first_expert=first, n_experts_global=n_experts,
                                        shared=shared)
            layers.append(ExpertParallelMoELayer(engine, comm, d_model))
            norm = RMSNormInference(d_model, eps=eps)
            norm.set_weights(torch.ones(d_model, dtype=act_dtype, device=device))
            norms.append(norm)
        final = RMSNormInference(d_model, eps=eps)
        final.set_weights(torch.ones(d_model, dtype=act_dtype, device=device))
        return cls(layers, norms, final)
