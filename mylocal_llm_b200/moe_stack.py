"""A stack of packed MoE layers with RMSNorm and an FP32 residual stream (decode-step harness).

Each layer is ``x -> x + MoE(RMSNorm(x))``: the residual stream is FP32, the normalised branch input
and the MoE output are BF16 (or FP32), and the residual add of layer i is fused into the RMSNorm
of layer i+1 (``residual_add_rmsnorm``), as the reference's low-precision engine chains them
(``mini_llm/blocks/transformer_block_inference.py:344-364``,
``mini_llm/ops/rmsnorm_inference.py:525-539``). Token mixing is the identity, which isolates the
quantized path exactly as the 48-layer benchmark configuration prescribes.
"""

import ctypes
import os

from . import _lib
from .experts_inference import ResidentExpertExecutor, synthetic_bank
from .moe_layer import PackedMoELayer, RMSNormInference
from .quantize import random_packed
from .quantized_linear import packed_to_device


def _torch():
    import torch
    return torch


class PackedMoEStack:
    def __init__(self, layers, norms, final_norm):
        if len(layers) != len(norms) or not layers:
            raise ValueError("one RMSNorm per MoE layer is required")
        self.layers, self.norms, self.final_norm = list(layers), list(norms), final_norm
        # B200Q_FUSE_NORM=1: combine + residual add + RMSNorm in one kernel where the layer allows. Off by
        # default: one CTA per row has less parallelism than the two kernels it replaces and measured slower
        # (1 token: 384 vs 425 tokens/s on the 48-layer stack; 64 tokens: 5019 vs 5069); the results are the same.
        self.fuse_residual_norm = os.environ.get("B200Q_FUSE_NORM", "0") == "1"
        # One-token steps run as one persistent kernel over all layers when the stack qualifies
        # (``B200Q_PERSISTENT=0``: always the chain of launches; the results are the same bits).
        self.persistent_step = os.environ.get("B200Q_PERSISTENT", "1") != "0"
        self._persistent = None           # (layer table, workspace, call arguments) or False once found unfit

    @property
    def packed_bytes(self):
        total = 0
        for layer in self.layers:
            total += layer.bank.nbytes
            if layer.shared is not None:
                total += sum(w.nbytes for w in layer.shared)
        return total

    def _persistent_setup(self):
        """Layer table and workspace of ``b200q_moe_decode_stack`` if every layer fits it: resident executor,
        routed and shared experts behind 16-byte aligned pointer tables, no router bias, no shared gate, one
        shape / format / top-k / floor for all layers, norm weights of one 16-bit type."""
        torch = _torch()
        first = self.layers[0]
        bank = first.bank
        norms = list(self.norms) + [self.final_norm]
        dtypes = {n.gamma.dtype for n in norms}
        key = lambda l: (l.bank.d_model, l.bank.d_ff, l.bank.n_experts, l.router.k, l.router.normalization_floor,
                         l.bank.gate_type, l.bank.up_type, l.bank.down_type)
        fits = (len(dtypes) == 1 and next(iter(dtypes)) in (torch.bfloat16, torch.float16)
                and len({n.eps for n in norms}) == 1
                and all(isinstance(l.executor, ResidentExpertExecutor) and l._tables is not None and l._tables[1]
                        and l.shared_gate is None and l.router.b_router is None and l.fuse_row_plan
                        and l.router._w_expert_major is not None and l.router._w_expert_major.data_ptr() % 16 == 0
                        and key(l) == key(first) for l in self.layers)
                and bank.gate_type == bank.up_type and bank.gate_type in ("Q4_K", "Q4_K_TILED")
                and bank.down_type == "Q6_K_TILED" and bank.n_experts <= 1024 and first.router.k <= 15
                and bank.d_model % 256 == 0 and bank.d_ff % 256 == 0)
        if not fits:
            return False
        rows = []
        for i, layer in enumerate(self.layers):
            tables = layer._tables[0]
            rows.append([layer.router._w_expert_major.data_ptr(), tables[0].data_ptr(), tables[1].data_ptr(),
                         tables[2].data_ptr(), norms[i + 1].gamma.data_ptr()])
        device = first.router._w_expert_major.device
        table = torch.tensor(rows, dtype=torch.int64, device=device)
        d, f, e, k = bank.d_model, bank.d_ff, bank.n_experts, first.router.k
        nbytes = int(_lib.load().b200q_moe_decode_stack_workspace(d, f, e, k))
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return table, workspace, (d, f, e, k)

    def forward_one_token(self, residual):
        """The step for a single row as one persistent kernel, or ``None`` when the stack does not fit it."""
        torch = _torch()
        if self._persistent is None:
            self._persistent = self._persistent_setup()
        if not self._persistent:
            return None
        table, workspace, (d, f, e, k) = self._persistent
        if not residual.is_contiguous() or residual.dtype != torch.float32 or residual.device != table.device:
            return None
        first, gamma0 = self.layers[0], self.norms[0].gamma
        res = torch.empty_like(residual)
        hidden = torch.empty(residual.shape, dtype=gamma0.dtype, device=residual.device)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        try:
            _lib.call("b200q_moe_decode_stack", ptr(table), len(self.layers), d, f, e, k, 1,
                      float(first.router.normalization_floor), _lib.FORMAT_ID[first.bank.gate_type],
                      _lib.FORMAT_ID[first.bank.down_type], ptr(gamma0),
                      _lib.DTYPE_ID[str(gamma0.dtype).replace("torch.", "")], float(self.norms[0].eps), ptr(residual),
                      ptr(res), ptr(hidden), ptr(workspace), int(workspace.numel()), _lib.current_stream())
        except NotImplementedError:
            self._persistent = False
            return None
        return res, hidden

    def stage_times(self):
        """Microseconds the stages of the last layer took in the latest persistent step (router, barrier, top-k +
        plan, gate/up, barrier, down, barrier, combine + norm), as seen by one CTA; needs ``B200Q_STAGE_TIMES=1``
        in the environment of that step. ``None`` when no such step ran."""
        if not self._persistent:
            return None
        workspace = self._persistent[1]
        raw = workspace[workspace.numel() - 192: workspace.numel() - 192 + 72].cpu().numpy().view("int64")
        if raw[0] == 0 or raw[8] < raw[0]:
            return None
        names = ("router", "barrier_1", "topk_plan", "gate_up", "barrier_2", "down", "barrier_3", "combine_norm")
        return {n: round(float(raw[i + 1] - raw[i]) / 1e3, 2) for i, n in enumerate(names)}

    def forward(self, residual, trace=None):
        """residual FP32 [B, T, D] -> (new residual FP32, final normalised activations). ``trace``: a list
        that receives, per layer, ``(layer input, layer output)`` - the tensors a layer-by-layer check
        against a reference needs; it forces the two-kernel combine + norm."""
        if trace is None and self.persistent_step and residual.ndim == 3 and residual.shape[0] * residual.shape[1] == 1:
            out = self.forward_one_token(residual)
            if out is not None:
                return out
        res = residual
        hidden = self.norms[0].forward_residual(res)
        for i, layer in enumerate(self.layers):
            norm = self.norms[i + 1] if i + 1 < len(self.layers) else self.final_norm
            if trace is None and self.fuse_residual_norm and layer.can_fuse_residual_norm():
                res, hidden = layer.forward(hidden, residual_norm=(norm, res))
            else:
                branch = layer.forward(hidden)
                if trace is not None:
                    trace.append((hidden, branch))
                res, hidden = norm.forward_residual_add(res, branch)
        return res, hidden

    @classmethod
    def synthetic(cls, n_layers, *, d_model=2048, d_ff=512, n_experts=512, top_k=10, shared_d_ff=512,
                  types=("Q4_K", "Q4_K", "Q6_K"), act_dtype=None, seed=0, eps=1e-5, device="cuda", keep_native=False):
        """Random-init stack with the benchmark shape; weights are generated on the device.
        ``keep_native`` keeps the banks in GGUF layout as ``stack.native_banks`` (the layers convert
        theirs to the tile layouts), e.g. to shard the same weights over several ranks."""
        torch = _torch()
        act_dtype = act_dtype or torch.bfloat16
        gen = torch.Generator(device=device)
        layers, norms, native = [], [], []
        for i in range(n_layers):
            bank = synthetic_bank(n_experts, d_model, d_ff, types, seed=seed * 1000 + i, device=device)
            if keep_native:
                native.append(bank)
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
            layers.append(PackedMoELayer(bank, w_router, top_k, shared=shared, layer_id=i))
            norm = RMSNormInference(d_model, eps=eps)
            norm.set_weights(torch.ones(d_model, dtype=act_dtype, device=device))
            norms.append(norm)
        final = RMSNormInference(d_model, eps=eps)
        final.set_weights(torch.ones(d_model, dtype=act_dtype, device=device))
        stack = cls(layers, norms, final)
        stack.native_banks = native
        return stack
