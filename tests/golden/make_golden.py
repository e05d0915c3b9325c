"""Generate the committed golden vectors by running the REFERENCE implementation.

Run where the reference tree is available (its location: ``MYLOCAL_REFERENCE_ROOT``):

    python tests/golden/make_golden.py

The script imports the reference with its NumPy backend, feeds it seeded packed bytes and
activations, and stores inputs and the reference's outputs in ``tests/golden/*.npz``. The tests
only read the ``.npz`` files, so they run on machines that do not have the reference.

What is recorded (reference entry point -> key prefix):
  PackedGGUFWeight.dequantize_reference                     -> deq_<fmt>
  quantized_linear(cpu_packed_backend="reference"|"native") -> lin_<fmt>
  quantized_swiglu / PackedExpertFFNInference.forward       -> ffn
  expert_topk_forward + RouterInference renormalisation     -> router
  RoutingPlan.from_router_outputs                           -> plan
  RouterInference + ExpertsInference + HeterogeneousExpertExecutor (native CPU) -> moe
  RMSNormInference.forward / forward_residual_add           -> rms
"""

import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REFERENCE = Path(os.environ.get("MYLOCAL_REFERENCE_ROOT") or REPO.parent / "reference")

os.environ["MINI_LLM_BACKEND"] = "numpy"
os.environ.setdefault("MINI_LLM_NATIVE_BUILD_DIR", tempfile.mkdtemp(prefix="ref_native_"))
sys.dont_write_bytecode = True
sys.path.insert(0, str(REFERENCE))
sys.path.insert(0, str(REPO))

from mini_llm.ops.quantized_weight import PackedGGUFWeight as RefPacked  # noqa: E402
from mini_llm.ops.quantized_linear import (  # noqa: E402
    quantized_linear as ref_linear, quantized_swiglu as ref_swiglu, PackedExpertFFNInference as RefFFN)
from mini_llm.ops.router import expert_topk_forward  # noqa: E402
from mini_llm.ops.router_inference import RouterInference as RefRouter  # noqa: E402
from mini_llm.ops.routing_plan import RoutingPlan as RefPlan  # noqa: E402
from mini_llm.ops.experts_inference import ExpertsInference as RefExperts  # noqa: E402
from mini_llm.ops.expert_residency import ExpertKey, HeterogeneousExpertExecutor  # noqa: E402
from mini_llm.ops.rmsnorm_inference import RMSNormInference as RefRMSNorm  # noqa: E402

from mylocal_llm_b200.quantize import quantize, random_packed  # noqa: E402

FORMATS = ("Q8_0", "Q4_K", "Q5_K", "Q6_K")


def ref_weight(p):
    return RefPacked(p.data, p.shape, p.quant_type)


def main():
    out = {}
    rng = np.random.default_rng(20240)

    # --- decoders: random-byte blocks (every bit pattern) and quantised normal weights
    for fmt in FORMATS:
        k = 64 if fmt == "Q8_0" else 512
        rnd = random_packed(fmt, (5, k), seed=1000 + len(fmt) + ord(fmt[1]))
        out[f"deq_{fmt}_random_bytes"] = rnd.data.copy()
        out[f"deq_{fmt}_random_shape"] = np.asarray(rnd.shape)
        out[f"deq_{fmt}_random_out"] = ref_weight(rnd).dequantize_reference()
        w = rng.normal(0, 0.02, (3, k)).astype(np.float32)
        qz = quantize(w, fmt)
        out[f"deq_{fmt}_quant_bytes"] = qz.data.copy()
        out[f"deq_{fmt}_quant_shape"] = np.asarray(qz.shape)
        out[f"deq_{fmt}_quant_src"] = w
        out[f"deq_{fmt}_quant_out"] = ref_weight(qz).dequantize_reference()

    # --- linear: both reference CPU back ends, tails in N and M
    for fmt in FORMATS:
        n, k, m = 13, 768 if fmt != "Q8_0" else 96, 3
        wq = random_packed(fmt, (n, k), seed=77 + ord(fmt[1]))
        x = rng.normal(0, 1, (m, k)).astype(np.float32)
        out[f"lin_{fmt}_bytes"] = wq.data.copy()
        out[f"lin_{fmt}_shape"] = np.asarray(wq.shape)
        out[f"lin_{fmt}_x"] = x
        out[f"lin_{fmt}_y_numpy"] = ref_linear(x, ref_weight(wq), cpu_packed_backend="reference")
        out[f"lin_{fmt}_y_native"] = ref_linear(x, ref_weight(wq), cpu_packed_backend="native")

    # --- SwiGLU + expert FFN with mixed formats (gate Q4_K, up Q5_K, down Q6_K)
    d, f, m = 512, 256, 2
    gate = quantize(rng.normal(0, 0.05, (f, d)).astype(np.float32), "Q4_K")
    up = quantize(rng.normal(0, 0.05, (f, d)).astype(np.float32), "Q5_K")
    down = quantize(rng.normal(0, 0.05, (d, f)).astype(np.float32), "Q6_K")
    x = rng.normal(0, 1, (m, d)).astype(np.float32)
    out["ffn_gate_bytes"], out["ffn_up_bytes"], out["ffn_down_bytes"] = gate.data.copy(), up.data.copy(), down.data.copy()
    out["ffn_dims"] = np.asarray([d, f])
    out["ffn_x"] = x
    out["ffn_swiglu"] = ref_swiglu(x, ref_weight(gate), ref_weight(up))
    out["ffn_out"] = RefFFN(ref_weight(gate), ref_weight(up), ref_weight(down)).forward(x)

    # --- router: raw selected probabilities, and renormalised with the 2^-14 floor; ties included
    logits = rng.normal(0, 2, (7, 24)).astype(np.float32)
    logits[1, 5] = logits[1, 9] = logits[1].max() + 1          # tie for the top slot
    logits[2, :] = 0.25                                         # all equal
    logits[3, 0] = -np.inf
    k = 4
    w_raw, ids, _ = expert_topk_forward(logits[None], k, output_dtype=None, return_cache=False)
    out["router_logits"] = logits
    out["router_k"] = np.asarray(k)
    out["router_ids"] = ids[0].astype(np.int64)
    out["router_w_raw"] = w_raw[0]
    router = RefRouter(16, 24, k, renormalize_selected=True, normalization_floor=2.0 ** -14)
    router.W_router = rng.normal(0, 0.3, (16, 24)).astype(np.float32)
    router.b_router = np.zeros(24, np.float32)
    xr = rng.normal(0, 1, (1, 6, 16)).astype(np.float32)
    rw, rids = router.forward(xr)
    out["router_fw_W"], out["router_fw_x"] = router.W_router, xr[0]
    out["router_fw_w"], out["router_fw_ids"] = rw[0], rids[0].astype(np.int64)

    # --- routing plan
    plan_ids = rng.integers(0, 9, (1, 11, 3))
    plan_w = rng.random((1, 11, 3)).astype(np.float32)
    plan = RefPlan.from_router_outputs(plan_ids, plan_w, 3, n_experts=9)
    out["plan_ids"] = plan_ids[0].astype(np.int64)
    out["plan_sizes"] = np.asarray(plan.expert_sizes)
    out["plan_offsets"] = np.asarray(plan.expert_offsets)
    out["plan_expert_sorted"] = np.asarray(plan.expert_indices)
    out["plan_token_sorted"] = np.asarray(plan.token_indices)

    # --- MoE dispatch: router + experts on the reference's native CPU back end
    d, f, e, k, t = 256, 256, 6, 3, 5
    bank = {}
    blobs = {}
    for ex in range(e):
        g = quantize(rng.normal(0, 0.06, (f, d)).astype(np.float32), "Q4_K")
        u = quantize(rng.normal(0, 0.06, (f, d)).astype(np.float32), "Q4_K")
        dn = quantize(rng.normal(0, 0.06, (d, f)).astype(np.float32), "Q6_K")
        bank[ExpertKey("golden", 0, ex)] = (ref_weight(g), ref_weight(u), ref_weight(dn))
        blobs[ex] = (g.data.copy(), u.data.copy(), dn.data.copy())
    executor = HeterogeneousExpertExecutor(bank.__getitem__, model_id="golden", d_model=d, d_ff=f,
                                           device_budget_bytes=0, compute_dtype="float32",
                                           cpu_packed_backend="native")
    router = RefRouter(d, e, k, renormalize_selected=True, normalization_floor=2.0 ** -14)
    router.W_router = rng.normal(0, 0.1, (d, e)).astype(np.float32)
    router.b_router = np.zeros(e, np.float32)
    experts = RefExperts(d, f, e, expert_executor=executor, layer_id=0)
    for tokens, tag in ((t, "moe"), (1, "moe1")):
        hidden = rng.normal(0, 1, (1, tokens, d)).astype(np.float32)
        weights, ids = router.forward(hidden)
        routed = experts.forward(hidden, weights, ids)
        out[f"{tag}_hidden"], out[f"{tag}_weights"] = hidden[0], weights[0]
        out[f"{tag}_ids"], out[f"{tag}_routed"] = ids[0].astype(np.int64), routed[0]
    out["moe_dims"] = np.asarray([d, f, e, k])
    out["moe_router_W"] = router.W_router
    out["moe_gate_bytes"] = np.stack([blobs[i][0] for i in range(e)])
    out["moe_up_bytes"] = np.stack([blobs[i][1] for i in range(e)])
    out["moe_down_bytes"] = np.stack([blobs[i][2] for i in range(e)])

    # --- RMSNorm and residual-add + RMSNorm
    xn = rng.normal(0, 1.5, (4, 320)).astype(np.float32)
    gamma = np.linspace(0.65, 1.45, 320, dtype=np.float32)
    eps = np.float32(1e-5)
    out["rms_x"], out["rms_gamma"], out["rms_eps"] = xn, gamma, np.asarray(eps)
    norm = RefRMSNorm(320, eps=float(eps))
    norm.set_weights(gamma)
    out["rms_y"] = norm.forward(xn)
    branch = rng.normal(0, 0.5, (4, 320)).astype(np.float32)
    res_out, y_res = norm.forward_residual_add(xn, branch, alpha=0.5)
    out["rms_branch"], out["rms_res_out"], out["rms_res_y"] = branch, res_out, y_res

    path = HERE / "packed_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path, path.stat().st_size, "bytes,", len(out), "arrays")


def legacy_formats():
    """Q4_0 and Q3_K (the two remaining FP32-lane formats of the reference's packed GPU path): decoder and
    linear fixtures, written to a file of their own so the first file's arrays keep their values."""
    out = {}
    rng = np.random.default_rng(4103)
    for fmt in ("Q4_0", "Q3_K"):
        k = 64 if fmt == "Q4_0" else 512
        rnd = random_packed(fmt, (5, k), seed=2000 + ord(fmt[1]))
        out[f"deq_{fmt}_random_bytes"] = rnd.data.copy()
        out[f"deq_{fmt}_random_shape"] = np.asarray(rnd.shape)
        out[f"deq_{fmt}_random_out"] = ref_weight(rnd).dequantize_reference()
        w = rng.normal(0, 0.02, (3, k)).astype(np.float32)
        qz = quantize(w, fmt)
        out[f"deq_{fmt}_quant_bytes"] = qz.data.copy()
        out[f"deq_{fmt}_quant_shape"] = np.asarray(qz.shape)
        out[f"deq_{fmt}_quant_src"] = w
        out[f"deq_{fmt}_quant_out"] = ref_weight(qz).dequantize_reference()
        n, k, m = 13, 768 if fmt != "Q4_0" else 96, 3
        wq = random_packed(fmt, (n, k), seed=88 + ord(fmt[1]))
        x = rng.normal(0, 1, (m, k)).astype(np.float32)
        out[f"lin_{fmt}_bytes"] = wq.data.copy()
        out[f"lin_{fmt}_shape"] = np.asarray(wq.shape)
        out[f"lin_{fmt}_x"] = x
        out[f"lin_{fmt}_y_numpy"] = ref_linear(x, ref_weight(wq), cpu_packed_backend="reference")
        out[f"lin_{fmt}_y_native"] = ref_linear(x, ref_weight(wq), cpu_packed_backend="native")
    path = HERE / "legacy_formats_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path, path.stat().st_size, "bytes,", len(out), "arrays")


LLAMA_CONFIG = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64, vocab_size=256, max_position_embeddings=64,
                    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)


def llama():
    """The reference's ExternalLlamaModel (mini_llm/external/llama_model.py, NumPy backend, FP32) on Q8_0
    weights: every matrix is quantised to Q8_0, and the reference is fed what its GGUF reader hands it for
    such a tensor - the dequantised dense FP32 matrix (mini_llm/external/gguf_loader.py). Stored: the packed
    bytes, the norm vectors, a prompt, the logits of the prompt's last position and of three greedy
    decode steps."""
    from mini_llm.external import ExternalLlamaModel as RefLlama
    from mini_llm.external.config import ExternalLlamaConfig as RefConfig
    cfg = RefConfig(**LLAMA_CONFIG)
    model = RefLlama(cfg, dtype="float32")
    rng = np.random.default_rng(85)
    out, dense = {}, {}
    for name, shape in model.expected_shapes().items():
        if name.endswith("norm.weight") or "layernorm.weight" in name:
            dense[name] = (np.ones(shape, dtype=np.float32) + 0.025 * rng.normal(size=shape)).astype(np.float32)
            out["norm:" + name] = dense[name]
        else:
            packed = quantize((rng.normal(size=shape) * 0.07).astype(np.float32), "Q8_0")
            out["q8:" + name] = packed.data.copy()
            dense[name] = ref_weight(packed).dequantize_reference()
    model.set_weights(dense)
    prompt = rng.integers(0, cfg.vocab_size, (1, 12))
    state = model.create_generation_state(1, 32)
    logits = np.asarray(model.prefill(prompt, state), dtype=np.float32)
    logits = logits.reshape(-1, cfg.vocab_size)[-1]
    steps, tokens = [logits], []
    for _ in range(3):
        token = int(np.argmax(steps[-1]))
        tokens.append(token)
        step = np.asarray(model.decode_one(np.asarray([[token]]), state), dtype=np.float32)
        steps.append(step.reshape(-1, cfg.vocab_size)[-1])
    out["prompt"] = prompt.astype(np.int64)
    out["greedy_tokens"] = np.asarray(tokens, np.int64)
    out["logits"] = np.stack(steps)                      # [4, vocab]: prompt's last position, then three decode steps
    path = HERE / "llama_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path, path.stat().st_size, "bytes,", len(out), "arrays; logits rms", float(np.sqrt((out["logits"] ** 2).mean())))


if __name__ == "__main__":
    which = sys.argv[1:] or ["packed", "legacy", "llama"]
    if "packed" in which:
        main()
    if "legacy" in which:
        legacy_formats()
    if "llama" in which:
        llama()
