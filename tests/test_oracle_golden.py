"""Pin the CPU oracle (NumPy and plain-C restatements) before anything trusts it.

Sources of truth, in order:
  1. hand-packed known-answer blocks, the same cases the reference's tests hold;
  2. golden vectors produced by running the reference itself (tests/golden/make_golden.py);
  3. the independent ``gguf`` package decoder, when installed;
  4. the reference's own C++ CPU library compiled into oracle/_ref, when it was built.
"""

import numpy as np
import pytest

from oracle import packed_oracle as po
from oracle import build_oracle as bo

FORMATS = ("Q8_0", "Q4_0", "Q3_K", "Q4_K", "Q5_K", "Q6_K")


def f16(value):
    return np.array([value], dtype="<f2").view(np.uint8).tobytes()


def c_dequantize(data, shape, fmt):
    lib, _, _ = bo.load_port()
    data = np.ascontiguousarray(data, np.uint8)
    n = int(np.prod(shape[:-1]))
    out = np.empty((n, shape[-1]), np.float32)
    rc = lib.oracle_dequantize(data.ctypes.data, bo.FORMAT_ID[fmt], n, shape[-1], out.ctypes.data)
    assert rc == 0
    return out.reshape(shape)


def both_decoders(data, shape, fmt):
    a = po.dequantize(data, shape, fmt)
    b = c_dequantize(data, shape, fmt)
    np.testing.assert_array_equal(a, b)
    return a


# ------------------------------------------------------------------ 1. hand-packed known answers
def test_q8_0_known_answer():
    # reference: tests/test_0085f_external_gguf.py:91-96
    block = np.arange(-16, 16, dtype=np.int8)
    raw = np.frombuffer(f16(0.25) + block.tobytes(), np.uint8)
    np.testing.assert_array_equal(both_decoders(raw, (1, 32), "Q8_0")[0], block * 0.25)


def test_q4_k_known_answer_scales_and_nibble_order():
    # reference: tests/test_0106a_packed_gguf.py:26-33
    raw = f16(1) + f16(0) + bytes([1] * 4 + [0] * 8) + bytes([0x12] * 128)
    expected = np.array(([2.0] * 32 + [1.0] * 32) * 2 + [0] * 128)
    np.testing.assert_array_equal(both_decoders(np.frombuffer(raw, np.uint8), (1, 256), "Q4_K").ravel(), expected)


def test_q5_k_known_answer_high_bits_and_minima():
    # reference: tests/test_0106g_q5k_packed.py:23-45
    raw = bytearray(176)
    raw[:2] = np.float16(.5).tobytes()
    raw[2:4] = np.float16(.25).tobytes()
    raw[4] = 1
    raw[8] = 1
    raw[16:48] = bytes([1] * 32)
    raw[48:176] = bytes([0x21] * 128)
    got = both_decoders(np.frombuffer(bytes(raw), np.uint8), (1, 256), "Q5_K").ravel()
    np.testing.assert_array_equal(got[:32], np.full(32, 8.25))
    np.testing.assert_array_equal(got[32:], np.zeros(224))
    raw[16:48] = bytes([0x80] * 32)
    raw[4:16] = bytes([0] * 12)
    raw[15] = 0x01
    got = both_decoders(np.frombuffer(bytes(raw), np.uint8), (1, 256), "Q5_K").ravel()
    np.testing.assert_array_equal(got[:224], np.zeros(224))
    np.testing.assert_array_equal(got[224:], np.full(32, .5 * 18))


def q6_all_lanes_block():
    quants = np.tile(np.arange(-32, 32, dtype=np.int16), 4)
    scales = np.array([-128, -64, -32, -16, -1, 0, 1, 2, 3, 7, 16, 31, 63, 100, 126, 127], dtype=np.int8)
    raw = bytearray(210)
    for half in range(2):
        for lane in range(32):
            q = [int(v) + 32 for v in quants[half * 128 + lane::32][:4]]
            raw[half * 64 + lane] = q[0] & 15 | ((q[2] & 15) << 4)
            raw[half * 64 + lane + 32] = q[1] & 15 | ((q[3] & 15) << 4)
            raw[128 + half * 32 + lane] = sum((q[g] >> 4) << (2 * g) for g in range(4))
    raw[192:208] = scales.tobytes()
    raw[208:210] = np.float16(.03125).tobytes()
    expected = .03125 * np.repeat(scales.astype(np.float32), 16) * quants
    return np.frombuffer(bytes(raw), np.uint8), expected.astype(np.float32)


def test_q6_k_known_answer_all_lanes_and_signed_scales():
    # reference: tests/test_0106l_q6k_packed.py:25-46
    raw, expected = q6_all_lanes_block()
    np.testing.assert_array_equal(both_decoders(raw, (1, 256), "Q6_K").ravel(), expected)
    # identity activations read back every coefficient through the C GEMV as well
    y = bo.cpu_gemv(bo.load_port(), raw, "Q6_K", 1, 256, np.eye(256, dtype=np.float32))
    np.testing.assert_array_equal(y.ravel(), expected)


# ------------------------------------------------------------------ 2. reference-generated golden
@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("kind", ["random", "quant"])
def test_dequantize_matches_reference_bit_for_bit(golden, fmt, kind):
    data = golden[f"deq_{fmt}_{kind}_bytes"]
    shape = tuple(golden[f"deq_{fmt}_{kind}_shape"])
    np.testing.assert_array_equal(both_decoders(data, shape, fmt), golden[f"deq_{fmt}_{kind}_out"])


@pytest.mark.parametrize("fmt", FORMATS)
def test_quantiser_fixture_is_close_to_its_source(golden, fmt):
    src, out = golden[f"deq_{fmt}_quant_src"], golden[f"deq_{fmt}_quant_out"]
    bound = {"Q8_0": 0.005, "Q4_0": 0.14, "Q3_K": 0.3, "Q4_K": 0.08, "Q5_K": 0.04, "Q6_K": 0.03}[fmt]
    assert np.abs(out - src).max() <= bound * np.abs(src).max()


@pytest.mark.parametrize("fmt", FORMATS)
def test_linear_oracles_match_reference_outputs(golden, fmt):
    data, shape, x = golden[f"lin_{fmt}_bytes"], tuple(golden[f"lin_{fmt}_shape"]), golden[f"lin_{fmt}_x"]
    y64 = po.linear_fp64(x, data, shape, fmt)
    # the reference's own tolerance for its CPU operator (tests/test_0106b_quantized_linear.py:44)
    np.testing.assert_allclose(golden[f"lin_{fmt}_y_numpy"], y64, rtol=1e-6, atol=2e-4)
    np.testing.assert_allclose(golden[f"lin_{fmt}_y_native"], y64, rtol=1e-5, atol=2e-4)
    yc = bo.cpu_gemv(bo.load_port(), data, fmt, shape[0], shape[1], x)
    np.testing.assert_allclose(yc, y64, rtol=1e-5, atol=2e-4)


def test_ffn_oracle_matches_reference(golden):
    d, f = (int(v) for v in golden["ffn_dims"])
    gate = (golden["ffn_gate_bytes"], (f, d), "Q4_K")
    up = (golden["ffn_up_bytes"], (f, d), "Q5_K")
    down = (golden["ffn_down_bytes"], (d, f), "Q6_K")
    x = golden["ffn_x"]
    np.testing.assert_allclose(golden["ffn_swiglu"], po.swiglu_fp64(x, gate, up), rtol=3e-4, atol=2e-4)
    np.testing.assert_allclose(golden["ffn_out"], po.expert_ffn_fp64(x, gate, up, down), rtol=2e-4, atol=2e-5)
    yc = bo.cpu_expert(bo.load_port(), (gate[0], "Q4_K"), (up[0], "Q5_K"), (down[0], "Q6_K"), d, f, x)
    np.testing.assert_allclose(yc, golden["ffn_out"], rtol=2e-4, atol=2e-5)


def test_router_oracle_matches_reference(golden):
    logits, k = golden["router_logits"], int(golden["router_k"])
    w, ids = po.router_topk(logits, k, None)
    np.testing.assert_array_equal(ids, golden["router_ids"])
    np.testing.assert_allclose(w, golden["router_w_raw"], rtol=2e-6, atol=2e-7)
    # projected + renormalised with the 2^-14 floor
    lg = golden["router_fw_x"].astype(np.float64) @ golden["router_fw_W"].astype(np.float64)
    w2, ids2 = po.router_topk(lg, k, 2.0 ** -14)
    np.testing.assert_array_equal(ids2, golden["router_fw_ids"])
    np.testing.assert_allclose(w2, golden["router_fw_w"], rtol=2e-6, atol=2e-7)
    # FP32 row kernel restatement agrees on ids exactly and weights to 2e-7
    lg32 = (golden["router_fw_x"] @ golden["router_fw_W"]).astype(np.float32)
    w3, ids3 = po.router_topk_rows_fp32(lg32, k, 2.0 ** -14)
    np.testing.assert_array_equal(ids3, golden["router_fw_ids"])
    np.testing.assert_allclose(w3, golden["router_fw_w"], rtol=0, atol=2e-7)


def test_router_rows_tie_nan_inf_table():
    # the table of tests/test_0106v_router_decode.py:28-62: ties -> lower id, NaN last
    rows = np.array([[1, 1, 1, 1], [0, np.inf, -np.inf, 5], [np.nan, 2, 2, 1], [3, np.nan, np.nan, 3]], np.float32)
    _, ids = po.router_topk_rows_fp32(rows, 3, 2.0 ** -14)
    np.testing.assert_array_equal(ids, [[0, 1, 2], [1, 3, 0], [1, 2, 3], [0, 3, 1]])


def test_routing_plan_oracle_matches_reference(golden):
    ids = golden["plan_ids"]
    order, counts, offsets = po.routing_plan(ids, 9)
    np.testing.assert_array_equal(counts, golden["plan_sizes"])
    np.testing.assert_array_equal(offsets, golden["plan_offsets"])
    np.testing.assert_array_equal(ids.reshape(-1)[order], golden["plan_expert_sorted"])
    # within an expert the reference's argsort may order tokens differently; compare as sets
    for e in range(9):
        mine = np.sort(order[offsets[e]:offsets[e + 1]] // 3)
        theirs = np.sort(golden["plan_token_sorted"][offsets[e]:offsets[e + 1]])
        np.testing.assert_array_equal(mine, theirs)


@pytest.mark.parametrize("tag", ["moe", "moe1"])
def test_moe_dispatch_oracle_matches_reference(golden, tag):
    d, f, e, k = (int(v) for v in golden["moe_dims"])
    experts = [((golden["moe_gate_bytes"][i], (f, d), "Q4_K"), (golden["moe_up_bytes"][i], (f, d), "Q4_K"),
                (golden["moe_down_bytes"][i], (d, f), "Q6_K")) for i in range(e)]
    hidden = golden[f"{tag}_hidden"]
    w, ids = po.router_topk(hidden.astype(np.float64) @ golden["moe_router_W"].astype(np.float64), k, 2.0 ** -14)
    np.testing.assert_array_equal(ids, golden[f"{tag}_ids"])
    np.testing.assert_allclose(w, golden[f"{tag}_weights"], rtol=3e-6, atol=3e-7)
    routed = po.experts_forward_fp32sum(
        hidden, golden[f"{tag}_weights"], golden[f"{tag}_ids"],
        lambda ex, rows: po.expert_ffn_fp64(rows, *experts[ex]), e)
    # the reference's own MoE tolerance (tests/test_0106o_qwen3next_decoder.py:192) is 3e-5/2e-6
    # against FP64; its native CPU kernels accumulate in FP32, hence the wider band here.
    np.testing.assert_allclose(routed, golden[f"{tag}_routed"], rtol=4e-4, atol=8e-6)


def test_rmsnorm_oracle_matches_reference(golden):
    y = po.rmsnorm_fp64(golden["rms_x"], golden["rms_gamma"], float(golden["rms_eps"]))
    np.testing.assert_allclose(y, golden["rms_y"], rtol=2e-6, atol=1e-6)
    res, y2 = po.residual_rmsnorm_fp64(golden["rms_x"], golden["rms_branch"], golden["rms_gamma"],
                                       float(golden["rms_eps"]), 0.5)
    np.testing.assert_allclose(res, golden["rms_res_out"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(y2, golden["rms_res_y"], rtol=3e-6, atol=2e-6)


# ------------------------------------------------------------------ 3. independent gguf decoder
@pytest.mark.parametrize("fmt", FORMATS)
def test_against_gguf_package_decoder(fmt):
    gguf = pytest.importorskip("gguf")
    from gguf.quants import dequantize
    from mylocal_llm_b200.quantize import random_packed
    qk, qb = po.BLOCKS[fmt]
    w = random_packed(fmt, (7, 4 * qk), seed=1606)
    expected = dequantize(w.data.reshape(7, -1), gguf.GGMLQuantizationType[fmt])
    np.testing.assert_array_equal(both_decoders(w.data, w.shape, fmt), expected)


# ------------------------------------------------------------------ 4. the reference's own C++ library
@pytest.mark.parametrize("fmt", FORMATS)
def test_port_matches_reference_cpu_library(fmt):
    ref = bo.load_ref()
    if ref is None:
        pytest.skip("oracle/_ref was not built (no reference tree on this machine)")
    from mylocal_llm_b200.quantize import random_packed
    qk, _ = po.BLOCKS[fmt]
    n, k = 19, 3 * qk if qk == 256 else 160
    w = random_packed(fmt, (n, k), seed=5)
    x = np.random.default_rng(6).normal(0, 1, (3, k)).astype(np.float32)
    y_ref = bo.cpu_gemv(ref, w.data, fmt, n, k, x)
    y_port = bo.cpu_gemv(bo.load_port(), w.data, fmt, n, k, x)
    np.testing.assert_allclose(y_port, y_ref, rtol=2e-5, atol=2e-4)
    np.testing.assert_allclose(y_ref, po.linear_fp64(x, w.data, w.shape, fmt), rtol=2e-5, atol=2e-4)


def test_cpu_libraries_reject_bad_arguments():
    lib, gemv, expert = bo.load_port()
    buf = np.zeros(256, np.uint8)
    out = np.zeros(8, np.float32)
    assert gemv(buf.ctypes.data, 2, 1, 255, out.ctypes.data, 1, out.ctypes.data) == 1   # K not block aligned
    assert gemv(buf.ctypes.data, 7, 1, 256, out.ctypes.data, 1, out.ctypes.data) == 1   # unknown format
    assert gemv(None, 2, 1, 256, out.ctypes.data, 1, out.ctypes.data) == 1
