"""GGUF file seam on CPU: index, zero-copy packed views, fused gate/up split, packed Q/K row permutation."""

import numpy as np
import pytest

from mylocal_llm_b200.gguf_index import (GGUFPackedIndex, decode_dense, restore_hf_rope_rows_packed, row_range)
from mylocal_llm_b200.quantized_weight import PackedGGUFWeight
from oracle import packed_oracle as po

from gguf_fixture import D, E, F, K, write_moe_gguf

gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = tmp_path_factory.mktemp("gguf") / "tiny_moe.gguf"
    arrays = write_moe_gguf(path)
    return GGUFPackedIndex.open(path), arrays


def test_metadata_and_shapes(model):
    index, _ = model
    assert (index.architecture, index.layers, index.d_model, index.expert_count, index.experts_per_token) == \
        ("qwen3next", 2, D, E, K)
    assert index.shape_of("blk.0.ffn_gate_exps.weight") == (E, F, D)
    assert index.shape_of("blk.1.ffn_gate_up_exps.weight") == (E, 2 * F, D)
    assert index.shape_of("blk.0.ffn_down_exps.weight") == (E, D, F)
    assert index.tensor_type("blk.0.ffn_down_exps.weight") == "Q6_K"
    assert "blk.0.ffn_gate_inp.weight" in index and "nope" not in index


def test_get_packed_is_a_view_of_the_mapping_with_the_written_bytes(model):
    index, arrays = model
    w = index.get_packed("blk.0.ffn_down_exps.weight")
    assert isinstance(w, PackedGGUFWeight) and w.shape == (E, D, F) and w.quant_type == "Q6_K"
    np.testing.assert_array_equal(np.asarray(w.data), arrays["blk.0.ffn_down_exps.weight"])
    assert np.shares_memory(w.data, index.tensors["blk.0.ffn_down_exps.weight"].data)      # no copy
    with pytest.raises(TypeError):
        index.get_packed("blk.0.ffn_gate_inp.weight")
    with pytest.raises(ValueError):
        index.non_expert_weight("blk.0.ffn_down_exps.weight")
    np.testing.assert_array_equal(index.non_expert_weight("blk.0.ffn_gate_inp.weight"), arrays["router"])


def test_expert_weights_split_the_fused_tensor_like_the_separate_ones(model):
    index, arrays = model
    for expert in (0, E - 1):
        g0, u0, d0 = index.expert_weights(0, expert)
        g1, u1, d1 = index.expert_weights(1, expert)
        for a, b in ((g0, g1), (u0, u1), (d0, d1)):
            assert a.shape == b.shape and a.quant_type == b.quant_type
            np.testing.assert_array_equal(np.asarray(a.data), np.asarray(b.data))
        np.testing.assert_array_equal(np.asarray(g0.data), arrays["gate"][expert].reshape(-1))
        np.testing.assert_array_equal(np.asarray(u1.data), arrays["up"][expert].reshape(-1))
        assert g1.shape == (F, D) and d1.shape == (D, F)
        # values, through the oracle's decoder
        np.testing.assert_array_equal(po.dequantize(np.asarray(g1.data), g1.shape, "Q4_K"),
                                      po.dequantize(arrays["gate"][expert].reshape(-1), (F, D), "Q4_K"))
    with pytest.raises(IndexError):
        index.expert_weights(0, E)
    with pytest.raises(IndexError):
        index.expert_weights(2, 0)


def test_row_range_rejects_bad_ranges(model):
    index, _ = model
    w = index.get_packed("blk.0.ffn_gate_shexp.weight")
    assert row_range(w, 16, 48).shape == (32, D)
    with pytest.raises(ValueError):
        row_range(w, 10, 10)
    with pytest.raises(ValueError):
        row_range(w, 0, F + 1)


def test_packed_rope_row_permutation_equals_the_dense_one(model):
    index, _ = model
    w = index.get_packed("blk.0.attn_q.weight")
    heads = 4
    restored = restore_hf_rope_rows_packed(w, heads)
    dense = po.dequantize(np.asarray(w.data), w.shape, "Q8_0")
    rows, cols = dense.shape
    half = rows // (heads * 2)
    want = dense.reshape(heads, half, 2, cols).swapaxes(1, 2).reshape(rows, cols)     # the reference's dense rule
    np.testing.assert_array_equal(po.dequantize(np.asarray(restored.data), restored.shape, "Q8_0"), want)
    with pytest.raises(ValueError):
        restore_hf_rope_rows_packed(w, 3)


def test_decode_dense_handles_f16_and_bf16():
    class Fake:
        def __init__(self, name, kind, data, shape):
            self.name, self.data, self.shape = name, data, shape
            self.tensor_type = type("T", (), {"name": kind})()
    x = np.array([[1.5, -2.0, 0.0078125]], np.float32)
    f16 = Fake("a", "F16", x.astype(np.float16), (3, 1))
    np.testing.assert_array_equal(decode_dense(f16), x)
    bf16 = Fake("b", "BF16", (x.view(np.uint32) >> 16).astype(np.uint16), (3, 1))
    np.testing.assert_array_equal(decode_dense(bf16), x)
    with pytest.raises(TypeError):
        decode_dense(Fake("c", "Q4_K", x, (3, 1)))
