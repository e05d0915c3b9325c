"""GGUF file seam on the GPU: banks and MoE layers built from a file equal the ones built from the
same bytes directly; lazy projections go through the packed kernels."""

import numpy as np
import pytest

from mylocal_llm_b200 import PackedExpertBank, PackedGGUFWeight, PackedMoELayer, packed_to_device, quantized_linear
from mylocal_llm_b200 import quantized_swiglu
from mylocal_llm_b200.gguf_index import GGUFPackedIndex, project_gguf_linear, project_gguf_swiglu
from mylocal_llm_b200.quantized_linear import packed_bytes_to_device

from gguf_fixture import D, E, F, K, TYPES, write_moe_gguf

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = tmp_path_factory.mktemp("gguf") / "tiny_moe.gguf"
    arrays = write_moe_gguf(path)
    return GGUFPackedIndex.open(path), arrays


def test_expert_bank_from_file_holds_the_file_bytes_fused_or_not(cuda, model):
    index, arrays = model
    separate, fused = index.expert_bank(0), index.expert_bank(1)
    for bank in (separate, fused):
        assert (bank.n_experts, bank.d_model, bank.d_ff) == (E, D, F)
        assert (bank.gate_type, bank.up_type, bank.down_type) == TYPES
        np.testing.assert_array_equal(bank.gate.cpu().numpy(), arrays["gate"].reshape(-1))
        np.testing.assert_array_equal(bank.up.cpu().numpy(), arrays["up"].reshape(-1))
        np.testing.assert_array_equal(bank.down.cpu().numpy(), arrays["down"].reshape(-1))


@pytest.mark.parametrize("tokens", [1, 9])
def test_moe_layer_from_file_equals_the_layer_built_from_the_arrays(cuda, model, tokens):
    torch = cuda
    index, arrays = model
    bank = PackedExpertBank(*(packed_bytes_to_device(arrays[n].reshape(-1)) for n in ("gate", "up", "down")),
                            *TYPES, E, D, F)
    shapes = ((F, D), (F, D), (D, F))
    shared = tuple(packed_to_device(PackedGGUFWeight(raw.reshape(-1), shape, fmt))
                   for raw, shape, fmt in zip(arrays["shared"], shapes, TYPES))
    router = torch.from_numpy(arrays["router"]).cuda().t().contiguous()
    gate = torch.from_numpy(arrays["shexp_gate"]).cuda()
    direct = PackedMoELayer(bank, router, K, shared=shared, shared_gate=gate)
    x = torch.from_numpy(np.random.default_rng(tokens).normal(0, 1, (1, tokens, D)).astype(np.float32)).cuda()
    want = direct.forward(x)
    for layer_id in (0, 1):
        layer = index.moe_layer(layer_id)
        assert layer.router.k == K
        assert torch.equal(layer.forward(x), want)


def test_lazy_projections_use_the_packed_kernels_and_cache_the_upload(cuda, model):
    torch = cuda
    index, arrays = model
    x = torch.from_numpy(np.random.default_rng(2).normal(0, 1, (1, 3, D)).astype(np.float32)).cuda()
    host_cache, device_cache, uploads = {}, {}, []

    def upload(weight):
        uploads.append(weight.shape)
        return packed_to_device(weight)

    name = "blk.0.ffn_gate_shexp.weight"
    y = project_gguf_linear(x, index, name, host_cache, device_cache, "g", upload=upload)
    y2 = project_gguf_linear(x, index, name, host_cache, device_cache, "g", upload=upload)
    direct = packed_to_device(PackedGGUFWeight(arrays[name], (F, D), "Q4_K"))
    assert torch.equal(y, quantized_linear(x, direct)) and torch.equal(y2, y)
    assert uploads == [(F, D)]                                          # promoted once
    h = project_gguf_swiglu(x, index, name, "blk.0.ffn_up_shexp.weight", host_cache, device_cache, "g", "u",
                            upload=upload)
    up = packed_to_device(PackedGGUFWeight(arrays["blk.0.ffn_up_shexp.weight"], (F, D), "Q4_K"))
    assert torch.equal(h, quantized_swiglu(x, direct, up))
    # a dense tensor takes the plain product
    r = project_gguf_linear(x, index, "blk.0.ffn_gate_inp.weight", host_cache, device_cache, "r")
    np.testing.assert_allclose(r.cpu().numpy(), x.cpu().numpy() @ arrays["router"].T, rtol=1e-4, atol=1e-4)
