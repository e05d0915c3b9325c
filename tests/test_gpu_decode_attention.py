"""Single-query attention over the KV cache (``b200q_decode_attention``) against an FP64 reference.

The kernel picks its shape from the grid: a cluster of four 32-warp CTAs per (batch, head) for a
handful of heads, one 32-warp CTA for a few hundred, one 8-warp CTA beyond that. Every shape has to
give softmax(q.K^T / sqrt(d)) V over positions 0..pos (the reference's inference attention,
mini_llm/ops/attention_inference.py:255-277), for positions inside the first group of a warp, across
several iterations, and at the end of the horizon.
"""

import ctypes

import numpy as np
import pytest

from mylocal_llm_b200 import _lib

pytestmark = pytest.mark.gpu


def run_kernel(torch, q, k, v, pos, out_dtype):
    batch, heads, dh = q.shape
    kv_heads, horizon = k.shape[1], k.shape[2]
    out = torch.empty((batch, heads * dh), dtype=out_dtype, device="cuda")
    position = torch.tensor([pos], dtype=torch.int64, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    ident = lambda dt: _lib.DTYPE_ID[str(dt).replace("torch.", "")]
    q2 = q.reshape(batch, heads * dh).contiguous()
    _lib.call("b200q_decode_attention", ptr(q2), q2.stride(0), ptr(k), ptr(v), ident(k.dtype), ptr(position), batch,
              heads, kv_heads, dh, horizon, float(dh ** -0.5), ptr(out), ident(out_dtype), _lib.current_stream())
    torch.cuda.synchronize()
    return out.reshape(batch, heads, dh)


def reference(torch, q, k, v, pos):
    batch, heads, dh = q.shape
    group = heads // k.shape[1]
    kk = k[:, :, :pos + 1].double().repeat_interleave(group, dim=1)          # [B, H, P, dh]
    vv = v[:, :, :pos + 1].double().repeat_interleave(group, dim=1)
    scores = torch.einsum("bhd,bhpd->bhp", q.double(), kk) * dh ** -0.5
    return torch.einsum("bhp,bhpd->bhd", torch.softmax(scores, dim=-1), vv)


@pytest.mark.parametrize("batch,heads,kv_heads", [(1, 8, 2), (1, 32, 32), (5, 16, 4), (10, 32, 8)])
@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("pos", [0, 5, 255, 256, 1023, 1024, 2299])
@pytest.mark.parametrize("cache", ["bfloat16", "float32"])
def test_decode_attention_matches_fp64(cuda, batch, heads, kv_heads, dh, pos, cache):
    torch = cuda
    if batch * heads * dh * pos > 10 * 32 * 64 * 1100 and cache == "float32":
        pytest.skip("large case: one cache type is enough")
    horizon = 2300
    gen = torch.Generator(device="cuda")
    gen.manual_seed(batch * 1000 + heads + dh + pos)
    cdt = getattr(torch, cache)
    q = torch.randn((batch, heads, dh), device="cuda", generator=gen)
    k = torch.randn((batch, kv_heads, horizon, dh), device="cuda", generator=gen).to(cdt)
    v = torch.randn((batch, kv_heads, horizon, dh), device="cuda", generator=gen).to(cdt)
    k[:, :, pos + 1:] = float("nan")                    # positions after `pos` must never be read into the result
    v[:, :, pos + 1:] = float("nan")
    got = run_kernel(torch, q, k, v, pos, torch.float32).double()
    ref = reference(torch, q, k, v, pos)
    assert bool(torch.isfinite(got).all())
    np.testing.assert_allclose(got.cpu().numpy(), ref.cpu().numpy(), rtol=2e-4, atol=2e-5)


def test_split_and_single_cta_shapes_agree(cuda, monkeypatch):
    torch = cuda
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    q = torch.randn((1, 8, 64), device="cuda", generator=gen)
    k = torch.randn((1, 8, 1500, 64), device="cuda", generator=gen).to(torch.bfloat16)
    v = torch.randn((1, 8, 1500, 64), device="cuda", generator=gen).to(torch.bfloat16)
    monkeypatch.setenv("B200Q_ATTENTION_SPLIT", "0")
    single = run_kernel(torch, q, k, v, 1400, torch.float32)
    monkeypatch.setenv("B200Q_ATTENTION_SPLIT", "1")
    split = run_kernel(torch, q, k, v, 1400, torch.float32)
    np.testing.assert_allclose(split.cpu().numpy(), single.cpu().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(split.double().cpu().numpy(), reference(torch, q, k, v, 1400).cpu().numpy(), rtol=2e-4,
                               atol=2e-5)


def run_rope(torch, q, k, v, positions, cos, sin, k_cache, v_cache):
    batch, heads, dh = q.shape
    kv_heads, horizon = k_cache.shape[1], k_cache.shape[2]
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    q2, k2, v2 = (a.reshape(batch, -1) for a in (q, k, v))
    _lib.call("b200q_rope_kv_store", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0),
              ptr(positions), ptr(cos), ptr(sin), int(cos.shape[0]), batch, 1, heads, kv_heads, dh, horizon,
              ptr(k_cache), ptr(v_cache), _lib.DTYPE_ID[str(k_cache.dtype).replace("torch.", "")],
              _lib.current_stream())
    torch.cuda.synchronize()


def rope_inputs(torch, table_rows, horizon, batch=2, heads=4, kv_heads=2, dh=64):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(17)
    q = torch.randn((batch, heads, dh), device="cuda", generator=gen)
    k = torch.randn((batch, kv_heads, dh), device="cuda", generator=gen)
    v = torch.randn((batch, kv_heads, dh), device="cuda", generator=gen)
    inv = 10000.0 ** (-torch.arange(0, dh, 2, dtype=torch.float64) / dh)
    ang = torch.arange(table_rows, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    k_cache = torch.full((batch, kv_heads, horizon, dh), 7.0, device="cuda")
    v_cache = torch.full((batch, kv_heads, horizon, dh), 7.0, device="cuda")
    return q, k, v, cos, sin, k_cache, v_cache


def test_rope_store_rotates_and_writes_one_cache_row(cuda):
    torch = cuda
    q, k, v, cos, sin, k_cache, v_cache = rope_inputs(torch, table_rows=40, horizon=32)
    pos = 9
    rot = lambda x: torch.cat([x[..., :32] * cos[pos] - x[..., 32:] * sin[pos],
                               x[..., :32] * sin[pos] + x[..., 32:] * cos[pos]], dim=-1)
    q_ref, k_ref = rot(q.clone()), rot(k.clone())
    run_rope(torch, q, k, v, torch.tensor([pos], dtype=torch.int64, device="cuda"), cos, sin, k_cache, v_cache)
    np.testing.assert_allclose(q.cpu().numpy(), q_ref.cpu().numpy(), rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(k_cache[:, :, pos].cpu().numpy(), k_ref.cpu().numpy(), rtol=1e-6, atol=1e-6)
    assert torch.equal(v_cache[:, :, pos], v)
    untouched = torch.ones(32, dtype=torch.bool, device="cuda")
    untouched[pos] = False
    assert bool((k_cache[:, :, untouched] == 7.0).all()) and bool((v_cache[:, :, untouched] == 7.0).all())
    assert _lib.device_status() == 0


@pytest.mark.parametrize("pos,table_rows,horizon", [(32, 40, 32), (36, 36, 48), (-1, 40, 32)])
def test_rope_store_skips_a_position_outside_cache_or_tables(cuda, pos, table_rows, horizon):
    """A captured decode step advances its position on the device; replayed past the end it must not read
    beyond the tables or write beyond the cache. Every address the kernel could form for the chosen
    positions lies inside the buffers allocated here, so the test itself cannot fault."""
    torch = cuda
    q, k, v, cos, sin, k_cache, v_cache = rope_inputs(torch, table_rows=table_rows, horizon=horizon)
    spare = torch.zeros((64, 32), device="cuda")                 # keeps table_rows an argument, not an allocation edge
    cos_big, sin_big = torch.cat([cos, spare]), torch.cat([sin, spare])
    q_before = q.clone()
    _lib.clear_device_status()
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    q2, k2, v2 = (a.reshape(2, -1) for a in (q, k, v))
    positions = torch.tensor([pos], dtype=torch.int64, device="cuda")
    _lib.call("b200q_rope_kv_store", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0),
              ptr(positions), ptr(cos_big), ptr(sin_big), table_rows, 2, 1, 4, 2, 64, horizon, ptr(k_cache),
              ptr(v_cache), _lib.DTYPE_ID["float32"], _lib.current_stream())
    torch.cuda.synchronize()
    try:
        assert _lib.device_status() == 301
        assert torch.equal(q, q_before)
        assert bool((k_cache == 7.0).all()) and bool((v_cache == 7.0).all())
    finally:
        _lib.clear_device_status()


def fused_case(torch, batch, heads, kv_heads, dh, pos, horizon, cache_dtype, seed):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    qkv = torch.randn((batch, (heads + 2 * kv_heads) * dh), device="cuda", generator=gen)        # one fused projection
    table_rows = horizon + 3
    inv = 10000.0 ** (-torch.arange(0, dh, 2, dtype=torch.float64) / dh)
    ang = torch.arange(table_rows, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    # rows before the position hold data, the position itself and everything after it NaN: a kernel that lets the
    # not-yet-written row (or a masked copy of it) into its sums shows it
    k_cache = torch.randn((batch, kv_heads, horizon, dh), device="cuda", generator=gen).to(cache_dtype)
    v_cache = torch.randn((batch, kv_heads, horizon, dh), device="cuda", generator=gen).to(cache_dtype)
    k_cache[:, :, max(pos, 0):] = float("nan")
    v_cache[:, :, max(pos, 0):] = float("nan")
    return qkv, cos, sin, k_cache, v_cache


def run_two_launches(torch, qkv, cos, sin, k_cache, v_cache, heads, kv_heads, dh, pos, out_dtype):
    batch, horizon = qkv.shape[0], k_cache.shape[2]
    qkv = qkv.clone()
    qd, kd = heads * dh, kv_heads * dh
    q2, k2, v2 = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    ident = lambda dt: _lib.DTYPE_ID[str(dt).replace("torch.", "")]
    positions = torch.tensor([pos], dtype=torch.int64, device="cuda")
    out = torch.full((batch, heads * dh), float("nan"), dtype=out_dtype, device="cuda")
    _lib.call("b200q_rope_kv_store", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0), ptr(positions),
              ptr(cos), ptr(sin), int(cos.shape[0]), batch, 1, heads, kv_heads, dh, horizon, ptr(k_cache), ptr(v_cache),
              ident(k_cache.dtype), _lib.current_stream())
    _lib.call("b200q_decode_attention", ptr(q2), q2.stride(0), ptr(k_cache), ptr(v_cache), ident(k_cache.dtype),
              ptr(positions), batch, heads, kv_heads, dh, horizon, float(dh ** -0.5), ptr(out), ident(out_dtype),
              _lib.current_stream())
    torch.cuda.synchronize()
    return out


def run_fused(torch, qkv, cos, sin, k_cache, v_cache, heads, kv_heads, dh, pos, out_dtype):
    batch, horizon = qkv.shape[0], k_cache.shape[2]
    before = qkv.clone()
    qd, kd = heads * dh, kv_heads * dh
    q2, k2, v2 = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    ident = lambda dt: _lib.DTYPE_ID[str(dt).replace("torch.", "")]
    positions = torch.tensor([pos], dtype=torch.int64, device="cuda")
    out = torch.full((batch, heads * dh), float("nan"), dtype=out_dtype, device="cuda")
    _lib.call("b200q_rope_attention", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0), ptr(positions),
              ptr(cos), ptr(sin), int(cos.shape[0]), batch, heads, kv_heads, dh, horizon, ptr(k_cache), ptr(v_cache),
              ident(k_cache.dtype), float(dh ** -0.5), ptr(out), ident(out_dtype), _lib.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(qkv, before), "the fused call must leave the projection output as it is"
    return out


@pytest.mark.parametrize("cache", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("batch,heads,kv_heads,dh,pos,horizon", [
    (1, 8, 8, 64, 0, 64), (1, 8, 2, 64, 7, 64), (2, 8, 4, 64, 8, 300), (1, 32, 32, 64, 255, 512),
    (1, 32, 8, 64, 1400, 1500), (3, 4, 2, 128, 33, 200), (1, 16, 16, 128, 511, 512), (40, 8, 2, 64, 100, 128),
    (20, 16, 4, 128, 65, 96)])
def test_rope_attention_in_one_launch_is_the_two_launches(cuda, monkeypatch, cache, batch, heads, kv_heads, dh, pos, horizon):
    """RoPE + cache store + attention as one kernel: same context vectors and same caches, bit for bit, as the two
    kernels in sequence - one or four CTAs per head, 32 or 8 warps, grouped KV heads, the position first / last /
    on a group boundary of the position loop."""
    torch = cuda
    dtype = getattr(torch, cache)
    for split in ("1", "0"):
        monkeypatch.setenv("B200Q_ATTENTION_SPLIT", split)
        qkv, cos, sin, k1, v1 = fused_case(torch, batch, heads, kv_heads, dh, pos, horizon, dtype, seed=pos + heads)
        k2, v2 = k1.clone(), v1.clone()
        two = run_two_launches(torch, qkv, cos, sin, k1, v1, heads, kv_heads, dh, pos, dtype)
        one = run_fused(torch, qkv, cos, sin, k2, v2, heads, kv_heads, dh, pos, dtype)
        assert bool(torch.isfinite(two.float()).all())
        assert torch.equal(one, two)
        assert torch.equal(k1[:, :, :pos + 1], k2[:, :, :pos + 1]) and torch.equal(v1[:, :, :pos + 1], v2[:, :, :pos + 1])
        assert bool(torch.isnan(k2[:, :, pos + 1:].float()).all()) and bool(torch.isnan(v2[:, :, pos + 1:].float()).all())
        assert _lib.device_status() == 0


@pytest.mark.parametrize("pos,table_rows,horizon", [(32, 40, 32), (36, 36, 48), (-1, 40, 32)])
def test_rope_attention_skips_a_position_outside_cache_or_tables(cuda, pos, table_rows, horizon):
    """The same bounds as the stand-alone RoPE kernel: no table entry read, caches untouched, status 301. Every address
    the kernel could form for these positions lies inside the buffers allocated here."""
    torch = cuda
    q, k, v, cos, sin, k_cache, v_cache = rope_inputs(torch, table_rows=table_rows, horizon=horizon)
    spare = torch.zeros((64, 32), device="cuda")
    cos_big, sin_big = torch.cat([cos, spare]), torch.cat([sin, spare])
    _lib.clear_device_status()
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    q2, k2, v2 = (a.reshape(2, -1) for a in (q, k, v))
    positions = torch.tensor([pos], dtype=torch.int64, device="cuda")
    out = torch.zeros((2, 4 * 64), device="cuda")
    _lib.call("b200q_rope_attention", ptr(q2), ptr(k2), ptr(v2), q2.stride(0), k2.stride(0), v2.stride(0), ptr(positions),
              ptr(cos_big), ptr(sin_big), table_rows, 2, 4, 2, 64, horizon, ptr(k_cache), ptr(v_cache),
              _lib.DTYPE_ID["float32"], 0.125, ptr(out), _lib.DTYPE_ID["float32"], _lib.current_stream())
    torch.cuda.synchronize()
    try:
        assert _lib.device_status() == 301
        assert bool((k_cache == 7.0).all()) and bool((v_cache == 7.0).all())
    finally:
        _lib.clear_device_status()
