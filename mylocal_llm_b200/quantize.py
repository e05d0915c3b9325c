"""Host-side packers that turn FP32 matrices into GGUF block bytes (synthetic-weight tooling).

These produce *inputs* for the kernels: benchmark and test weights are drawn from a seeded
normal distribution and packed here. Nothing on the inference path calls this module.

* ``quantize_q8_0`` follows the only quantiser the reference holds, the Q8_0 packer of its
  GGUF test reader (tests/test_0085f_external_gguf.py:67-76 of the reference):
  ``d = max|w|/127`` (0 -> 1) stored as FP16, ``q = clip(round(w/d), -127, 127)``.
* The K-quant packers are this project's own simple min/max quantisers (the reference ships
  none): per sub-block affine (Q4_K/Q5_K) or symmetric (Q6_K) codes with 6-bit / 8-bit
  sub-block scales under one FP16 super-block scale. They only have to produce valid blocks
  whose decode is close to the input; they make no claim to match any other tool's choices.
* ``random_packed`` makes random-byte blocks with forced finite FP16 scales, the fixture
  style of the reference's operator tests (tests/test_0106b_quantized_linear.py:15-31).
"""

import numpy as np

from .quantized_weight import BLOCK_FORMATS, PackedGGUFWeight


def _f16_bytes(values):
    return np.ascontiguousarray(values.astype("<f2")).view(np.uint8).reshape(-1, 2)


def quantize_q8_0(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    blocks = w.reshape(-1, 32)
    scales = np.max(np.abs(blocks), axis=1) / 127.0
    scales[scales == 0] = 1
    scales = scales.astype("<f2")
    q = np.clip(np.round(blocks / scales.astype(np.float32)[:, None]), -127, 127).astype(np.int8)
    raw = np.concatenate([scales.view(np.uint8).reshape(-1, 2), q.view(np.uint8)], axis=1)
    return PackedGGUFWeight(raw.reshape(-1), w.shape, "Q8_0")


def _pack_k_scales(sc, mn):
    """[nb,8] 6-bit scales and mins -> [nb,12] metadata bytes (inverse of the GGUF unpacking)."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    m = np.zeros((sc.shape[0], 12), np.uint8)
    m[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    m[:, 4:8] = mn[:, 0:4] | ((mn[:, 4:8] >> 4) << 6)
    m[:, 8:12] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
    return m


def _quantize_affine_k(w, levels):
    """Shared Q4_K (levels=15) / Q5_K (levels=31) code assignment."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    sub = w.reshape(-1, 8, 32)
    lo = np.minimum(sub.min(axis=2), 0.0)
    hi = np.maximum(sub.max(axis=2), lo + 1e-30)
    scale = (hi - lo) / levels                               # [nb,8] >= 0
    minimum = -lo                                            # [nb,8] >= 0
    d = (scale.max(axis=1) / 63.0).astype("<f2").astype(np.float32)
    dmin = (minimum.max(axis=1) / 63.0).astype("<f2").astype(np.float32)
    d_safe = np.where(d > 0, d, 1.0)
    dmin_safe = np.where(dmin > 0, dmin, 1.0)
    sc = np.clip(np.round(scale / d_safe[:, None]), 0, 63)
    mn = np.clip(np.round(minimum / dmin_safe[:, None]), 0, 63)
    eff_scale = d[:, None] * sc
    eff_min = dmin[:, None] * mn
    q = np.round((sub + eff_min[:, :, None]) / np.where(eff_scale > 0, eff_scale, 1.0)[:, :, None])
    q = np.clip(q, 0, levels).astype(np.uint8)
    return w.shape, d, dmin, sc, mn, q


def quantize_q4_k(w):
    shape, d, dmin, sc, mn, q = _quantize_affine_k(w, 15)
    nb = q.shape[0]
    raw = np.zeros((nb, 144), np.uint8)
    raw[:, 0:2] = _f16_bytes(d)
    raw[:, 2:4] = _f16_bytes(dmin)
    raw[:, 4:16] = _pack_k_scales(sc, mn)
    for pair in range(4):
        raw[:, 16 + 32 * pair:48 + 32 * pair] = q[:, 2 * pair] | (q[:, 2 * pair + 1] << 4)
    return PackedGGUFWeight(raw.reshape(-1), shape, "Q4_K")


def quantize_q5_k(w):
    shape, d, dmin, sc, mn, q = _quantize_affine_k(w, 31)
    nb = q.shape[0]
    raw = np.zeros((nb, 176), np.uint8)
    raw[:, 0:2] = _f16_bytes(d)
    raw[:, 2:4] = _f16_bytes(dmin)
    raw[:, 4:16] = _pack_k_scales(sc, mn)
    high = np.zeros((nb, 32), np.uint8)
    for g in range(8):
        high |= ((q[:, g] >> 4) & 1) << g
    raw[:, 16:48] = high
    low = q & 15
    for pair in range(4):
        raw[:, 48 + 32 * pair:80 + 32 * pair] = low[:, 2 * pair] | (low[:, 2 * pair + 1] << 4)
    return PackedGGUFWeight(raw.reshape(-1), shape, "Q5_K")


def quantize_q6_k(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    sub = w.reshape(-1, 16, 16)
    amax = np.abs(sub).max(axis=2)                            # [nb,16]
    scale = amax / 31.0
    d = (scale.max(axis=1) / 127.0).astype("<f2").astype(np.float32)
    d_safe = np.where(d > 0, d, 1.0)
    sc = np.clip(np.round(scale / d_safe[:, None]), 0, 127).astype(np.int8)
    eff = d[:, None] * sc.astype(np.float32)
    q = np.round(sub / np.where(eff > 0, eff, 1.0)[:, :, None])
    q6 = (np.clip(q, -32, 31) + 32).astype(np.uint8).reshape(-1, 256)
    nb = q6.shape[0]
    raw = np.zeros((nb, 210), np.uint8)
    for half in range(2):
        for quarter in range(4):
            v = q6[:, 128 * half + 32 * quarter:128 * half + 32 * quarter + 32]
            lo_at = 64 * half + 32 * (quarter % 2)
            raw[:, lo_at:lo_at + 32] |= (v & 15) << (4 * (quarter // 2))
            raw[:, 128 + 32 * half:160 + 32 * half] |= (v >> 4) << (2 * quarter)
    raw[:, 192:208] = sc.view(np.uint8)
    raw[:, 208:210] = _f16_bytes(d)
    return PackedGGUFWeight(raw.reshape(-1), w.shape, "Q6_K")


def quantize_q4_0(w):
    """32-value blocks: d = -(value of largest magnitude) / 8, codes round(w / d) + 8 clipped to 0..15."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    blocks = w.reshape(-1, 32)
    pick = np.argmax(np.abs(blocks), axis=1)
    extreme = blocks[np.arange(blocks.shape[0]), pick]
    d = (extreme / -8.0).astype("<f2")
    d32 = d.astype(np.float32)
    q = np.clip(np.round(blocks / np.where(d32 != 0, d32, 1.0)[:, None]) + 8, 0, 15).astype(np.uint8)
    raw = np.concatenate([d.view(np.uint8).reshape(-1, 2), q[:, :16] | (q[:, 16:] << 4)], axis=1)
    return PackedGGUFWeight(raw.reshape(-1), w.shape, "Q4_0")


def quantize_q3_k(w):
    """256-value super-blocks, sixteen groups of 16 with signed 6-bit scales and 3-bit codes in -4..3."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    sub = w.reshape(-1, 16, 16)
    pick = np.argmax(np.abs(sub), axis=2)
    extreme = np.take_along_axis(sub, pick[:, :, None], axis=2)[:, :, 0]
    scale = extreme / -4.0                                     # the extreme value maps to code -4
    d = (np.abs(scale).max(axis=1) / 31.0).astype("<f2").astype(np.float32)
    d_safe = np.where(d > 0, d, 1.0)
    sc = np.clip(np.round(scale / d_safe[:, None]), -32, 31).astype(np.int32)
    eff = d[:, None] * sc.astype(np.float32)
    q = np.clip(np.round(sub / np.where(eff != 0, eff, 1.0)[:, :, None]), -4, 3).astype(np.int32).reshape(-1, 256)
    nb = q.shape[0]
    raw = np.zeros((nb, 110), np.uint8)
    code = (q + 4).astype(np.uint8)                            # 0..7: bit 2 = "not lowered by 4" flag, bits 0-1 = low
    pos = np.arange(256)
    for p0 in range(0, 256, 32):
        blk = code[:, p0:p0 + 32]
        raw[:, 0:32] |= ((blk >> 2) & 1) << (p0 // 32)
        at = 32 + 32 * (p0 // 128)
        raw[:, at:at + 32] |= (blk & 3) << (2 * ((p0 // 32) % 4))
    stored = (sc + 32).astype(np.uint8)                        # 6-bit field
    for s_i in range(16):
        raw[:, 96 + (s_i & 7)] |= (stored[:, s_i] & 15) << (4 * (s_i >> 3))
        raw[:, 104 + (s_i & 3)] |= ((stored[:, s_i] >> 4) & 3) << (2 * (s_i >> 2))
    raw[:, 108:110] = _f16_bytes(d)
    return PackedGGUFWeight(raw.reshape(-1), w.shape, "Q3_K")


QUANTIZERS = {"Q8_0": quantize_q8_0, "Q4_0": quantize_q4_0, "Q3_K": quantize_q3_k, "Q4_K": quantize_q4_k,
              "Q5_K": quantize_q5_k, "Q6_K": quantize_q6_k}


def quantize(w, quant_type):
    """Pack an FP32 array whose last dimension is block-aligned."""
    if quant_type not in QUANTIZERS:
        raise ValueError(f"no quantiser for {quant_type}")
    if w.shape[-1] % BLOCK_FORMATS[quant_type][0]:
        raise ValueError("innermost dimension must be block-aligned")
    return QUANTIZERS[quant_type](w)


def set_sane_scales(raw, quant_type, d=None, dmin=None):
    """Overwrite the FP16 scale fields of random blocks ``raw`` [nb, block_bytes] with finite values."""
    if quant_type == "Q6_K":
        raw[:, 208:210] = _f16_bytes(np.asarray([1 / 1024 if d is None else d], np.float32))
    elif quant_type == "Q3_K":
        raw[:, 108:110] = _f16_bytes(np.asarray([1 / 256 if d is None else d], np.float32))
    elif quant_type in ("Q4_K", "Q5_K"):
        raw[:, 0:2] = _f16_bytes(np.asarray([0.03125 if d is None else d], np.float32))
        raw[:, 2:4] = _f16_bytes(np.asarray([0.015625 if dmin is None else dmin], np.float32))
    else:
        raw[:, 0:2] = _f16_bytes(np.asarray([0.5 if d is None else d], np.float32))
    return raw


def random_packed(quant_type, shape, seed, d=None, dmin=None):
    """Random-byte blocks with finite scales: exercises every bit of the decoders."""
    qk, qb = BLOCK_FORMATS[quant_type]
    nb = int(np.prod(shape)) // qk
    raw = np.random.default_rng(seed).integers(0, 256, size=(nb, qb), dtype=np.uint8)
    set_sane_scales(raw, quant_type, d, dmin)
    return PackedGGUFWeight(raw.reshape(-1), tuple(shape), quant_type)
