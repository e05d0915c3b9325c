"""CPU oracle of the Q8_1 integer-dot mode (TEST INFRASTRUCTURE ONLY; imported by tests/ and nothing else).

Restates, in NumPy:
  * the Q8_1 activation codec of the reference, ``mini_llm/ops/q8_1_gpu.py:30-58`` in its non-fast-math
    ("ieee") arithmetic: per 32 inputs d32 = bounded(max|x| / 127), codes = round-half-away(x / d32)
    clamped to +-127 (all zero for a zero block), stored fp16(d32), fp16(bounded(sum)), 32 x int8; the sum
    is the xor-butterfly sum (offsets 16, 8, 4, 2, 1) as lane 0 of a warp sees it;
  * the mixed Q8 linear for Q4_K, ``mini_llm/ops/mixed_q8_gpu.py:86-139,203-251``: per 16-position part
    integer dots of nibble codes with activation codes and integer sums of the activation codes, scaled
    by the activation block scale and the 6-bit sub-block scale / minimum, times the super-block's d and
    dmin. The integer quantities are evaluated exactly; the floating-point combination is done in FP64.

Parity UNPINNED against reference outputs: the reference's implementation of this mode is CuPy/NVRTC
only and cannot run without a GPU-side CuPy, and its bit-exact fixture is a CUDA header of a third-party
project. What pins this file instead: (a) ``tests/test_q8_oracle.py`` shows that the integer formula
equals the FP64 product of the (pinned) dequantised weights with the dequantised Q8_1 activations, and
(b) the codec is checked against its definition (code range, scale, zero blocks, ties away from zero).
"""

import numpy as np

from . import packed_oracle as po


def _bounded(x):
    return np.where(np.abs(x) > np.float32(65504.0), np.copysign(np.float32(65504.0), x), x).astype(np.float32)


def quantize_q8_1(x):
    """x float32 [rows, K] -> uint8 [rows, K/32, 36] (IEEE arithmetic, see the module docstring)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    b = x.reshape(rows, k // 32, 32)
    a = np.abs(b).max(axis=2)
    s = b.copy()
    for off in (16, 8, 4, 2, 1):                                # lane i adds lane i ^ off; lane 0 is read
        s = (s + s[..., np.arange(32) ^ off]).astype(np.float32)
    total = s[..., 0]
    d = _bounded((a / np.float32(127.0)).astype(np.float32))
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = (b / d[..., None]).astype(np.float32)
    q = np.where(a[..., None] == 0, np.float32(0), np.sign(ratio) * np.floor(np.abs(ratio) + np.float32(0.5)))
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.zeros((rows, k // 32, 36), np.uint8)
    out[..., 0:2] = _bounded(d).astype("<f2").view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 2:4] = _bounded(total).astype("<f2").view(np.uint8).reshape(rows, k // 32, 2)
    out[..., 4:] = q.view(np.uint8)
    return out


def dequantize_q8_1(blocks):
    """uint8 [rows, K/32, 36] -> float64 [rows, K]: d * code."""
    d = blocks[..., 0:2].copy().view("<f2").astype(np.float64)[..., 0]
    q = blocks[..., 4:].view(np.int8).astype(np.float64)
    return (d[..., None] * q).reshape(blocks.shape[0], -1)


def q4k_q8_1_linear(blocks, data, shape, fmt="Q4_K"):
    """Integer-dot evaluation of dequant(blocks) @ W.T for a Q4_K or Q5_K matrix (data, shape): float64
    [rows, N]. Q5_K: the same formula with 5-bit codes (the fifth bit of element l of sub-block s is bit s of
    byte l of the block's 32 high-bit bytes, ``mini_llm/ops/quantized_weight.py:233-241``)."""
    n, k = shape
    block = 176 if fmt == "Q5_K" else 144
    raw = np.asarray(data, np.uint8).reshape(n, k // 256, block)
    d = raw[..., 0:2].copy().view("<f2").astype(np.float64)[..., 0]            # [n, nsb]
    dmin = raw[..., 2:4].copy().view("<f2").astype(np.float64)[..., 0]
    sc, mn = po._k_scales_mins(raw[..., 4:16].reshape(-1, 12))
    sc, mn = sc.reshape(n, k // 256, 8).astype(np.int64), mn.reshape(n, k // 256, 8).astype(np.int64)
    nib = raw[..., block - 128:].astype(np.int64)                              # [n, nsb, 128]
    codes = np.empty((n, k // 256, 8, 32), np.int64)
    for pair in range(4):
        chunk = nib[..., 32 * pair:32 * pair + 32]
        codes[..., 2 * pair, :] = chunk & 15
        codes[..., 2 * pair + 1, :] = chunk >> 4
    if fmt == "Q5_K":
        high = raw[..., 16:48].astype(np.int64)                                # [n, nsb, 32]
        for sub in range(8):
            codes[..., sub, :] |= ((high >> sub) & 1) << 4
    rows = blocks.shape[0]
    dx = blocks[..., 0:2].copy().view("<f2").astype(np.float64)[..., 0].reshape(rows, k // 256, 8)
    u = blocks[..., 4:].view(np.int8).astype(np.int64).reshape(rows, k // 256, 8, 32)
    dot = np.einsum("nbsj,rbsj->rnbs", codes, u)                               # exact integers
    usum = u.sum(axis=3)                                                       # [rows, nsb, 8]
    sd = (dx[:, None] * (dot * sc[None])).sum(axis=3)                          # [rows, n, nsb]
    sm = (dx[:, None] * (usum[:, None] * mn[None])).sum(axis=3)
    return (d[None] * sd - dmin[None] * sm).sum(axis=2)
