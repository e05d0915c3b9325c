"""Packed GGUF weight container - host-side mirror of the reference's
``mini_llm/ops/quantized_weight.py`` (``BLOCK_FORMATS`` :24-37, ``PackedGGUFWeight`` :44-99).

The object is a validated *view* of packed bytes; it never materialises floating-point
weights on the host. The three ``*_reference`` helpers of the reference API are kept, but
they are executed by the CUDA kernels of this package (upload the selected packed rows, run
``b200q_dequantize`` / ``b200q_gemv``, copy the result back): this package contains no CPU
decoder at all.
"""

from dataclasses import dataclass
import math

import numpy as np

# elements per block, bytes per block (GGUF packs along the innermost dimension)
BLOCK_FORMATS = {
    "Q8_0": (32, 34),
    "Q4_0": (32, 18),
    "Q3_K": (256, 110),
    "Q4_K": (256, 144),
    "Q5_K": (256, 176),
    "Q6_K": (256, 210),
}


# Device-only layouts: a lossless re-ordering of a GGUF type's bytes (same size) that only the GPU
# kernels read; host-side PackedGGUFWeight never carries them.
DEVICE_LAYOUTS = {"Q6_K_TILED": "Q6_K", "Q4_K_TILED": "Q4_K", "Q8_0_TILED": "Q8_0", "Q5_K_TILED": "Q5_K"}


def block_format(quant_type):
    """(values per block, bytes per block) of a GGUF type or of a device layout of it."""
    return BLOCK_FORMATS[DEVICE_LAYOUTS.get(quant_type, quant_type)]


def packed_nbytes(shape, quant_type):
    qk, qb = block_format(quant_type)
    return math.prod(int(d) for d in shape) // qk * qb


@dataclass(frozen=True)
class PackedGGUFWeight:
    """Validated packed tensor; ``data`` references the original byte owner (e.g. an mmap).

    ``shape`` is canonical row-major ``[..., K]`` (the reverse of a GGUF tensor header).
    """

    data: np.ndarray
    shape: tuple
    quant_type: str

    def __post_init__(self):
        if self.quant_type not in BLOCK_FORMATS:
            raise ValueError(f"Unsupported packed GGUF type: {self.quant_type}")
        shape = tuple(int(d) for d in self.shape)
        if not shape or any(d <= 0 for d in shape):
            raise ValueError("Packed GGUF shape must have positive dimensions")
        qk, _ = BLOCK_FORMATS[self.quant_type]
        if shape[-1] % qk:
            raise ValueError(f"GGUF {self.quant_type}: innermost dimension must be a multiple of {qk}")
        raw = np.asarray(self.data)
        if not raw.flags.c_contiguous:
            raise ValueError("GGUF packed data must be contiguous")
        raw = raw.view(np.uint8).reshape(-1)
        expected = packed_nbytes(shape, self.quant_type)
        if raw.size != expected:
            raise ValueError(f"GGUF {self.quant_type}: expected {expected} bytes, got {raw.size}")
        object.__setattr__(self, "shape", shape)
        object.__setattr__(self, "data", raw)

    @property
    def nbytes(self):
        return int(self.data.nbytes)

    @property
    def block_elements(self):
        return BLOCK_FORMATS[self.quant_type][0]

    @property
    def row_bytes(self):
        qk, qb = BLOCK_FORMATS[self.quant_type]
        return self.shape[-1] // qk * qb

    def select_outer(self, index):
        """Zero-copy slice along the leading dimension (one expert of an ``[E, N, K]`` bank)."""
        if len(self.shape) < 2:
            raise ValueError("select_outer requires at least two dimensions")
        if not 0 <= int(index) < self.shape[0]:
            raise IndexError(index)
        chunk = packed_nbytes(self.shape[1:], self.quant_type)
        begin = int(index) * chunk
        return PackedGGUFWeight(self.data[begin:begin + chunk], self.shape[1:], self.quant_type)

    # -- reference-named helpers, executed on the GPU --------------------------------------
    def _as_matrix(self):
        rows = math.prod(self.shape[:-1])
        return rows, self.shape[-1]

    def dequantize_reference(self):
        """FP32 ndarray of ``shape`` (bit-exact GGUF decode), computed by ``b200q_dequantize``."""
        from .quantized_linear import dequantize_device, packed_bytes_to_device
        rows, k = self._as_matrix()
        dev = packed_bytes_to_device(self.data)
        return dequantize_device(dev, rows, k, self.quant_type).cpu().numpy().reshape(self.shape)

    def dequantize_rows_reference(self, indices, *, tile_rows=32):
        """Decode selected rows of a matrix, keeping order and duplicates."""
        if len(self.shape) != 2:
            raise ValueError("selected rows require a matrix; select_outer first")
        _check_tile_rows(tile_rows)
        indices = np.asarray(indices)
        if indices.ndim != 1 or indices.dtype.kind not in "iu":
            raise ValueError("indices must be a one-dimensional integer array")
        if np.any(indices >= self.shape[0]) or np.any(indices < 0):
            raise IndexError("packed row index out of range")
        if len(indices) == 0:
            return np.empty((0, self.shape[1]), np.float32)
        picked = np.ascontiguousarray(self.data.reshape(self.shape[0], self.row_bytes)[indices])
        return PackedGGUFWeight(picked.reshape(-1), (len(indices), self.shape[1]),
                                self.quant_type).dequantize_reference()

    def matvec_reference(self, vector, *, tile_rows=32):
        """FP32 ``W @ vector`` through the packed GEMV kernel."""
        if len(self.shape) != 2:
            raise ValueError("matvec requires a matrix; select_outer first")
        _check_tile_rows(tile_rows)
        vector = np.asarray(vector, dtype=np.float32)
        if vector.shape != (self.shape[1],):
            raise ValueError("vector shape must equal (matrix columns,)")
        import torch
        from .quantized_linear import packed_to_device, quantized_linear
        x = torch.from_numpy(np.ascontiguousarray(vector)).cuda().reshape(1, -1)
        return quantized_linear(x, packed_to_device(self)).reshape(-1).cpu().numpy()


def _check_tile_rows(tile_rows):
    if isinstance(tile_rows, (bool, np.bool_)) or not isinstance(tile_rows, (int, np.integer)) or tile_rows <= 0:
        raise ValueError("tile_rows must be a positive integer")
