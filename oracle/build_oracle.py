"""Build recipe and ctypes loader for the CPU checkers (TEST INFRASTRUCTURE ONLY).

Two shared libraries are produced, both outside version control:

* ``oracle/_build/libpacked_oracle.so`` - this repository's plain-C restatement
  (``oracle/packed_oracle.c``), the "port" checker / CPU baseline.
* ``oracle/_ref/libref_packed_cpu.so`` - the reference's own CPU kernels, compiled with
  ``g++`` straight from its source file ``mini_llm/ops/native_packed_cpu.cpp`` (plus the
  header beside it) where the reference tree is mounted. No reference source is copied
  into this repository; on a machine without the reference tree the prebuilt file is used
  if it is already there.

Run ``python oracle/build_oracle.py`` to (re)build both.
"""

import ctypes
import os
import shutil
import subprocess
import threading
from pathlib import Path

HERE = Path(__file__).resolve().parent
PORT_SO = HERE / "_build" / "libpacked_oracle.so"
REF_SO = HERE / "_ref" / "libref_packed_cpu.so"
# the reference checkout: MYLOCAL_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE_ROOT = Path(os.environ.get("MYLOCAL_REFERENCE_ROOT") or HERE.parent.parent / "reference")
REFERENCE_CPP = REFERENCE_ROOT / "mini_llm" / "ops" / "native_packed_cpu.cpp"

FORMAT_ID = {"Q8_0": 0, "Q4_0": 1, "Q4_K": 2, "Q3_K": 3, "Q5_K": 4, "Q6_K": 5}
_LOCK = threading.Lock()
_LIBS = {}


def _newer(target, *sources):
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources)


def build_port(force=False):
    src = HERE / "packed_oracle.c"
    if not force and _newer(PORT_SO, src):
        return PORT_SO
    cc = os.environ.get("CC") or shutil.which("gcc") or shutil.which("cc")
    if not cc:
        raise RuntimeError("no C compiler for the oracle")
    PORT_SO.parent.mkdir(parents=True, exist_ok=True)
    tmp = PORT_SO.with_suffix(f".{os.getpid()}.tmp.so")
    subprocess.run([cc, "-O2", "-std=c11", "-shared", "-fPIC", "-ffp-contract=off", str(src),
                    "-lm", "-o", str(tmp)], check=True)
    os.replace(tmp, PORT_SO)
    return PORT_SO


def build_ref(force=False):
    """Compile the reference's CPU library where its source tree is mounted.

    Returns the path, or None when neither the source tree nor a prebuilt file exists.
    """
    if REFERENCE_CPP.exists():
        if not force and _newer(REF_SO, REFERENCE_CPP):
            return REF_SO
        cxx = os.environ.get("CXX") or shutil.which("g++")
        if not cxx:
            return REF_SO if REF_SO.exists() else None
        REF_SO.parent.mkdir(parents=True, exist_ok=True)
        tmp = REF_SO.with_suffix(f".{os.getpid()}.tmp.so")
        # Same flags as the reference's on-demand build (mini_llm/ops/native_packed_cpu.py:62-64).
        subprocess.run([cxx, "-O3", "-std=c++17", "-shared", "-fPIC", str(REFERENCE_CPP),
                        "-o", str(tmp)], check=True)
        os.replace(tmp, REF_SO)
        return REF_SO
    return REF_SO if REF_SO.exists() else None


def _declare(lib, prefix):
    ptr, i = ctypes.c_void_p, ctypes.c_int
    gemv = getattr(lib, prefix + "_gemv")
    gemv.argtypes = [ptr, i, i, i, ptr, i, ptr]
    gemv.restype = i
    expert = getattr(lib, prefix + "_expert")
    expert.argtypes = [ptr, i, ptr, i, ptr, i, i, i, ptr, i, ptr]
    expert.restype = i
    return gemv, expert


def load_port():
    """ctypes handle of the plain-C oracle (built on demand)."""
    with _LOCK:
        if "port" not in _LIBS:
            lib = ctypes.CDLL(str(build_port()))
            lib.oracle_dequantize.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_void_p]
            lib.oracle_dequantize.restype = ctypes.c_int
            gemv, expert = _declare(lib, "oracle")
            _LIBS["port"] = (lib, gemv, expert)
        return _LIBS["port"]


def load_ref():
    """ctypes handle of the reference's own CPU library, or None if unavailable."""
    with _LOCK:
        if "ref" not in _LIBS:
            path = build_ref()
            if path is None:
                _LIBS["ref"] = None
            else:
                lib = ctypes.CDLL(str(path))
                gemv = lib.mylocal_packed_gemv
                gemv.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                 ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
                gemv.restype = ctypes.c_int
                expert = lib.mylocal_packed_expert
                expert.argtypes = [ctypes.c_void_p, ctypes.c_int] * 3 + [
                    ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
                expert.restype = ctypes.c_int
                _LIBS["ref"] = (lib, gemv, expert)
        return _LIBS["ref"]


def port_dequantize(data, shape, fmt):
    """Bit-exact dequantisation by the plain-C port (pinned against the NumPy oracle and the reference's
    golden vectors in tests/test_oracle_golden.py); about 20x faster than the NumPy loops, which is
    what makes FP64 checks of whole 512-expert layers affordable."""
    import numpy as np
    lib, _, _ = load_port()
    raw = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    k = int(shape[-1])
    n = int(np.prod(shape[:-1], dtype=np.int64))
    out = np.empty((n, k), np.float32)
    rc = lib.oracle_dequantize(raw.ctypes.data, FORMAT_ID[fmt], n, k, out.ctypes.data)
    if rc:
        raise RuntimeError(f"oracle_dequantize rc={rc}")
    return out.reshape(shape)


def cpu_gemv(handle, data, fmt, n, k, x):
    """Run a (port or reference) GEMV: x float32 [tokens,k] -> float32 [tokens,n]."""
    import numpy as np
    _, gemv, _ = handle
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.empty((x.shape[0], n), np.float32)
    rc = gemv(data.ctypes.data, FORMAT_ID[fmt], n, k, x.ctypes.data, x.shape[0], out.ctypes.data)
    if rc:
        raise RuntimeError(f"cpu gemv rc={rc}")
    return out


def cpu_expert(handle, gate, up, down, d_model, d_ff, x):
    """Run a (port or reference) SwiGLU expert; gate/up/down are (data, fmt) pairs."""
    import numpy as np
    _, _, expert = handle
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, d_model)
    out = np.empty_like(x)
    bufs = [np.ascontiguousarray(p[0], dtype=np.uint8) for p in (gate, up, down)]
    rc = expert(bufs[0].ctypes.data, FORMAT_ID[gate[1]], bufs[1].ctypes.data, FORMAT_ID[up[1]],
                bufs[2].ctypes.data, FORMAT_ID[down[1]], d_model, d_ff, x.ctypes.data,
                x.shape[0], out.ctypes.data)
    if rc:
        raise RuntimeError(f"cpu expert rc={rc}")
    return out


if __name__ == "__main__":
    print("port:", build_port(force=True))
    print("ref :", build_ref(force=True))
