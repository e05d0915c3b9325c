"""In-tree build of ``libb200q.so`` with nvcc for sm_100a.

``python -m mylocal_llm_b200.build`` compiles every ``.cu`` file under ``csrc/`` (in parallel,
one object per file) and links them into ``mylocal_llm_b200/libb200q.so``. The shared object is
kept in the source tree, next to the package, so that it travels with a snapshot of the tree;
it is rebuilt only when a source or header is newer.
"""

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libb200q.so"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas=-v",
]


def _nvcc():
    path = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(path).exists():
        raise RuntimeError("nvcc not found; the b200q kernels cannot be built")
    return path


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _headers():
    return sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def needs_build():
    if not LIB.exists():
        return True
    stamp = LIB.stat().st_mtime
    return any(p.stat().st_mtime > stamp for p in _sources() + _headers())


def build(force=False, verbose=False):
    """Compile and link the in-tree ``libb200q.so``; returns its path."""
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    header_stamp = max(p.stat().st_mtime for p in _headers())

    def compile_one(src):
        obj = OBJ_DIR / (src.stem + ".o")
        if (not force and obj.exists() and obj.stat().st_mtime >= src.stat().st_mtime
                and obj.stat().st_mtime >= header_stamp):
            return obj, ""
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stderr[-4000:]}")
        return obj, proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, _sources()))
    if verbose:
        for obj, log in results:
            if log:
                sys.stderr.write(f"--- {obj.name}\n{log}\n")
    tmp = LIB.with_suffix(f".{os.getpid()}.tmp.so")
    cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o, _ in results]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        raise RuntimeError(f"link failed:\n{proc.stderr[-4000:]}")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
