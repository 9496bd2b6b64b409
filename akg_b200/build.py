"""Builds the in-tree shared library ``akg_b200/lib/libakgb.so`` with nvcc for sm_100a.

Every translation unit under ``csrc/`` is compiled with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked with the
static CUDA runtime, so the library loads (and plans) on a machine without a
GPU.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib" / "libakgb.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list((ROOT.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, hdr_mtime: float, verbose: bool) -> Path:
    obj = OBJ / (src.name + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj
    cmd = [NVCC, *FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ / (src.name + ".log")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"[akg_b200.build] compiled {src.name}\n")
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source and link ``libakgb.so``; returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    hdr = _newest_header()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr, verbose), srcs))
    if LIB.exists() and all(LIB.stat().st_mtime > o.stat().st_mtime for o in objs):
        return LIB
    cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl", "-lrt"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"[akg_b200.build] linked {LIB}\n")
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
