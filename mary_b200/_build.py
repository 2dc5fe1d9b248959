"""Builds the native libraries in-tree.

Two shared objects are produced next to this file:

* ``_core.so``    — C++17 host runtime: pile store, BLAKE3, paged-KV allocator, batch scheduler
                   (compiled with g++).
* ``_kernels.so`` — every CUDA kernel, compiled by nvcc for sm_100a only.  The launchers are plain
                   ``extern "C"`` functions taking raw device pointers and a stream, so the library
                   has no dependency on torch headers and builds in seconds per file.

Both are loaded with ctypes (``mary_b200._native``).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "csrc" / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _stamp(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd, log=None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        Path(log).write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)))
    return r.stdout + r.stderr


def build_core(force: bool = False) -> Path:
    out = ROOT / "_core.so"
    srcs = sorted((CSRC / "core").glob("*.cpp"))
    hdrs = sorted((CSRC / "core").glob("*.hpp"))
    stamp = _stamp(srcs + hdrs)
    sf = OBJ / "core.stamp"
    if out.exists() and not force and sf.exists() and sf.read_text() == stamp:
        return out
    OBJ.mkdir(parents=True, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    _run([cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(out)] + [str(s) for s in srcs])
    sf.write_text(stamp)
    return out


def nvcc_path() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def build_kernels(force: bool = False) -> Path:
    out = ROOT / "_kernels.so"
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h"))
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = nvcc_path()
    hdr_stamp = _stamp(hdrs, " ".join(NVCC_FLAGS))

    def compile_one(src: Path):
        obj = OBJ / (src.stem + ".o")
        sf = OBJ / (src.stem + ".stamp")
        stamp = _stamp([src], hdr_stamp)
        if obj.exists() and not force and sf.exists() and sf.read_text() == stamp:
            return obj, False
        _run([nvcc] + NVCC_FLAGS + ["-I", str(CSRC / "kernels"), "-c", str(src), "-o", str(obj)],
             log=OBJ / (src.stem + ".ptxas.log"))
        sf.write_text(stamp)
        return obj, True

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        res = list(ex.map(compile_one, srcs))
    objs = [str(o) for o, _ in res]
    if out.exists() and not force and not any(ch for _, ch in res):
        return out
    _run([nvcc, "-shared", "-o", str(out)] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"])
    return out


def build_all(force: bool = False):
    return build_core(force), build_kernels(force)


if __name__ == "__main__":
    print(build_all("--force" in sys.argv))
