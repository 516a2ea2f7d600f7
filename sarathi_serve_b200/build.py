"""In-tree build of libsarathi_b200.so with nvcc for sm_100a.

The library is torch-free (plain CUDA runtime + driver entry points looked up
at run time), so each translation unit compiles in seconds and the resulting
shared object is loaded through ctypes.  Objects are rebuilt only when their
source (or a header) is newer.

    python -m sarathi_serve_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libsarathi_b200.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the sm_100a library cannot be built")
    return nvcc


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "sarathi_b200.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force: bool = False, verbose: bool = False, defines=(), lib: str = LIB, obj_dir: str = OBJ) -> str:
    """``defines``: extra -D macros, e.g. ("SB200_TRACE",) for a profiling build whose collective kernels record
    per-phase time stamps (give such a build its own ``lib`` / ``obj_dir``; ``SB200_LIBRARY`` makes the package load it)."""
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    hm = _headers_mtime()
    todo, objs = [], []
    for f in sources():
        src = os.path.join(CSRC, f)
        obj = os.path.join(obj_dir, f[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            todo.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = obj[:-2] + ".ptxas.log"
        with open(log, "w") as fh:
            fh.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    if todo:
        with ThreadPoolExecutor(min(len(todo), os.cpu_count() or 1)) as ex:
            list(ex.map(compile_one, todo))
    if todo or not os.path.exists(lib):
        cmd = [nvcc, "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--trace", metavar="DIR", default=None,
                    help="build a profiling variant (-DSB200_TRACE) into DIR/libsarathi_b200_trace.so instead")
    a = ap.parse_args()
    if a.trace:
        print(build(a.force, a.verbose, defines=("SB200_TRACE",), lib=os.path.join(a.trace, "libsarathi_b200_trace.so"),
                    obj_dir=os.path.join(a.trace, "obj")))
    else:
        print(build(a.force, a.verbose))
    sys.exit(0)
