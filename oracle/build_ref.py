"""Recipe: compile the reference's own CUDA ops into oracle/_ref/ (TEST INFRASTRUCTURE ONLY).

The four pybind extensions of the reference (`layernorm_ops`, `activation_ops`,
`pos_encoding_ops`, `moe_ops`; reference setup.py:95-136) are compiled from the
sources where they lie in the reference checkout, with the reference's own
flags (-O2 -std=c++17, setup.py:15-17) for compute_100/sm_100 -- the generic
code a stock build of the reference would produce on a B200.  Nothing is copied
into this repository: only the built `.so` files land in `oracle/_ref/`, which
is git-ignored.  The GPU parity tests load them (when present) to compare this
library's kernels with the reference's kernels on identical inputs.

Run:  python oracle/build_ref.py [--reference PATH] [--jobs N]
The build is skipped for every extension whose `.so` is newer than its sources.
Each translation unit includes torch/extension.h and takes minutes to compile.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

EXTENSIONS = {
    "layernorm_ops": ["layernorm.cpp", "layernorm_kernels.cu"],
    "activation_ops": ["activation.cpp", "activation_kernels.cu"],
    "pos_encoding_ops": ["pos_encoding.cpp", "pos_encoding_kernels.cu"],
    "moe_ops": ["moe.cpp", "moe_topk_softmax_kernels.cu", "moe_align_block_size_kernels.cu"],
}


def _flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths("cuda")]
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = inc + [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    lib_dirs = ce.library_paths("cuda")
    return common, lib_dirs


def _compile(src: str, obj: str, name: str, common):
    if src.endswith(".cu"):
        cmd = ["nvcc", "-O2", "-std=c++17", "--expt-relaxed-constexpr",
               "-gencode", "arch=compute_100,code=sm_100",
               "-Xcompiler", "-fPIC", f"-DTORCH_EXTENSION_NAME={name}",
               *common, "-c", src, "-o", obj]
    else:
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-DTORCH_EXTENSION_NAME={name}",
               *common, "-c", src, "-o", obj]
    subprocess.run(cmd, check=True)
    return obj


def build(reference: str, jobs: int = 0, verbose: bool = True) -> bool:
    """Build every extension that is out of date. Returns False if the reference is absent."""
    csrc = os.path.join(reference, "csrc")
    if not os.path.isdir(csrc):
        if verbose:
            print(f"[oracle/_ref] reference sources not found at {csrc}; nothing built")
        return False
    os.makedirs(OUT, exist_ok=True)
    common, lib_dirs = _flags()
    work = []
    stale = {}
    for name, files in EXTENSIONS.items():
        so = os.path.join(OUT, f"{name}.so")
        srcs = [os.path.join(csrc, f) for f in files]
        newest = max(os.path.getmtime(s) for s in srcs)
        if os.path.exists(so) and os.path.getmtime(so) >= newest:
            continue
        stale[name] = []
        for s in srcs:
            obj = os.path.join(OUT, f"{name}__{os.path.basename(s)}.o")
            stale[name].append(obj)
            work.append((s, obj, name))
    if not work:
        if verbose:
            print("[oracle/_ref] up to date")
        return True
    jobs = jobs or min(len(work), os.cpu_count() or 1)
    if verbose:
        print(f"[oracle/_ref] compiling {len(work)} translation units with {jobs} jobs "
              "(minutes each: they include torch/extension.h)")
    with ThreadPoolExecutor(jobs) as ex:
        list(ex.map(lambda a: _compile(*a, common), work))
    for name, objs in stale.items():
        so = os.path.join(OUT, f"{name}.so")
        cmd = ["g++", "-shared", *objs, "-o", so,
               *[f"-L{d}" for d in lib_dirs], *[f"-Wl,-rpath,{d}" for d in lib_dirs],
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        subprocess.run(cmd, check=True)
        for o in objs:
            os.remove(o)
        if verbose:
            print(f"[oracle/_ref] built {so}")
    return True


def complete_python_install(reference: str, target: str, verbose: bool = True) -> int:
    """The reference's setup.py lists its packages with find_packages(), which skips the four directories of
    the package that have no __init__.py (core/proto, core/sequence_manager,
    model_executor/parallel_utils/pipeline_parallel, layers/fused_moe/configs), so a
    `pip install --target <target> <reference>` cannot even `import sarathi`.  This adds those directories to
    such an install (a git-ignored directory; nothing of the reference enters the repository).  Returns the
    number of files added."""
    import shutil
    src_root, dst_root = os.path.join(reference, "sarathi"), os.path.join(target, "sarathi")
    if not (os.path.isdir(src_root) and os.path.isdir(dst_root)):
        return 0
    added = 0
    for d, dirs, files in os.walk(src_root):
        dirs[:] = [x for x in dirs if x != "__pycache__"]
        rel = os.path.relpath(d, src_root)
        dst = os.path.join(dst_root, rel)
        if os.path.isdir(dst):
            continue
        os.makedirs(dst)
        for f in files:
            if f.endswith((".py", ".pyi", ".json")):
                shutil.copy2(os.path.join(d, f), os.path.join(dst, f))
                added += 1
        if verbose:
            print(f"[baseline/_ref] added sarathi/{rel}")
    return added


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SARATHI_REFERENCE"), required="SARATHI_REFERENCE" not in os.environ,
                    help="checkout of microsoft/sarathi-serve (or $SARATHI_REFERENCE)")
    ap.add_argument("--jobs", type=int, default=0)
    a = ap.parse_args()
    sys.exit(0 if build(a.reference, a.jobs) else 1)
