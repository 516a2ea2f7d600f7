"""Loader for the reference's own CUDA ops compiled into oracle/_ref/ (test infrastructure).

The `.so` files are pybind/torch extensions built by oracle/build_ref.py from the
reference checkout; they are git-ignored build products.  When they are absent the
tests that compare against them are skipped (the oracle comparisons still run)."""
import importlib.util
import os

_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
_cache = {}


def load(name: str):
    """Returns the extension module `name` (e.g. "layernorm_ops") or None."""
    if name in _cache:
        return _cache[name]
    path = os.path.join(_DIR, f"{name}.so")
    mod = None
    if os.path.exists(path):
        try:
            import torch  # noqa: F401  (the extension links against libtorch)
            spec = importlib.util.spec_from_file_location(name, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        except Exception as e:  # pragma: no cover - depends on the box
            print(f"[ref_kernels] cannot load {path}: {e}")
            mod = None
    _cache[name] = mod
    return mod
