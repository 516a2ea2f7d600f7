"""The shared library loads without a GPU and exports every entry point the
public header declares (no compute calls here)."""
import ctypes
import os
import re

from sarathi_serve_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sarathi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_native.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/sarathi_b200.h but not exported: {missing}"


def test_binding_covers_header():
    lib = _native.lib()
    for n in declared_symbols():
        fn = getattr(lib, n)
        assert fn.argtypes is not None, f"{n} has no ctypes signature in _native.py"


def test_version_and_error_strings():
    lib = _native.lib()
    assert b"sm_100a" in lib.sb200_version()
    assert isinstance(lib.sb200_last_error(), bytes)


def test_argument_validation_without_gpu():
    """Shape checks run before any CUDA call, so they can be exercised on a CPU-only box."""
    lib = _native.lib()
    assert lib.sb200_rms_norm(None, None, None, 1e-5, 4, 0, 2, None) == 1
    assert b"bad shape" in lib.sb200_last_error()
    assert lib.sb200_rotary_embedding(None, None, None, 4, 1, 1, 64, 63, 64, 64, None, 1, 2, None) == 1
    assert lib.sb200_moe_align_block_size(None, 0, 8, 0, 16, None, 0, None, 0, None, None, 0, None) == 1
    assert lib.sb200_comm_heap_bytes(1 << 20) == 4096 + 7 * (1 << 20)
