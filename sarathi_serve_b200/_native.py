"""ctypes binding of libsarathi_b200.so (the C ABI declared in include/sarathi_b200.h).

There is no fallback: if the shared library is missing or fails to load, every
op of this package raises.  Build it with ``python -m sarathi_serve_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# SB200_LIBRARY: load another build of the library (e.g. the profiling variant of `build.py --trace`)
LIB_PATH = os.environ.get("SB200_LIBRARY") or os.path.join(_PKG, "libsarathi_b200.so")

F32, F16, BF16 = 0, 1, 2
I32, I64, I16, I8, U8 = 0, 1, 2, 3, 4

_DTYPE_ID = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
_ITYPE_ID = {torch.int32: I32, torch.int64: I64, torch.int16: I16, torch.int8: I8, torch.uint8: U8}

_lib = None


class NativeLibraryError(RuntimeError):
    pass


_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float


class RotaryArgs(ctypes.Structure):
    """Mirror of ``sb200_rotary_args`` (include/sarathi_b200.h)."""
    _fields_ = [("positions", c_void_p), ("cos_sin_cache", c_void_p), ("head_size", c_int),
                ("rot_dim", c_int), ("rot_cols", c_int), ("is_neox", c_int),
                ("kv_cache", c_void_p), ("kv_slots", c_void_p), ("kv_page_size", c_int), ("num_kv_heads", c_int)]


_PP = ctypes.POINTER(c_void_p)
_GEMM_SIGS: dict = {
    "sb200_gemm_colpar": (_I, [_P, _L, _P, _L, _P, _L, _P, _P, _L, _L, _L, _L, _I, _I, ctypes.POINTER(RotaryArgs), _P, _I,
                               _P, _L, _P]),
    "sb200_moe_block_rows": (_I, []),
    "sb200_moe_gather_rows": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _P]),
    "sb200_moe_gemm1": (_I, [_P, _P, _P, _P, _P, _L, _I, _L, _L, _I, _P, _I, _P]),
    "sb200_moe_gemm2": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _L, _I, _L, _L, _I, _P, _I, _P]),
    "sb200_moe_sum": (_I, [_P, _P, _P, _L, _I, _L, _I, _P]),
    "sb200_moe_sum_all_reduce": (_I, [_P, _P, _P, _L, _I, _L, _I, _P, _P, _PP]),
    "sb200_gemm_plan": (_I, [_I, _L, _L, _L, _I, _I, _L, ctypes.POINTER(c_int)]),
    "sb200_kv_cache_slots": (_I, [_P, _P, _P, _P, _P, _L, _I, _P]),
    "sb200_kv_cache_append": (_I, [_P, _P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _P]),
    "sb200_diag_mma_rate": (_I, [_I, _I, _I, _P, _P]),
    "sb200_comm_heap_bytes": (_L, [_L]),
    "sb200_comm_create": (_I, [_PP, _I, _I, _L]),
    "sb200_comm_create_external": (_I, [_PP, _I, _I, _L, _PP]),
    "sb200_comm_ipc_handle": (_I, [_P, _P]),
    "sb200_comm_open_peers": (_I, [_P, _P]),
    "sb200_comm_destroy": (_I, [_P]),
    "sb200_comm_local_heap": (_P, [_P]),
    "sb200_comm_scratch": (_P, [_P]),
    "sb200_comm_region_bytes": (_L, [_P]),
    "sb200_gemm_rowpar_arrivals": (_L, [_L, _L, _L, _I, _L, _L, _L]),
    "sb200_vocab_embedding": (_I, [_P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "sb200_comm_set_wait_limit": (_I, [_P, _L]),
    "sb200_comm_set_one_shot_bytes": (_I, [_P, _L]),
    "sb200_comm_set_multicast": (_I, [_P, _P]),
    "sb200_comm_has_multicast": (_I, [_P]),
    "sb200_comm_reset": (_I, [_P, _P]),
    "sb200_all_gather_rows": (_I, [_P, _P, _L, _L, _I, _P, _P, _PP]),
    "sb200_comm_status": (_I, [_P, _P, ctypes.POINTER(ctypes.c_uint32)]),
    "sb200_comm_clear_status": (_I, [_P, _P]),
    "sb200_all_reduce": (_I, [_P, _P, _L, _L, _I, _P, _P, _P, _F, _I, _P, _P, _P, _PP, _PP]),
    "sb200_gemm_rowpar": (_I, [_P, _P, _L, _P, _L, _L, _L, _L, _I, _P, _P, _P, _F, _I, _P, _P, _I, _P, _PP, _PP]),
}


def _declare(lib):
    P, I, L, F = c_void_p, c_int, c_int64, c_float
    sigs = {
        "sb200_last_error": (c_char_p, []),
        "sb200_version": (c_char_p, []),
        "sb200_rms_norm": (I, [P, P, P, F, L, L, I, P]),
        "sb200_fused_add_rms_norm": (I, [P, P, P, P, P, F, L, L, I, P]),
        "sb200_silu_and_mul": (I, [P, P, L, L, I, P]),
        "sb200_gelu_new": (I, [P, P, L, L, I, P]),
        "sb200_gelu_fast": (I, [P, P, L, L, I, P]),
        "sb200_rotary_embedding": (I, [P, P, P, L, I, I, I, I, L, L, P, I, I, P]),
        "sb200_topk_softmax": (I, [P, P, P, P, I, L, I, I, I, P]),
        "sb200_moe_align_block_size": (I, [P, I, L, I, I, P, L, P, L, P, P, L, P]),
        "sb200_moe_align_scratch_bytes": (L, [L, I]),
        "sb200_moe_align_block_size_noalloc": (I, [P, I, L, I, I, P, L, P, L, P, P]),
    }
    optional = {}
    optional.update(_GEMM_SIGS)
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for name, (res, args) in optional.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args


def lib():
    """The loaded shared library (loads it on first use, loudly)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m sarathi_serve_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)")
        try:
            handle = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
            _declare(handle)
        except (OSError, AttributeError) as e:
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().sb200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (status {status}): {msg}")


def dtype_id(t: torch.Tensor) -> int:
    try:
        return _DTYPE_ID[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported floating dtype {t.dtype}") from None


def itype_id(t: torch.Tensor) -> int:
    try:
        return _ITYPE_ID[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported integer dtype {t.dtype}") from None


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("sarathi_serve_b200 ops run on CUDA tensors only (no CPU fallback)")


def ptr(t):
    return None if t is None else t.data_ptr()
