"""Tensor-level wrappers of the dense projection entry points of the C ABI
(``sb200_gemm_colpar``): the local matmul of a column-parallel / replicated
linear layer, optionally with the rotary embedding or SiLU*mul applied in the
GEMM epilogue.  bf16/fp16 run on tcgen05 tensor cores, fp32 on an FFMA kernel."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native as N

EPI_NONE, EPI_ROTARY, EPI_SILU_MUL = 0, 1, 2

_status_words: dict = {}
_workspaces: dict = {}

# Split-K workspace per device: 64 KiB of arrival counters (kept zero by the kernels) + fp32 partial tiles.
WORKSPACE_BYTES = (64 << 10) + (96 << 20)


def workspace(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _workspaces.get(key)
    if w is None:
        w = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[key] = w
    return w


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device uint32 word the GEMM kernels write a non-zero code into when a
    bounded pipeline wait runs out (checked by ``check_status``)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def check_status(device: torch.device) -> None:
    """Synchronises and raises if any GEMM on ``device`` reported a timed-out wait."""
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"sm_100a GEMM pipeline wait timed out (device status code {v})")


def _ws(x: torch.Tensor):
    """(pointer, bytes) of the split-K workspace for x's device; fp32 runs the FFMA kernel and needs none."""
    if x.dtype == torch.float32:
        return None, 0
    w = workspace(x.device)
    return N.ptr(w), w.numel()


def _rows_2d(x: torch.Tensor, what: str) -> torch.Tensor:
    if x.dim() != 2:
        x = x.reshape(-1, x.shape[-1])
    if x.stride(1) != 1:
        raise RuntimeError(f"{what}: inner stride must be 1")
    return x


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, tile_n: int = 0) -> torch.Tensor:
    """y[T, N] = x[T, K] @ weight[N, K]^T (+ bias): F.linear semantics
    (reference call sites: tensor_parallel/layers.py:284,423,518)."""
    N.require_cuda(x, weight, bias)
    lead = x.shape[:-1]
    x2 = _rows_2d(x, "linear input")
    if weight.dim() != 2 or weight.stride(1) != 1 or weight.shape[1] != x2.shape[1]:
        raise RuntimeError(f"linear: weight {tuple(weight.shape)} does not match input {tuple(x.shape)}")
    if weight.dtype != x2.dtype or (bias is not None and bias.dtype != x2.dtype):
        raise RuntimeError("linear: dtype mismatch")
    T, K = x2.shape
    Nn = weight.shape[0]
    if out is None:
        out = torch.empty(T, Nn, dtype=x2.dtype, device=x2.device)
    elif out.shape != (T, Nn) or out.stride(1) != 1 or out.dtype != x2.dtype:
        raise RuntimeError("linear: bad out tensor")
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), N.ptr(bias), T, Nn, K, N.dtype_id(x2), EPI_NONE, None,
                                      N.ptr(status_word(x2.device)), tile_n, *_ws(x2), N.stream_ptr()), "gemm_colpar")
    return out.view(*lead, Nn) if len(lead) != 1 else out


def fused_rotary_supported(x: torch.Tensor, head_size: int, rot_dim: int) -> bool:
    return x.dtype in (torch.bfloat16, torch.float16) and rot_dim == head_size and head_size in (64, 128, 256)


def linear_rotary(x: torch.Tensor, weight: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
                  head_size: int, rot_cols: int, is_neox: bool, out: Optional[torch.Tensor] = None,
                  tile_n: int = 0) -> torch.Tensor:
    """qkv[T, N] = x @ weight^T with rotary_embedding applied to columns [0, rot_cols)
    (the q and k heads) in the GEMM epilogue -- the qkv_proj + rotary_emb pair of
    models/llama.py:175-177 in one kernel."""
    N.require_cuda(x, weight, positions, cos_sin_cache)
    x2 = _rows_2d(x, "linear_rotary input")
    T, K = x2.shape
    Nn = weight.shape[0]
    if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
        raise RuntimeError("linear_rotary: positions must be contiguous int64 [T]")
    if cos_sin_cache.dtype != x2.dtype or not cos_sin_cache.is_contiguous():
        raise RuntimeError("linear_rotary: cos_sin_cache must be contiguous and share the activation dtype")
    if out is None:
        out = torch.empty(T, Nn, dtype=x2.dtype, device=x2.device)
    rot = N.RotaryArgs(N.ptr(positions), N.ptr(cos_sin_cache), head_size, cos_sin_cache.shape[1], rot_cols,
                       1 if is_neox else 0)
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), None, T, Nn, K, N.dtype_id(x2), EPI_ROTARY,
                                      ctypes.byref(rot), N.ptr(status_word(x2.device)), tile_n, *_ws(x2),
                                      N.stream_ptr()),
            "gemm_colpar[rotary]")
    return out


def linear_silu_mul(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                    tile_n: int = 0) -> torch.Tensor:
    """act[T, d] = silu(x @ Wgate^T) * (x @ Wup^T) with weight = [Wgate; Wup] ([2d, K]):
    the gate_up_proj + SiluAndMul pair of models/llama.py:101-104 in one kernel."""
    N.require_cuda(x, weight)
    x2 = _rows_2d(x, "linear_silu_mul input")
    T, K = x2.shape
    Nn = weight.shape[0]
    if out is None:
        out = torch.empty(T, Nn // 2, dtype=x2.dtype, device=x2.device)
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), None, T, Nn, K, N.dtype_id(x2), EPI_SILU_MUL, None,
                                      N.ptr(status_word(x2.device)), tile_n, *_ws(x2), N.stream_ptr()),
            "gemm_colpar[silu_mul]")
    return out


def gemm_plan(epilogue: int, T: int, Nn: int, K: int, head_size: int = 128, tile_cfg: int = 0,
              workspace_bytes: int = WORKSPACE_BYTES) -> dict:
    """The tile shape / schedule the library would use for a [T, K] x [Nn, K]^T projection."""
    out = (ctypes.c_int * 11)()
    N.check(N.lib().sb200_gemm_plan(epilogue, T, Nn, K, head_size, tile_cfg, workspace_bytes, out), "gemm_plan")
    keys = ("cta_pairs", "accumulators", "bn", "units", "tiles_full", "k_parts", "kb_per_part", "stages", "m_tiles",
            "n_tiles", "k_blocks")
    return dict(zip(keys, out))
