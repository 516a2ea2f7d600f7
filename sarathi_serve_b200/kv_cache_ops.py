"""Append of a step's keys and values to the paged KV cache (layout
[pages, 2, page_size, kv_heads, head_dim]), with the call signature of flashinfer's
``append_paged_kv_cache`` that the reference's attention wrapper uses
(sarathi/model_executor/attention/flashinfer_attention_wrapper.py:261-270).

``slots`` computes, once per step, the cache row of every token; ``append_paged_kv_cache`` copies
strided k / v views (no ``.contiguous()``) there.  ``dense_ops.linear_rotary(..., kv_cache=, kv_slots=)``
stores k and v from the qkv GEMM's epilogue instead, so that only ``slots`` remains as a launch."""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as N


def slots(batch_indices: torch.Tensor, positions: torch.Tensor, kv_indices: torch.Tensor, kv_indptr: torch.Tensor,
          page_size: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int64 [n]: row of the cache (seen as [pages * 2 * page_size, kv_heads * head_dim]) that receives token i's key;
    -1 where ``batch_indices[i] < 0``."""
    N.require_cuda(batch_indices, positions, kv_indices, kv_indptr, out)
    for name, t in (("batch_indices", batch_indices), ("positions", positions), ("kv_indices", kv_indices),
                    ("kv_indptr", kv_indptr)):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise RuntimeError(f"kv_cache_ops.slots: {name} must be a contiguous int32 tensor")
    n = batch_indices.numel()
    if positions.numel() != n:
        raise RuntimeError("kv_cache_ops.slots: batch_indices and positions differ in length")
    if out is None:
        out = torch.empty(n, dtype=torch.int64, device=batch_indices.device)
    N.check(N.lib().sb200_kv_cache_slots(N.ptr(out), N.ptr(batch_indices), N.ptr(positions), N.ptr(kv_indices),
                                         N.ptr(kv_indptr), n, int(page_size), N.stream_ptr()), "kv_cache_slots")
    return out


def append_rows(paged_kv_cache: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_slots: torch.Tensor) -> None:
    """key / value: [n, kv_heads * head_dim] (or [n, kv_heads, head_dim]), rows may be strided views of the
    fused qkv buffer; ``kv_slots`` from ``slots``."""
    N.require_cuda(paged_kv_cache, key, value, kv_slots)
    if paged_kv_cache.dim() != 5 or paged_kv_cache.shape[1] != 2 or not paged_kv_cache.is_contiguous():
        raise RuntimeError("append_rows: the cache must be a contiguous [pages, 2, page_size, kv_heads, head_dim] tensor")
    _, _, page, nkv, hd = paged_kv_cache.shape
    n = kv_slots.numel()
    k2 = key.reshape(n, -1) if key.dim() == 3 and key.is_contiguous() else key.view(n, -1) if key.dim() == 3 else key
    v2 = value.reshape(n, -1) if value.dim() == 3 and value.is_contiguous() else value.view(n, -1) if value.dim() == 3 else value
    for name, t in (("key", k2), ("value", v2)):
        if t.dim() != 2 or t.shape != (n, nkv * hd) or t.stride(1) != 1 or t.dtype != paged_kv_cache.dtype:
            raise RuntimeError(f"append_rows: {name} must be [n, kv_heads * head_dim] with unit inner stride and the cache's dtype")
    if kv_slots.dtype != torch.int64 or not kv_slots.is_contiguous():
        raise RuntimeError("append_rows: kv_slots must be a contiguous int64 tensor")
    N.check(N.lib().sb200_kv_cache_append(N.ptr(paged_kv_cache), N.ptr(k2), k2.stride(0), N.ptr(v2), v2.stride(0),
                                          N.ptr(kv_slots), n, nkv, hd, page, N.dtype_id(k2), N.stream_ptr()),
            "kv_cache_append")


def append_paged_kv_cache(append_key: torch.Tensor, append_value: torch.Tensor, batch_indices: torch.Tensor,
                          positions: torch.Tensor, paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor,
                          kv_indptr: torch.Tensor, kv_last_page_len: Optional[torch.Tensor] = None,
                          kv_layout: str = "NHD") -> None:
    """Drop-in for ``flashinfer.append_paged_kv_cache`` with a single 5-D NHD cache tensor (what the reference
    allocates).  ``kv_last_page_len`` is accepted and unused (flashinfer's kernel does not read it either: the
    slot follows from the position)."""
    if kv_layout != "NHD":
        raise RuntimeError("append_paged_kv_cache: only the NHD layout of the reference's cache is supported")
    s = slots(batch_indices, positions, kv_indices, kv_indptr, paged_kv_cache.shape[2])
    append_rows(paged_kv_cache, append_key, append_value, s)
