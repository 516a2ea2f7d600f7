"""Drop-in for the reference's pybind module ``sarathi.moe_ops`` (csrc/moe.cpp:3-27)."""
from typing import Optional

import torch

from . import _native as N


def topk_softmax(topk_weights: torch.Tensor, topk_indices: torch.Tensor, token_expert_indices: Optional[torch.Tensor],
                 gating_output: torch.Tensor, renormalize: bool = False) -> None:
    """Softmax + top-k over gating_output [T,E] (csrc/moe_topk_softmax_kernels.cu:476-503).

    Extensions over the reference op: gating_output may be fp16/bf16 (the
    ``.float()`` of fused_moe.py:367 is folded in) and ``renormalize=True`` applies
    fused_moe.py:371-372 in the same launch."""
    N.require_cuda(topk_weights, topk_indices, gating_output, token_expert_indices)
    if topk_weights.dtype != torch.float32 or topk_indices.dtype != torch.int32:
        raise RuntimeError("topk_softmax: topk_weights must be float32 and topk_indices int32")
    if token_expert_indices is not None and token_expert_indices.dtype != torch.int32:
        raise RuntimeError("topk_softmax: token_expert_indices must be int32")
    for t in (topk_weights, topk_indices, gating_output, token_expert_indices):
        if t is not None and not t.is_contiguous():
            raise RuntimeError("topk_softmax: tensors must be contiguous")
    E = gating_output.shape[-1]
    T = gating_output.numel() // E
    k = topk_weights.shape[-1]
    N.check(N.lib().sb200_topk_softmax(N.ptr(topk_weights), N.ptr(topk_indices), N.ptr(token_expert_indices),
                                       N.ptr(gating_output), N.dtype_id(gating_output), T, E, k,
                                       1 if renormalize else 0, N.stream_ptr()), "topk_softmax")


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int, sorted_token_ids: torch.Tensor,
                         experts_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor,
                         scratch: Optional[torch.Tensor] = None) -> None:
    """Block-aligned stable counting sort (csrc/moe_align_block_size_kernels.cu:112-135).

    ``sorted_token_ids`` is fully overwritten (pad value = topk_ids.numel()), so
    the caller's pre-fill (fused_moe.py:195) is not required."""
    N.require_cuda(topk_ids, sorted_token_ids, experts_ids, num_tokens_post_pad, scratch)
    if sorted_token_ids.dtype != torch.int32 or experts_ids.dtype != torch.int32 or num_tokens_post_pad.dtype != torch.int32:
        raise RuntimeError("moe_align_block_size: outputs must be int32")
    if not (topk_ids.is_contiguous() and sorted_token_ids.is_contiguous() and experts_ids.is_contiguous()):
        raise RuntimeError("moe_align_block_size: tensors must be contiguous")
    sb = scratch.numel() * scratch.element_size() if scratch is not None else 0
    N.check(N.lib().sb200_moe_align_block_size(N.ptr(topk_ids), N.itype_id(topk_ids), topk_ids.numel(),
                                               int(num_experts), int(block_size), N.ptr(sorted_token_ids),
                                               sorted_token_ids.numel(), N.ptr(experts_ids), experts_ids.numel(),
                                               N.ptr(num_tokens_post_pad), N.ptr(scratch), sb, N.stream_ptr()),
            "moe_align_block_size")


def moe_align_scratch_bytes(numel: int, num_experts: int) -> int:
    return int(N.lib().sb200_moe_align_scratch_bytes(int(numel), int(num_experts)))


NOALLOC_MAX_SLOTS = 65536
NOALLOC_MAX_EXPERTS = 256


def moe_align_block_size_noalloc(topk_ids: torch.Tensor, num_experts: int, block_size: int,
                                 sorted_token_ids: torch.Tensor, experts_ids: torch.Tensor,
                                 num_tokens_post_pad: torch.Tensor) -> None:
    """``moe_align_block_size`` for callers that cannot allocate device memory or pass scratch.

    Same outputs; the kernels' working counters live in a fixed array inside the library
    instead of a caller buffer, so the call itself allocates nothing (no cudaMalloc, no torch
    allocation).  Meant for hosts whose GPU memory is fully committed (a serving worker after
    its KV cache is sized) or that must avoid the device-wide stall of an allocation.  At most
    ``NOALLOC_MAX_SLOTS`` slots and ``NOALLOC_MAX_EXPERTS`` experts; larger inputs raise.  All
    calls on a device share the array, so keep them on one stream; make the first call on a
    device outside any stream capture."""
    N.require_cuda(topk_ids, sorted_token_ids, experts_ids, num_tokens_post_pad)
    if sorted_token_ids.dtype != torch.int32 or experts_ids.dtype != torch.int32 or num_tokens_post_pad.dtype != torch.int32:
        raise RuntimeError("moe_align_block_size_noalloc: outputs must be int32")
    if not (topk_ids.is_contiguous() and sorted_token_ids.is_contiguous() and experts_ids.is_contiguous()):
        raise RuntimeError("moe_align_block_size_noalloc: tensors must be contiguous")
    N.check(N.lib().sb200_moe_align_block_size_noalloc(N.ptr(topk_ids), N.itype_id(topk_ids), topk_ids.numel(),
                                                       int(num_experts), int(block_size), N.ptr(sorted_token_ids),
                                                       sorted_token_ids.numel(), N.ptr(experts_ids),
                                                       experts_ids.numel(), N.ptr(num_tokens_post_pad),
                                                       N.stream_ptr()), "moe_align_block_size_noalloc")
