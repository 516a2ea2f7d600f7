"""Vocabulary-parallel embedding lookup behind the C ABI (no counterpart among the reference's pybind
modules: the reference builds it from torch ops, tensor_parallel/layers.py:147-168)."""
import torch

from . import _native as N


def vocab_embedding(out: torch.Tensor, ids: torch.Tensor, weight: torch.Tensor, vocab_start: int,
                    vocab_end: int) -> None:
    """out[t, :] <- weight[ids[t] - vocab_start, :] if vocab_start <= ids[t] < vocab_end else 0."""
    N.require_cuda(out, ids, weight)
    if ids.dtype != torch.int64 or not ids.is_contiguous():
        raise RuntimeError("vocab_embedding: ids must be a contiguous int64 tensor")
    if not (out.is_contiguous() and weight.is_contiguous()) or out.dtype != weight.dtype:
        raise RuntimeError("vocab_embedding: out and weight must be contiguous and share a dtype")
    H = weight.shape[1]
    T = ids.numel()
    if out.numel() != T * H or weight.shape[0] != vocab_end - vocab_start:
        raise RuntimeError("vocab_embedding: shapes do not match")
    N.check(N.lib().sb200_vocab_embedding(N.ptr(out), N.ptr(ids), N.ptr(weight), T, H, int(vocab_start),
                                          int(vocab_end), N.dtype_id(weight), N.stream_ptr()), "vocab_embedding")
