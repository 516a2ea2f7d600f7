"""Drop-in for the reference's pybind module ``sarathi.pos_encoding_ops``
(csrc/pos_encoding.cpp:3-15)."""
import torch

from . import _native as N


def rotary_embedding(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor, head_size: int,
                     cos_sin_cache: torch.Tensor, is_neox: bool) -> None:
    """Rotate query [T, nq*head_size] and key [T, nkv*head_size] in place
    (csrc/pos_encoding_kernels.cu:80-127).  Row strides are taken from the
    tensors, so views into a fused qkv buffer work as in the reference."""
    N.require_cuda(positions, query, key, cos_sin_cache)
    if positions.dtype != torch.int64:
        raise RuntimeError("rotary_embedding: positions must be int64")
    if query.dim() != 2 or key.dim() != 2 or query.stride(1) != 1 or key.stride(1) != 1:
        raise RuntimeError("rotary_embedding: query/key must be 2-D with unit inner stride")
    if query.dtype != key.dtype or cos_sin_cache.dtype != query.dtype:
        raise RuntimeError("rotary_embedding: dtype mismatch")
    if not (cos_sin_cache.is_contiguous() and positions.is_contiguous()):
        raise RuntimeError("rotary_embedding: positions and cos_sin_cache must be contiguous")
    T = query.shape[0]
    rot_dim = cos_sin_cache.shape[1]
    nq = query.shape[1] // head_size
    nkv = key.shape[1] // head_size
    N.check(N.lib().sb200_rotary_embedding(N.ptr(positions), N.ptr(query), N.ptr(key), T, nq, nkv, head_size,
                                           rot_dim, query.stride(0), key.stride(0), N.ptr(cos_sin_cache),
                                           1 if is_neox else 0, N.dtype_id(query), N.stream_ptr()),
            "rotary_embedding")
