"""The tensor-parallel region mappings of the reference
(sarathi/model_executor/parallel_utils/tensor_parallel/mappings.py:266-279) as
plain inference-time functions.  The all-reduce and the all-gather run this
library's own kernels over the symmetric heaps (comm.py)."""
from __future__ import annotations

import torch

from . import parallel_state as ps


def divide(numerator: int, denominator: int) -> int:
    """Exact division (reference: tensor_parallel/utils.py:10-21); raises AssertionError otherwise."""
    assert numerator % denominator == 0, "{} is not divisible by {}".format(numerator, denominator)
    return numerator // denominator


_MAX_ROW_BYTES = 32 * 1024


def _regroup_width(numel: int, es: int) -> int:
    """Largest row length (elements) with 16-byte-multiple rows of at most 32 KiB that divides ``numel``; 0 if none."""
    step = 16 // es
    if numel % step != 0:
        return 0
    w = min(numel, _MAX_ROW_BYTES // es) // step * step
    while w >= step:
        if numel % w == 0:
            return w
        w -= step
    return 0


def copy_to_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return input_


def reduce_from_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """In-place sum over the tensor-parallel group; returns its argument (mappings.py:16-26)."""
    if ps.get_tensor_model_parallel_world_size() == 1:
        return input_
    if not input_.is_contiguous():
        raise RuntimeError("reduce_from_tensor_model_parallel_region: tensor must be contiguous")
    es = input_.element_size()
    width = input_.shape[-1]
    if (width * es) % 16 != 0 or width * es > _MAX_ROW_BYTES:
        # The kernels move whole 16-byte vectors of rows of at most 32 KiB.  An element-wise sum does not care
        # about the row structure: regroup the elements into rows the kernels take, or, when the tensor's size
        # itself is not a multiple of 16 bytes, leave this (off-path) call to torch.distributed.
        width = _regroup_width(input_.numel(), es)
        if width == 0:
            import torch.distributed as dist
            dist.all_reduce(input_, group=ps.get_tensor_model_parallel_group())
            return input_
    flat = input_.view(-1, width)
    es_total = flat.shape[0] * width * es
    comm = ps.get_tensor_model_parallel_comm(max(es_total, ps.default_comm_region_bytes())
                                             if ps._TP_COMM is None else None)
    rows_per_call = max(1, comm.region_bytes // (width * es) // comm.world * comm.world)
    for r0 in range(0, flat.shape[0], rows_per_call):  # batches larger than the context's regions go in slices
        part = flat[r0:r0 + rows_per_call]
        comm.all_reduce(part, out=part)
    return input_


def scatter_to_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """Keep this rank's slice of the last dimension (mappings.py:29-45)."""
    world = ps.get_tensor_model_parallel_world_size()
    if world == 1:
        return input_
    size = divide(input_.shape[-1], world)
    rank = ps.get_tensor_model_parallel_rank()
    return input_[..., rank * size:(rank + 1) * size].contiguous()


def gather_from_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """Concatenate the ranks' shards along the last dimension (mappings.py:71-92), e.g. the vocabulary slices of
    the logits (layers/sampler.py:89-97).  Every rank's shard travels as one block of this library's all-gather
    (multicast stores or peer loads over NVLink, comm.py); the blocks are then interleaved locally.  Shards whose
    size is not a multiple of 16 bytes go through torch.distributed."""
    world = ps.get_tensor_model_parallel_world_size()
    if world == 1:
        return input_
    shard = input_.contiguous()
    es = shard.element_size()
    width = _regroup_width(shard.numel(), es)
    if width == 0 or not shard.is_cuda:
        import torch.distributed as dist
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard, group=ps.get_tensor_model_parallel_group())
        return torch.cat(parts, dim=-1).contiguous()
    rows = shard.numel() // width
    need = world * shard.numel() * es
    comm = ps.get_tensor_model_parallel_comm(max(need, ps.default_comm_region_bytes()) if ps._TP_COMM is None else None)
    if need > comm.region_bytes:
        raise RuntimeError(f"gather_from_tensor_model_parallel_region: {need} bytes exceed the communication context's "
                           f"regions ({comm.region_bytes}); create the context with a larger size first")
    full = comm.all_gather_rows(shard.view(rows, width), world * rows)     # [world * rows, width]: rank-major blocks
    blocks = full.view(world, *shard.shape)                                # [world, ..., d]
    return torch.cat(list(blocks.unbind(0)), dim=-1)                       # [..., world * d], a new tensor
