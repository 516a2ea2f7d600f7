"""The tensor-parallel region mappings of the reference
(sarathi/model_executor/parallel_utils/tensor_parallel/mappings.py:266-279) as
plain inference-time functions.  The all-reduce runs this library's own kernels
over the symmetric heaps (comm.py); the all-gather, which is not on the decoder
layer path, goes through torch.distributed."""
from __future__ import annotations

import torch

from . import parallel_state as ps


def divide(numerator: int, denominator: int) -> int:
    """Exact division (reference: tensor_parallel/utils.py:10-21); raises AssertionError otherwise."""
    assert numerator % denominator == 0, "{} is not divisible by {}".format(numerator, denominator)
    return numerator // denominator


def copy_to_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return input_


def reduce_from_tensor_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """In-place sum over the tensor-parallel group; returns its argument (mappings.py:16-26)."""
    if ps.get_tensor_model_parallel_world_size() == 1:
        return input_
    if not input_.is_contiguous():
        raise RuntimeError("reduce_from_tensor_model_parallel_region: tensor must be contiguous")
    flat = input_.view(-1, input_.shape[-1])
    comm = ps.get_tensor_model_parallel_comm()
    comm.all_reduce(flat, out=flat)
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
    """Concatenate the ranks' shards along the last dimension (mappings.py:71-92)."""
    world = ps.get_tensor_model_parallel_world_size()
    if world == 1:
        return input_
    import torch.distributed as dist
    parts = [torch.empty_like(input_) for _ in range(world)]
    dist.all_gather(parts, input_.contiguous(), group=ps.get_tensor_model_parallel_group())
    return torch.cat(parts, dim=-1).contiguous()
