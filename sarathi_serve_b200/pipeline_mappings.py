"""Hand-off of the hidden states between pipeline stages, with the reference's function names
(sarathi/model_executor/parallel_utils/pipeline_parallel/mappings.py:12-41; called by the model's forward at
models/llama.py:347-359).  As in the reference these are plain ``torch.distributed`` point-to-point calls on the
pipeline group (NCCL between GPUs, which on one node is a copy over NVLink); there is no kernel of this package
on this row -- the stage boundary moves one [T, H] tensor per step, outside the tensor-parallel layer path."""
from __future__ import annotations

import torch

from . import parallel_state as ps


def send(hidden_states: torch.Tensor) -> torch.Tensor:
    """Send the hidden states to the next pipeline stage (nothing to do with a single stage)."""
    if ps.get_pipeline_model_parallel_world_size() == 1:
        return hidden_states
    import torch.distributed as dist
    dist.send(tensor=hidden_states, dst=ps.get_pipeline_model_parallel_next_rank(),
              group=ps.get_pipeline_model_parallel_group())
    return hidden_states


def recv(hidden_states: torch.Tensor) -> torch.Tensor:
    """Receive the previous stage's hidden states into ``hidden_states`` (same shape and dtype on both sides)."""
    if ps.get_pipeline_model_parallel_world_size() == 1:
        return hidden_states
    import torch.distributed as dist
    dist.recv(tensor=hidden_states, src=ps.get_pipeline_model_parallel_prev_rank(),
              group=ps.get_pipeline_model_parallel_group())
    return hidden_states
