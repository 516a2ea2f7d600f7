"""Tensor-parallel (and pipeline-parallel) group bookkeeping with the accessor names the
reference's layers read (sarathi/model_executor/parallel_utils/parallel_state.py:49-215,
235-330,398-470,512-537).  The tensor-parallel group carries this package's path; the
pipeline-parallel group exists for the stage hand-off (pipeline_mappings.send / recv) and is
only created when its size is above 1.  Data and embedding groups are outside this package's path."""
from __future__ import annotations

from typing import Optional


_TP_GROUP = None
_TP_RANKS = None
_TP_WORLD_SIZE_OVERRIDE: Optional[int] = None
_TP_RANK_OVERRIDE: Optional[int] = None
_TP_COMM = None
_INITIALISED = False
_PP_GROUP = None
_PP_RANKS = None
# The reference's own parallel_state module, when this package runs underneath the reference's model_executor
# (sarathi_serve_b200.install): group, rank and size are then read from there.
_FOLLOWED = None


def follow(reference_parallel_state) -> None:
    """Read the tensor-parallel group / rank / size from another module with the reference's accessor names
    (``get_tensor_model_parallel_{group,rank,world_size}``, ``model_parallel_is_initialized``); ``None`` stops that."""
    global _FOLLOWED, _TP_COMM
    if _TP_COMM is not None and reference_parallel_state is not _FOLLOWED:
        _TP_COMM.close()
        _TP_COMM = None
    _FOLLOWED = reference_parallel_state


def _following() -> bool:
    return _FOLLOWED is not None and _FOLLOWED.model_parallel_is_initialized()

# Largest [T, H] batch (bytes) a collective of the shared context may carry.
DEFAULT_COMM_REGION_BYTES = 64 << 20


def default_comm_region_bytes() -> int:
    """``DEFAULT_COMM_REGION_BYTES``, or SB200_COMM_REGION_BYTES from the environment (a worker sets it to
    max_num_batched_tokens * hidden_size * itemsize when that exceeds 64 MiB; every rank the same)."""
    import os
    v = os.environ.get("SB200_COMM_REGION_BYTES")
    return max(int(v), 1 << 20) if v else DEFAULT_COMM_REGION_BYTES


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1,
                              virtual_pipeline_model_parallel_size=None,
                              pipeline_model_parallel_split_rank=None) -> None:
    """Create the tensor-parallel group(s): consecutive blocks of ``tensor_model_parallel_size`` ranks
    (reference: parallel_state.py:147-158).  Works without torch.distributed when the size is 1."""
    global _TP_GROUP, _TP_RANKS, _INITIALISED, _PP_GROUP, _PP_RANKS
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized():
        if tensor_model_parallel_size != 1 or pipeline_model_parallel_size != 1:
            raise RuntimeError("torch.distributed must be initialised for model-parallel sizes > 1")
        _TP_GROUP, _TP_RANKS, _INITIALISED = None, [0], True
        return
    world = dist.get_world_size()
    if world % (tensor_model_parallel_size * pipeline_model_parallel_size) != 0:
        raise RuntimeError(f"world size {world} is not divisible by tensor parallel size {tensor_model_parallel_size} "
                           f"x pipeline parallel size {pipeline_model_parallel_size}")
    assert _TP_GROUP is None or not _INITIALISED, "tensor model parallel group is already initialized"
    rank = dist.get_rank()
    for i in range(world // tensor_model_parallel_size):
        ranks = list(range(i * tensor_model_parallel_size, (i + 1) * tensor_model_parallel_size))
        group = dist.new_group(ranks)
        if rank in ranks:
            _TP_GROUP, _TP_RANKS = group, ranks
    if pipeline_model_parallel_size > 1:
        # stage s of pipeline i is global rank i + s * (world / pp): ranks a stride apart (reference:
        # parallel_state.py:160-170), so that the ranks of a tensor-parallel group stay neighbours
        num_pipelines = world // pipeline_model_parallel_size
        for i in range(num_pipelines):
            ranks = list(range(i, world, num_pipelines))
            group = dist.new_group(ranks)
            if rank in ranks:
                _PP_GROUP, _PP_RANKS = group, ranks
    _INITIALISED = True


def model_parallel_is_initialized() -> bool:
    return _INITIALISED or _following()


def get_tensor_model_parallel_group():
    if _following():
        return _FOLLOWED.get_tensor_model_parallel_group()
    assert _INITIALISED, "tensor model parallel group is not initialized"
    return _TP_GROUP


def set_tensor_model_parallel_world_size(world_size: Optional[int]) -> None:
    global _TP_WORLD_SIZE_OVERRIDE
    _TP_WORLD_SIZE_OVERRIDE = world_size


def set_tensor_model_parallel_rank(rank: Optional[int]) -> None:
    global _TP_RANK_OVERRIDE
    _TP_RANK_OVERRIDE = rank


def get_tensor_model_parallel_world_size() -> int:
    if _TP_WORLD_SIZE_OVERRIDE is not None:
        return _TP_WORLD_SIZE_OVERRIDE
    if _following():
        return _FOLLOWED.get_tensor_model_parallel_world_size()
    if not _INITIALISED or _TP_GROUP is None:
        return 1 if _TP_RANKS is None else len(_TP_RANKS)
    import torch.distributed as dist
    return dist.get_world_size(group=_TP_GROUP)


def get_tensor_model_parallel_rank() -> int:
    if _TP_RANK_OVERRIDE is not None:
        return _TP_RANK_OVERRIDE
    if _following():
        return _FOLLOWED.get_tensor_model_parallel_rank()
    if not _INITIALISED or _TP_GROUP is None:
        return 0
    import torch.distributed as dist
    return dist.get_rank(group=_TP_GROUP)


def get_tensor_model_parallel_src_rank() -> int:
    return 0 if _TP_RANKS is None else _TP_RANKS[0]


def get_pipeline_model_parallel_group():
    """The group of the pipeline this rank is a stage of, or None when there is a single stage."""
    assert _INITIALISED, "pipeline model parallel group is not initialized"
    return _PP_GROUP


def get_pipeline_model_parallel_world_size() -> int:
    return 1 if _PP_RANKS is None else len(_PP_RANKS)


def get_pipeline_model_parallel_rank() -> int:
    if _PP_RANKS is None:
        return 0
    import torch.distributed as dist
    return _PP_RANKS.index(dist.get_rank())


def is_pipeline_first_stage() -> bool:
    return get_pipeline_model_parallel_rank() == 0


def is_pipeline_last_stage() -> bool:
    return get_pipeline_model_parallel_rank() == get_pipeline_model_parallel_world_size() - 1


def get_pipeline_model_parallel_next_rank() -> int:
    """Global rank of the next stage (the last stage wraps to the first; reference: parallel_state.py:448-453)."""
    assert _PP_RANKS is not None, "pipeline parallel group is not initialized"
    return _PP_RANKS[(get_pipeline_model_parallel_rank() + 1) % len(_PP_RANKS)]


def get_pipeline_model_parallel_prev_rank() -> int:
    assert _PP_RANKS is not None, "pipeline parallel group is not initialized"
    return _PP_RANKS[(get_pipeline_model_parallel_rank() - 1) % len(_PP_RANKS)]


def get_tensor_model_parallel_comm(region_bytes: Optional[int] = None):
    """The process-wide communication context of the tensor-parallel group
    (created on first use; every rank must reach this call together)."""
    global _TP_COMM
    if _TP_COMM is None:
        from .comm import TPComm
        _TP_COMM = TPComm(get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size(),
                          region_bytes or default_comm_region_bytes(),
                          group=get_tensor_model_parallel_group() if model_parallel_is_initialized() else None)
    elif region_bytes is not None and region_bytes > _TP_COMM.region_bytes:
        raise RuntimeError(f"the tensor-parallel context was created with {_TP_COMM.region_bytes} byte regions; "
                           f"{region_bytes} requested -- create it first with the larger size")
    return _TP_COMM


def destroy_model_parallel() -> None:
    global _TP_GROUP, _TP_RANKS, _TP_COMM, _INITIALISED, _TP_WORLD_SIZE_OVERRIDE, _TP_RANK_OVERRIDE, _PP_GROUP, _PP_RANKS
    if _TP_COMM is not None:
        _TP_COMM.close()
    _TP_GROUP = _TP_RANKS = _TP_COMM = None
    _PP_GROUP = _PP_RANKS = None
    _TP_WORLD_SIZE_OVERRIDE = _TP_RANK_OVERRIDE = None
    _INITIALISED = False
