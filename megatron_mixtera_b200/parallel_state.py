"""Tensor-parallel process-group state (the slice of the reference's
``megatron/core/parallel_state.py`` that the decode path uses: TP group, rank and size)."""
from __future__ import annotations

from typing import Optional

import torch

_TP_GROUP = None
_TP_SIZE = 1
_TP_RANK = 0
_INITIALIZED = False


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1, **_) -> None:
    """Create the tensor-parallel group.  ``torch.distributed`` must be initialised when size > 1;
    ranks are grouped contiguously (rank // tp_size), as the reference does."""
    global _TP_GROUP, _TP_SIZE, _TP_RANK, _INITIALIZED
    if pipeline_model_parallel_size != 1:
        raise NotImplementedError("pipeline parallelism is outside the decode path built here")
    tp = int(tensor_model_parallel_size)
    if tp > 1:
        import torch.distributed as dist

        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before initialize_model_parallel(tp > 1)")
        world, rank = dist.get_world_size(), dist.get_rank()
        if world % tp != 0:
            raise RuntimeError(f"world size {world} is not divisible by tensor parallel size {tp}")
        for g in range(world // tp):
            ranks = list(range(g * tp, (g + 1) * tp))
            group = dist.new_group(ranks)
            if rank in ranks:
                _TP_GROUP, _TP_RANK = group, rank - g * tp
    else:
        _TP_GROUP, _TP_RANK = None, 0
    _TP_SIZE = tp
    _INITIALIZED = True


def is_initialized() -> bool:
    return _INITIALIZED


def destroy_model_parallel() -> None:
    global _TP_GROUP, _TP_SIZE, _TP_RANK, _INITIALIZED
    _TP_GROUP, _TP_SIZE, _TP_RANK, _INITIALIZED = None, 1, 0, False


def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE


def get_tensor_model_parallel_rank() -> int:
    return _TP_RANK


def get_tensor_model_parallel_group():
    return _TP_GROUP


def _world_and_rank():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def get_data_parallel_world_size() -> int:
    """Number of model replicas: the ranks that are not inside one tensor-parallel group (serving plumbing only)."""
    world, _ = _world_and_rank()
    return max(1, world // _TP_SIZE)


def get_data_parallel_rank() -> int:
    """Index of this rank's replica (ranks are grouped contiguously into tensor-parallel groups)."""
    _, rank = _world_and_rank()
    return rank // _TP_SIZE


def get_pipeline_model_parallel_rank() -> int:
    return 0


def get_pipeline_model_parallel_world_size() -> int:
    return 1


def is_pipeline_first_stage(*_, **__) -> bool:
    """There is one pipeline stage (pipeline parallelism is outside this path): it is first and last."""
    return True


def is_pipeline_last_stage(*_, **__) -> bool:
    return True


def model_parallel_is_initialized() -> bool:
    """The reference's older name of `is_initialized`."""
    return _INITIALIZED


def get_pipeline_model_parallel_group():
    """No process group: a single pipeline stage has nobody to talk to."""
    return None
