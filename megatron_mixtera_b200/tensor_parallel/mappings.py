"""Forward-only tensor-parallel collectives (reference ``megatron/core/tensor_parallel/mappings.py:22-33,
80-96``): NCCL all-reduce / all-gather over the TP group via ``torch.distributed``."""
from __future__ import annotations

import torch

from .. import parallel_state


def reduce_from_tensor_model_parallel_region(x: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the TP group (identity at TP=1)."""
    if parallel_state.get_tensor_model_parallel_world_size() == 1:
        return x
    torch.distributed.all_reduce(x, group=group or parallel_state.get_tensor_model_parallel_group())
    return x


def gather_from_tensor_model_parallel_region(x: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate the last dimension over the TP group (identity at TP=1)."""
    tp = parallel_state.get_tensor_model_parallel_world_size()
    if tp == 1:
        return x
    group = group or parallel_state.get_tensor_model_parallel_group()
    x = x.contiguous()
    out = torch.empty((tp * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)  # rank-major along dim 0
    torch.distributed.all_gather_into_tensor(out, x, group=group)
    # [tp, ..., n] -> [..., tp * n]
    return out.view(tp, *x.shape).movedim(0, -2).reshape(*x.shape[:-1], tp * x.shape[-1])
