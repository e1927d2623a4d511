"""LIFO allocator of KV-pool chunk ids.

Same contract as the reference's ``ChunkAllocator``
(``megatron/core/inference/contexts/dynamic_chunk_allocator.py:9-92``): the pool is a stack held in
``chunk_bag``; allocating n chunks pops the top n entries (returned bottom-to-top), releasing pushes
them back in the order given; the last chunk id is reserved as the dummy chunk that padding tokens
write to.  The stack lives on the host: it is touched a few times per step with a handful of ids, and
keeping it next to the request bookkeeping avoids device round trips.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


class ChunkAllocator:
    def __init__(self, chunk_count_total: int, gtd_chunk_count: int):
        self.chunk_count_total = chunk_count_total
        self.gtd_chunk_count = gtd_chunk_count
        self.chunk_count_avail = chunk_count_total - 1
        self.dummy_chunk_idx = chunk_count_total - 1
        self.chunk_bag = torch.arange(chunk_count_total, dtype=torch.int32)
        self._bag = self.chunk_bag.numpy()  # zero-copy view for the hot path

    def is_memory_available(self, num_chunks: int, safe: bool = False) -> bool:
        """``safe`` keeps the guaranteed-request reserve untouched."""
        if safe:
            return self.chunk_count_avail >= num_chunks + self.gtd_chunk_count
        return self.chunk_count_avail >= num_chunks

    def allocate_memory_chunks(self, num_chunks: int = 1, safe: bool = False) -> Optional[torch.Tensor]:
        """Pop ``num_chunks`` ids, or return None when they are not available."""
        if not self.is_memory_available(num_chunks, safe):
            return None
        self.chunk_count_avail -= num_chunks
        return self.chunk_bag[self.chunk_count_avail : self.chunk_count_avail + num_chunks].clone()

    def release_memory_chunks(self, chunks) -> None:
        """Push ids back (accepts a tensor on any device, an array or a list)."""
        if isinstance(chunks, torch.Tensor):
            chunks = chunks.detach().cpu().numpy()
        chunks = np.asarray(chunks, dtype=np.int32).reshape(-1)
        n = chunks.shape[0]
        self._bag[self.chunk_count_avail : self.chunk_count_avail + n] = chunks
        self.chunk_count_avail += n

    def reset(self) -> None:
        """All chunks but the dummy one become available again (ids keep their current order)."""
        self.chunk_count_avail = self.chunk_count_total - 1
