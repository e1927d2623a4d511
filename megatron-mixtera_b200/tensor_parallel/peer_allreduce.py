"""All-reduce of a row-parallel linear's output fused into the residual-add + norm kernel.

The reference reduces the partial outputs of ``RowParallelLinear`` with an NCCL all-reduce
(``megatron/core/tensor_parallel/mappings.py:22-33``) and then runs bias-dropout-add and the next norm as separate
kernels.  Here every tensor-parallel rank of the node writes its bf16 partial output into a buffer that the other
ranks map through CUDA IPC, and the norm kernel itself synchronises per token row (flags in peer memory, bounded
waits) and sums the ranks' rows with plain peer loads over NVLink - one kernel for collective + add + norm, no
NCCL launch.  All ranks compute the same bits (fixed rank order, fp32 sum, one bf16 rounding).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib


class _DeviceBytes:
    """Lets torch wrap device memory that was not allocated by its own allocator."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class TpPending:
    """A row-parallel output that still has to be summed over the ranks: lives in slot ``slot`` of the peer buffers."""

    __slots__ = ("comm", "slot", "shape")

    def __init__(self, comm: "PeerAllReduce", slot: int, shape):
        self.comm, self.slot, self.shape = comm, slot, tuple(shape)


class PeerAllReduce:
    """Peer buffers of one tensor-parallel group (all ranks on one node).  Creation is a collective."""

    def __init__(self, group, rank: int, world_size: int, max_rows: int, hidden: int, device: torch.device):
        import torch.distributed as dist

        if not 2 <= world_size <= 8:
            raise ValueError("peer all-reduce supports 2..8 ranks")
        self.group, self.rank, self.world_size = group, rank, world_size
        self.max_rows, self.hidden, self.device = int(max_rows), int(hidden), device
        lib = _lib.load()
        self._lib = lib
        self._slot_bytes = self.max_rows * self.hidden * 2
        sizes = (2 * self._slot_bytes, world_size * self.max_rows * 4)
        self._own, handles = [], []
        for nbytes in sizes:
            ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _lib.check("b200_peer_buffer_create", lib.b200_peer_buffer_create(nbytes, ctypes.byref(ptr), handle))
            self._own.append(ptr.value)
            handles.append(handle.raw)
        gathered = [None] * world_size
        dist.all_gather_object(gathered, tuple(handles), group=group)
        self._opened = []
        comm = _lib.TpComm()
        comm.world_size, comm.rank, comm.max_rows, comm.hidden = world_size, rank, self.max_rows, self.hidden
        for r in range(world_size):
            if r == rank:
                comm.data[r], comm.flags[r] = self._own[0], self._own[1]
                continue
            ptrs = []
            for h in gathered[r]:
                ptr = ctypes.c_void_p()
                _lib.check("b200_peer_buffer_open", lib.b200_peer_buffer_open(h, ctypes.byref(ptr)))
                ptrs.append(ptr.value)
                self._opened.append(ptr.value)
            comm.data[r], comm.flags[r] = ptrs
        self._counters = torch.zeros(2, dtype=torch.int32, device=device)
        comm.counters = self._counters.data_ptr()
        self.comm = comm
        self._local = torch.as_tensor(_DeviceBytes(self._own[0], sizes[0]), device=device).view(torch.bfloat16)
        self._next_slot = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone uses them

    def output_slot(self, rows: int):
        """(slot index, [rows, hidden] bf16 view of this rank's slot) for the next call; slots alternate."""
        assert rows <= self.max_rows
        slot = self._next_slot
        self._next_slot ^= 1
        base = slot * self.max_rows * self.hidden
        return slot, self._local[base : base + rows * self.hidden].view(rows, self.hidden)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self._lib.b200_peer_buffer_close(p)
        for p in self._own:
            self._lib.b200_peer_buffer_destroy(p)
        self._opened, self._own = [], []


_COMM: Optional[PeerAllReduce] = None


def get_peer_allreduce(hidden: int, rows: int, max_rows: int = 512, max_world: int = 4) -> Optional[PeerAllReduce]:
    """The group's communicator (created on first use: a collective, so every rank must get here together), or None
    when this output cannot go through it (more rows than a slot holds, a different width, capture in progress
    before the first eager use)."""
    from .. import parallel_state

    global _COMM
    tp = parallel_state.get_tensor_model_parallel_world_size()
    # Every rank pulls every peer's row: measured on config 1 the fused kernel wins at 2 ranks (4.44 vs 4.71 ms per
    # step), ties at 4 (4.00 vs 4.02) and loses at 8 (5.61 vs 4.17, where NCCL reduces inside the switch), so larger
    # groups stay on NCCL unless asked (`max_world`).
    if tp < 2 or tp > max_world or rows > max_rows or hidden > 8192 or hidden % 8 != 0 or not torch.cuda.is_available():
        return None
    if _COMM is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        dev = torch.device("cuda", torch.cuda.current_device())
        _COMM = PeerAllReduce(parallel_state.get_tensor_model_parallel_group(),
                              parallel_state.get_tensor_model_parallel_rank(), tp, max_rows, hidden, dev)
    return _COMM if _COMM.hidden == hidden else None


def destroy_peer_allreduce() -> None:
    global _COMM
    if _COMM is not None:
        _COMM.close()
        _COMM = None
