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
    """A row-parallel output that still has to be summed over the ranks: lives in slot ``slot`` of the peer buffers, or
    (two-shot form, ``partials``) is still the GEMM's split-K partial sums, which the exchange kernel sums into the
    buffer itself."""

    __slots__ = ("comm", "slot", "shape", "partials")

    def __init__(self, comm: "PeerAllReduce", slot: int, shape, partials=None):
        self.comm, self.slot, self.shape, self.partials = comm, slot, tuple(shape), partials


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

    two_shot = False

    def begin_forward(self) -> None:
        """Called where a forward pass starts (and its CUDA graph, if any): see `end_forward`."""
        self._slot_at_entry = self._next_slot

    def end_forward(self) -> None:
        """The handshake only fences the call after next, so consecutive calls must use different slots - also across
        replays of one captured forward, whose slots are baked in.  That holds iff a forward makes an even number of
        calls (it then ends on the slot it did not start with): two per decoder layer.  Anything else is refused."""
        if self._next_slot != getattr(self, "_slot_at_entry", self._next_slot):
            raise RuntimeError("a forward pass made an odd number of fused all-reduce calls: replays of its CUDA graph "
                               "would use the same peer slot twice in a row; use the two-shot exchange or NCCL")

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


class PeerExchange:
    """Two-shot form: peer buffers for the ranks' partial outputs AND for the finished rows.  Every rank reduces,
    normalises and (for an FP8 recipe) quantises only its share of the token rows and stores them into all ranks'
    output buffers (`b200_allreduce2_add_norm`).  The results of a call live in this object's buffers until the next
    call overwrites them: `hidden` (the residual stream) is rewritten in place row by row, the normalised rows are
    consumed by the linear that follows.  Creation is a collective."""

    two_shot = True

    def begin_forward(self) -> None:  # one buffer, two flag exchanges per call: any number of calls per forward is safe
        pass

    end_forward = begin_forward

    def __init__(self, group, rank: int, world_size: int, max_rows: int, hidden: int, device: torch.device):
        import torch.distributed as dist

        if not 2 <= world_size <= 8:
            raise ValueError("peer exchange supports 2..8 ranks")
        self.group, self.rank, self.world_size = group, rank, world_size
        self.max_rows, self.hidden, self.device = int(max_rows), int(hidden), device
        lib = _lib.load()
        self._lib = lib
        self.m_pad = (self.max_rows + 3) // 4 * 4
        row_bytes = self.max_rows * self.hidden
        sf_bytes = max(lib.b200_mxfp8_scale_bytes(self.max_rows, self.hidden) if self.hidden % 128 == 0 else 0,
                       (self.hidden // 128) * self.m_pad * 4, 16)
        # in (bf16), hidden_out (bf16), normed_out (bf16 or E4M3 bytes), scales_out, flags (2 x 8 int32, one 128-byte line each way)
        self._sizes = (2 * row_bytes, 2 * row_bytes, 2 * row_bytes, sf_bytes, 256)
        self._own, handles = [], []
        for nbytes in self._sizes:
            ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _lib.check("b200_peer_buffer_create", lib.b200_peer_buffer_create(nbytes, ctypes.byref(ptr), handle))
            self._own.append(ptr.value)
            handles.append(handle.raw)
        gathered = [None] * world_size
        dist.all_gather_object(gathered, tuple(handles), group=group)
        self._opened = []
        comm = _lib.TpExchange()
        comm.world_size, comm.rank, comm.max_rows, comm.hidden, comm.m_pad = world_size, rank, self.max_rows, self.hidden, self.m_pad
        for r in range(world_size):
            if r == rank:
                ptrs = list(self._own)
            else:
                ptrs = []
                for h in gathered[r]:
                    ptr = ctypes.c_void_p()
                    _lib.check("b200_peer_buffer_open", lib.b200_peer_buffer_open(h, ctypes.byref(ptr)))
                    ptrs.append(ptr.value)
                    self._opened.append(ptr.value)
            comm.in_[r], comm.hidden_out[r], comm.normed_out[r], comm.scales_out[r], comm.flags[r] = ptrs
        self._counters = torch.zeros(4, dtype=torch.int32, device=device)
        comm.counters = self._counters.data_ptr()
        self.comm = comm
        wrap = lambda i: torch.as_tensor(_DeviceBytes(self._own[i], self._sizes[i]), device=device)
        self._in = wrap(0).view(torch.bfloat16)
        self._hidden = wrap(1).view(torch.bfloat16)
        self._normed = wrap(2)
        self._scales = wrap(3)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone uses them

    def output_slot(self, rows: int):
        """(0, [rows, hidden] bf16 view of this rank's input buffer): where the row-parallel GEMM writes."""
        assert rows <= self.max_rows
        return 0, self._in[: rows * self.hidden].view(rows, self.hidden)

    def accepts_partials(self, rows: int) -> bool:
        """Whether the exchange kernel may be given split-K partial sums for this many rows: its grid (one CTA per owned
        row) must be resident at once, because the peers wait for all of its CTAs."""
        return SPLITK_INTO_EXCHANGE and -(-rows // self.world_size) <= 128

    def hidden_view(self, shape):
        n = 1
        for d in shape:
            n *= d
        return self._hidden[:n].view(shape)

    def normed_view(self, rows: int, quantize, shape):
        """The local copy of the finished normalised rows: bf16 tensor, `ops.Mxfp8Tensor` or `ops.Fp8BlockTensor`."""
        from .. import ops

        H = self.hidden
        if quantize == "mxfp8":
            nbytes = self._lib.b200_mxfp8_scale_bytes(rows, H)
            return ops.Mxfp8Tensor(self._normed[: rows * H].view(rows, H), self._scales[:nbytes], shape)
        if quantize == "blockwise":
            scale = self._scales[: (H // 128) * self.m_pad * 4].view(torch.float32).view(H // 128, self.m_pad)
            return ops.Fp8BlockTensor(self._normed[: rows * H].view(rows, H), scale, shape, self.m_pad)
        return self._normed[: rows * H * 2].view(torch.bfloat16).view(shape)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self._lib.b200_peer_buffer_close(p)
        for p in self._own:
            self._lib.b200_peer_buffer_destroy(p)
        self._opened, self._own = [], []


_COMMS = {}  # form ("one_shot" | "two_shot") -> communicator of the tensor-parallel group


# Hand the split-K partial sums of a row-parallel GEMM to the two-shot exchange kernel instead of launching the GEMM's
# reduction kernel.  Same bits, one launch fewer; off by default: measured slower at 4 ranks (the sums then sit on the
# critical path in front of the first flag exchange instead of overlapping with the GEMM's tail).
SPLITK_INTO_EXCHANGE = False

# One-shot form (every rank pulls every peer's rows: one flag exchange, no end-of-call exchange, w - 1 times the data per
# rank) or two-shot form (two exchanges, 2 (w - 1) / w of the data per rank)?  One-shot for groups of up to
# ONE_SHOT_MAX_WORLD ranks while a rank pulls at most ONE_SHOT_MAX_BYTES per call.  Measured per call (collective + add +
# norm, B200, NVLink 5): 128 x 4096 bf16 at 2 ranks 8 us one-shot / 18 us two-shot, at 4 ranks 12 / 17 us (3 MB pulled);
# 256 x 8192 at 2 ranks 17 / 22 us (4 MB), at 4 ranks 29 / 27 us (12 MB).
ONE_SHOT_MAX_WORLD = 8
ONE_SHOT_MAX_BYTES = 8 << 20


def use_one_shot(world: int, rows: int, hidden: int) -> bool:
    return world <= ONE_SHOT_MAX_WORLD and (world - 1) * rows * hidden * 2 <= ONE_SHOT_MAX_BYTES


def get_peer_allreduce(hidden: int, rows: int, max_rows: int = 512):
    """The group's communicator for this output (created on first use: a collective, so every rank must get here
    together - the choice of form depends only on sizes every rank knows), or None when this output cannot go through
    one (more rows than a buffer holds, a different width, capture in progress before the first eager use)."""
    from .. import parallel_state

    tp = parallel_state.get_tensor_model_parallel_world_size()
    if tp < 2 or tp > 8 or rows > max_rows or hidden > 8192 or hidden % 8 != 0 or not torch.cuda.is_available():
        return None
    form = "one_shot" if use_one_shot(tp, rows, hidden) else "two_shot"
    comm = _COMMS.get(form)
    if comm is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        dev = torch.device("cuda", torch.cuda.current_device())
        cls = PeerAllReduce if form == "one_shot" else PeerExchange
        comm = _COMMS[form] = cls(parallel_state.get_tensor_model_parallel_group(),
                                  parallel_state.get_tensor_model_parallel_rank(), tp, max_rows, hidden, dev)
    return comm if comm.hidden == hidden else None


def begin_forward() -> dict:
    """Called where a forward pass (and its CUDA graph, if any) starts; returns what `end_forward` needs."""
    for comm in _COMMS.values():
        comm.begin_forward()
    return dict(_COMMS)


def end_forward(at_entry: dict) -> None:
    """Checks the slot discipline of the communicators that existed when the forward started (one created during the
    forward started on slot 0 and is checked against that)."""
    for form, comm in _COMMS.items():
        if form not in at_entry:
            comm._slot_at_entry = 0
        comm.end_forward()


def destroy_peer_allreduce() -> None:
    for comm in list(_COMMS.values()):
        comm.close()
    _COMMS.clear()
