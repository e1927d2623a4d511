"""A device-side wait that runs out: the kernel returns, the status word says why, the context stays usable.

Nothing faults here.  A 2-rank communicator is built on ONE GPU out of local buffers; the flags that the other "rank"
would write are simply never written, so the wait for them reaches its limit (set to a few milliseconds for the test),
the kernel records status 4 (tensor-parallel peer), carries on with whatever the buffers hold and ends normally.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


@pytest.fixture()
def ops():
    from megatron_mixtera_b200 import build, ops as _ops

    build.build()
    torch.cuda.synchronize()
    assert _ops.device_status(reset=True) == 0
    yield _ops
    _ops.set_wait_limit_ns(2_000_000_000)  # back to the default for whatever runs next in this process
    torch.cuda.synchronize()
    _ops.device_status(reset=True)


def test_two_shot_exchange_gives_up_on_a_silent_peer(ops):
    from megatron_mixtera_b200 import _lib

    lib = _lib.load()
    rows, hidden = 8, 1024
    dev = "cuda"
    bufs = {k: [torch.zeros(rows * hidden, dtype=BF16, device=dev) for _ in range(2)] for k in ("in", "hid", "nrm")}
    scales = [torch.zeros(4096, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]  # nobody ever writes rank 1's announcements
    counters = torch.zeros(2, dtype=torch.int32, device=dev)
    comm = _lib.TpExchange()
    comm.world_size, comm.rank, comm.max_rows, comm.hidden, comm.m_pad = 2, 0, rows, hidden, rows
    comm.in_ = _ptr_array([t.data_ptr() for t in bufs["in"]])
    comm.hidden_out = _ptr_array([t.data_ptr() for t in bufs["hid"]])
    comm.normed_out = _ptr_array([t.data_ptr() for t in bufs["nrm"]])
    comm.scales_out = _ptr_array([t.data_ptr() for t in scales])
    comm.flags = _ptr_array([t.data_ptr() for t in flags])
    comm.counters = counters.data_ptr()
    gamma = torch.ones(hidden, dtype=BF16, device=dev)
    bufs["in"][0].fill_(1.0)
    ops.set_wait_limit_ns(3_000_000)  # 3 ms
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.b200_allreduce2_add_norm(ctypes.byref(comm), None, None, gamma.data_ptr(), None, 0, rows, hidden, 1e-5,
                                      torch.cuda.current_stream().cuda_stream)
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()  # the kernel ENDS: two waits of 3 ms each ran out (inputs ready / outputs stored)
    assert 2.0 < t0.elapsed_time(t1) < 500.0
    assert ops.device_status(reset=True) == 4
    assert int(counters[0]) == 1  # the call was completed and counted: the next call uses the next number
    # this rank's share of the rows (the first half) was still reduced from what the buffers held: 1 + 0
    assert torch.all(bufs["hid"][0].view(rows, hidden)[: rows // 2] == 1.0)
    # the context is usable: a healthy launch works and leaves the status word clean
    x = torch.randn(16, hidden, device=dev).to(BF16)
    _, y = ops.add_norm(x, gamma)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ref = torch.nn.functional.rms_norm(x.float(), (hidden,), gamma.float(), 1e-5)
    assert float((y.float() - ref).norm() / ref.norm()) < 1e-2


def test_one_shot_row_handshake_gives_up_on_a_silent_peer(ops):
    from megatron_mixtera_b200 import _lib

    lib = _lib.load()
    rows, hidden = 4, 512
    dev = "cuda"
    data = [torch.ones(2 * rows * hidden, dtype=BF16, device=dev) for _ in range(2)]
    flags = [torch.zeros(2 * rows, dtype=torch.int32, device=dev) for _ in range(2)]
    counters = torch.zeros(2, dtype=torch.int32, device=dev)
    comm = _lib.TpComm()
    comm.world_size, comm.rank, comm.max_rows, comm.hidden = 2, 0, rows, hidden
    comm.data = _ptr_array([t.data_ptr() for t in data])
    comm.flags = _ptr_array([t.data_ptr() for t in flags])
    comm.counters = counters.data_ptr()
    gamma = torch.ones(hidden, dtype=BF16, device=dev)
    hid = torch.zeros(rows, hidden, dtype=BF16, device=dev)
    nrm = torch.zeros(rows, hidden, dtype=BF16, device=dev)
    ops.set_wait_limit_ns(2_000_000)
    rc = lib.b200_allreduce_add_norm_bf16(ctypes.byref(comm), 0, None, None, gamma.data_ptr(), None, hid.data_ptr(),
                                          nrm.data_ptr(), rows, hidden, 1e-5, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status(reset=True) == 4
    assert torch.all(hid == 2.0)  # carried on with what the two slots held
    assert ops.device_status() == 0
