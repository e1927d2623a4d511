"""The allocation-free GEMM entry point (b200_gemm_bf16_static_scratch) against the regular one.

Callers such as a serving loop that must stay clear of the allocator, a process whose device memory is
owned by another pool, or a plugin that only gets input/output pointers cannot provide a workspace; this
entry point keeps its split-K scratch in an array inside the library.  The file name makes pytest collect
it last, so a run that stops at the first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF16).cuda()


def _static_gemm(lib, x, w, bias, y):
    M, K = x.shape
    N = w.shape[0]
    return lib.b200_gemm_bf16_static_scratch(
        x.data_ptr(), K, w.data_ptr(), None if bias is None else bias.data_ptr(), y.data_ptr(), N, M, N, K,
        torch.cuda.current_stream().cuda_stream)


def test_static_scratch_gemm_matches_workspace_gemm_twice_in_a_row():
    from megatron_mixtera_b200 import _lib, build, ops

    build.build()
    lib = _lib.load()
    limit = lib.b200_gemm_bf16_static_scratch_limit()
    assert limit == 16 * 1024 * 1024
    # split-K shapes that need the scratch (few output tiles, long K) and shapes without split-K (many tiles)
    cases = [(200, 1024, 2048, False), (16, 256, 8192, True), (64, 4096, 4096, False), (64, 6144, 4096, True),
             (33, 1000, 576, False), (16, 20000, 512, True)]
    assert lib.b200_gemm_bf16_workspace_bytes(200, 1024, 2048) > 0
    assert lib.b200_gemm_bf16_workspace_bytes(16, 256, 8192) > 0
    assert lib.b200_gemm_bf16_workspace_bytes(16, 20000, 512) == 0
    inputs = []
    for i, (M, N, K, has_bias) in enumerate(cases):
        x, w = _randn((M, K), 10 + i), _randn((N, K), 20 + i, 0.05)
        b = _randn((N,), 30 + i) if has_bias else None
        inputs.append((x, w, b, ops.gemm(x, w, b), torch.empty((M, N), dtype=BF16, device="cuda")))
    # first call on this device (address look-up) happens here, outside any capture
    assert _static_gemm(lib, *inputs[0][:3], inputs[0][4]) == 0
    ys = [torch.empty_like(t[4]) for t in inputs]
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    for round_ in range(2):  # two calls in a row per shape: the second finds the first one's leftovers
        for x, w, b, ref, y in inputs:
            y.fill_(float("nan"))
            assert _static_gemm(lib, x, w, b, y) == 0
            assert _static_gemm(lib, x, w, b, y) == 0
            torch.cuda.synchronize()
            assert torch.equal(y, ref), (round_, tuple(x.shape), tuple(w.shape))
    # back to back on the same stream with different operands, checked only at the end
    for (x, w, b, _, _), y in zip(inputs, ys):
        assert _static_gemm(lib, x, w, b, y) == 0
    torch.cuda.synchronize()
    for (_, _, _, ref, _), y in zip(inputs, ys):
        assert torch.equal(y, ref)
    # nothing was allocated on the device by the calls above
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == allocated_before
    assert free_after == free_before
    assert ops.device_status() == 0


def test_static_scratch_gemm_rejects_what_does_not_fit():
    from megatron_mixtera_b200 import _lib, build

    build.build()
    lib = _lib.load()
    M, N, K = 256, 4096, 14336  # split-K partial sums of 9 x 256 x 4096 floats exceed the 16 MiB array
    assert lib.b200_gemm_bf16_workspace_bytes(M, N, K) > lib.b200_gemm_bf16_static_scratch_limit()
    x, w = _randn((M, K), 1), _randn((N, K), 2, 0.05)
    y = torch.zeros((M, N), dtype=BF16, device="cuda")
    code = _static_gemm(lib, x, w, None, y)
    assert code == -7
    assert b"scratch" in lib.b200_error_string(code)
    torch.cuda.synchronize()
    assert torch.count_nonzero(y) == 0  # nothing ran
    assert _static_gemm(lib, x[:, :100], w, None, y) < 0  # argument checks are the regular GEMM's
