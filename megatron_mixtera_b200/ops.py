"""Tensor-level wrappers over the library's torch custom ops (``torch.ops.b200_decode.*``).

The ops are registered by ``libb200_decode_torch.so`` (``csrc/torch_binding.cpp``), a thin front of the C ABI in
``include/b200_decode.h``: each checks device / dtype / contiguity, takes the current CUDA stream and raises on a
non-zero return code; the wrappers here allocate the outputs, keep the split-K workspace and re-raise failures as
`B200Error`.  Calls that launch nothing (size queries, the status word, the wait limit) and the 2-D host copy go to
the C ABI directly through ctypes.  Nothing here computes on the CPU or through PyTorch kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import AttentionArgs, B200Error  # noqa: F401  (re-exported)

BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise B200Error(name, -1, f"{name} must be a CUDA tensor (no CPU fallback exists)")
    if t.dtype != dtype:
        raise B200Error(name, -1, f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise B200Error(name, -1, f"{name} must be contiguous")


class _Workspace:
    """Grow-only device scratch per (device, tag) (split-K partial sums, attention split partials).

    A captured CUDA graph has the address of the buffer it was captured with baked in, so a buffer that is
    superseded by a larger one is never released: it stays in `_retired` for the life of the process and
    graph replays keep writing to memory that is still theirs.  `reserve` sizes a buffer up front (before any
    capture) so that the common case never grows at all.
    """

    def __init__(self):
        self._buf = {}
        self._retired = []

    def get(self, device: torch.device, tag: str, nbytes: int) -> torch.Tensor:
        key = (device.index, tag)
        buf = self._buf.get(key)
        if buf is None or buf.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise B200Error("workspace", -3, "workspace would have to grow during CUDA graph capture; "
                                "run one eager warm-up step of the same shapes first")
            if buf is not None:
                self._retired.append(buf)  # a graph may still replay into it
            buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self._buf[key] = buf
        return buf

    def reserve(self, device: torch.device, tag: str, nbytes: int) -> None:
        self.get(device, tag, nbytes)


_workspace = _Workspace()

# Kernel launches issued through this module since import (attention with context splits and GEMMs with a
# split-K reduction kernel count two).
launch_count = 0
# Number of GEMMs that have used the shared split-K workspace: a `GemmPartials` is only valid while this has not moved.
_gemm_epoch = 0
# Tensor-parallel exchanges that were handed split-K partial sums (instead of a reduced bf16 output) since import.
tp_splitk_exchanges = 0


def _gemm_workspace(device, nbytes: int, count_reduction: bool = False) -> torch.Tensor:
    global _gemm_epoch, launch_count
    _gemm_epoch += 1
    if count_reduction and nbytes > 0:
        launch_count += 1  # the split-K reduction kernel behind the GEMM kernel
    return _workspace.get(device, "gemm", nbytes)


_NOT_A_LAUNCH = ("b200_device_status", "b200_copy_rows_h2d", "b200_set_wait_limit_ns")


def check(fn_name: str, code: int) -> None:
    """Raise on a non-zero return code; count the kernel launch otherwise."""
    global launch_count
    _lib.check(fn_name, code)
    if fn_name not in _NOT_A_LAUNCH:
        launch_count += 1


_ops = None


def _launch(name: str, *args):
    """Call ``torch.ops.b200_decode.<name>`` (one kernel launch); a failed check or return code becomes `B200Error`."""
    global launch_count, _ops
    if _ops is None:
        _ops = _lib.load_torch_ops()
    try:
        out = getattr(_ops, name)(*args)
    except (RuntimeError, NotImplementedError) as e:
        raise B200Error(name, -1, str(e).split("\nException raised from")[0]) from None
    launch_count += 1
    return out


def _blob(struct) -> torch.Tensor:
    """The bytes of a ctypes argument struct as a CPU uint8 tensor sharing its memory (made once per struct)."""
    t = getattr(struct, "_as_tensor", None)
    if t is None:
        t = torch.frombuffer(struct, dtype=torch.uint8)
        struct._as_tensor = t
    return t


def set_wait_limit_ns(limit_ns: int) -> None:
    """Bound of the library's device-side waits on the current device (default 2 s)."""
    check("b200_set_wait_limit_ns", _lib.load().b200_set_wait_limit_ns(int(limit_ns)))


def device_status(reset: bool = False) -> int:
    """Status word set by kernels whose bounded waits gave up (0 = healthy).  Synchronises."""
    out = ctypes.c_int(0)
    check("b200_device_status", _lib.load().b200_device_status(int(reset), ctypes.byref(out)))
    return out.value


def copy_rows_h2d(dst: torch.Tensor, src: torch.Tensor, rows: int, lo: int, hi: int) -> None:
    """dst[:rows, lo:hi] = src[:rows, lo:hi] for two 2-D tensors of the same dtype (src pinned host memory, dst on the
    device, unit stride along the last dimension) as one asynchronous 2-D copy on the current stream."""
    es = src.element_size()
    assert dst.dtype == src.dtype and src.stride(1) == 1 and dst.stride(1) == 1 and not src.is_cuda and dst.is_cuda
    check("b200_copy_rows_h2d", _lib.load().b200_copy_rows_h2d(
        dst.data_ptr() + lo * es, dst.stride(0) * es, src.data_ptr() + lo * es, src.stride(0) * es, (hi - lo) * es, rows,
        _stream()))


def gather_rows(table, ids, *, vocab_start: int = 0, vocab_end: Optional[int] = None, add_table=None, add_ids=None,
                out=None):
    """out[i] = table[ids[i] - vocab_start] (0 when outside the shard) (+ add_table[add_ids[i]])."""
    _need(table, BF16, "table")
    _need(ids, torch.int64, "ids")
    n, width = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((n, width), dtype=BF16, device=table.device)
    if add_table is not None:
        _need(add_table, BF16, "add_table")
        _need(add_ids, torch.int64, "add_ids")
    hi = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    _launch("gather_rows", table, ids, out, vocab_start, hi, add_table, add_ids)
    return out


def add_norm(x, gamma, *, bias=None, residual=None, beta=None, eps: float = 1e-5, want_hidden: bool = False,
             want_normed: bool = True) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """h = x (+bias) (+residual); returns (h or None, norm(h) * gamma (+beta) or None)."""
    _need(x, BF16, "x")
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    h = torch.empty_like(x) if want_hidden else None
    y = torch.empty_like(x) if want_normed else None
    _launch("add_norm", x, None, 0, bias, residual, gamma, beta, h, y, None, None, 0, 0, rows, hidden, eps)
    return h, y


_ACT_KIND = {"swiglu": 0, "gelu": 1, "swiglu_interleaved": 2}


def _act_kind(kind: str) -> int:
    if kind not in _ACT_KIND:
        raise B200Error("activation", -1, f"unknown activation kind {kind!r} (one of {sorted(_ACT_KIND)})")
    return _ACT_KIND[kind]


def activation(x, kind: str, bias=None):
    """kind 'swiglu': x [rows, 2F] = [gate | up] -> [rows, F]; 'swiglu_interleaved': the same on the column order of
    an fc1 whose weight went through `interleave_gate_up`; 'gelu': x [rows, F] (+bias) -> [rows, F]."""
    _need(x, BF16, "x")
    rows = x.numel() // x.shape[-1]
    F = x.shape[-1] if _act_kind(kind) == 1 else x.shape[-1] // 2
    out = torch.empty((*x.shape[:-1], F), dtype=BF16, device=x.device)
    _launch("activation", x, None, 0, bias, out, None, None, 0, 0, rows, F, _act_kind(kind))
    return out


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[gate ; up] fc1 weight [2F, K] -> the row order `gemm_swiglu` reads: per 128 rows, 64 gate rows then the 64
    matching up rows.  F must be a multiple of 64.  `deinterleave_gate_up` is the inverse."""
    F2, K = w.shape
    F = F2 // 2
    assert F2 % 2 == 0 and F % 64 == 0, "gated fc1 rows must come in pairs of 64"
    return torch.stack([w[:F].view(F // 64, 64, K), w[F:].view(F // 64, 64, K)], dim=1).reshape(F2, K)


def deinterleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    F2, K = w.shape
    v = w.view(F2 // 128, 2, 64, K)
    return torch.cat([v[:, 0].reshape(F2 // 2, K), v[:, 1].reshape(F2 // 2, K)], dim=0)


def gemm_swiglu_supported(M: int, N: int, K: int) -> bool:
    return bool(_lib.load().b200_gemm_bf16_swiglu_supported(M, N, K))


def gemm_swiglu(x, w_interleaved, out=None):
    """[rows, F] = swiglu(x @ w.T) for an interleaved fc1 weight [2F, K], in one kernel (no split-K shapes only)."""
    _need(x, BF16, "x")
    _need(w_interleaved, BF16, "w")
    K = x.shape[-1]
    M, N = x.numel() // K, w_interleaved.shape[0]
    if out is None:
        out = torch.empty((*x.shape[:-1], N // 2), dtype=BF16, device=x.device)
    _launch("gemm_bf16_swiglu", x, w_interleaved, out)
    return out


def gemm(x, w, bias=None, out=None):
    """y[M, N] = x[M, K] @ w[N, K].T (+ bias), bf16 with fp32 accumulation on tcgen05."""
    _need(x, BF16, "x")
    _need(w, BF16, "w")
    K = x.shape[-1]
    M = x.numel() // K
    N = w.shape[0]
    if w.shape[1] != K:
        raise B200Error("gemm", -1, f"shape mismatch x[..., {K}] vs w{tuple(w.shape)}")
    if out is None:
        out = torch.empty((*x.shape[:-1], N), dtype=BF16, device=x.device)
    lib = _lib.load()
    nbytes = lib.b200_gemm_bf16_workspace_bytes(M, N, K)
    ws = _gemm_workspace(x.device, nbytes, True)
    _launch("gemm", 0, x, None, 0, w, None, bias, out, ws, M, N, K)
    return out


class Mxfp8Tensor:
    """An MXFP8-quantised [rows, K] matrix: E4M3 bytes + E8M0 scales in the GEMM's tile layout.  Activations keep
    their bytes row-major (``q [rows, K]``); weights (``packed``) keep them tile-major, see `weight_tiles_to_rows`."""

    __slots__ = ("q", "sf", "shape", "packed")

    def __init__(self, q: torch.Tensor, sf: torch.Tensor, shape, packed: bool = False):
        self.q, self.sf, self.shape, self.packed = q, sf, tuple(shape), packed


def weight_tiles_to_rows(q: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Tile-major FP8 weight bytes ([ceil(N/128)][K/128] tiles of 128 rows x 128 bytes) -> row-major [N, K]."""
    nt = (N + 127) // 128
    return q.view(nt, K // 128, 128, 128).permute(0, 2, 1, 3).reshape(nt * 128, K)[:N]


def quantize_mxfp8_weight(w) -> Mxfp8Tensor:
    """bf16 weight [N, K] -> MXFP8 with tile-major bytes (what the MXFP8 GEMMs stream)."""
    _need(w, BF16, "w")
    N, K = w.shape
    lib = _lib.load()
    q = torch.zeros((lib.b200_fp8_weight_bytes(N, K),), dtype=torch.uint8, device=w.device)
    sf = torch.empty((lib.b200_mxfp8_scale_bytes(N, K),), dtype=torch.uint8, device=w.device)
    _launch("quantize", 3, w, q, sf, N, K, 0)
    return Mxfp8Tensor(q, sf, w.shape, packed=True)


def _mx_buffers(rows: int, K: int, device):
    q = torch.empty((rows, K), dtype=torch.uint8, device=device)
    sf = torch.empty((_lib.load().b200_mxfp8_scale_bytes(rows, K),), dtype=torch.uint8, device=device)
    return q, sf


def quantize_mxfp8(x) -> Mxfp8Tensor:
    """bf16 [..., K] -> MXFP8 (K a multiple of 128)."""
    _need(x, BF16, "x")
    K = x.shape[-1]
    rows = x.numel() // K
    q, sf = _mx_buffers(rows, K, x.device)
    _launch("quantize", 1, x, q, sf, rows, K, 0)
    return Mxfp8Tensor(q, sf, x.shape)


def add_norm_mxfp8(x, gamma, *, bias=None, residual=None, beta=None, eps: float = 1e-5, want_hidden: bool = False):
    """`add_norm` whose normalised output is MXFP8: returns (h or None, Mxfp8Tensor)."""
    _need(x, BF16, "x")
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    h = torch.empty_like(x) if want_hidden else None
    q, sf = _mx_buffers(rows, hidden, x.device)
    _launch("add_norm", x, None, 0, bias, residual, gamma, beta, h, None, q, sf, 1, 0, rows, hidden, eps)
    return h, Mxfp8Tensor(q, sf, x.shape)


def activation_mxfp8(x, kind: str, bias=None) -> Mxfp8Tensor:
    """`activation` with MXFP8 output."""
    _need(x, BF16, "x")
    rows = x.numel() // x.shape[-1]
    F = x.shape[-1] if _act_kind(kind) == 1 else x.shape[-1] // 2
    q, sf = _mx_buffers(rows, F, x.device)
    _launch("activation", x, None, 0, bias, None, q, sf, 1, 0, rows, F, _act_kind(kind))
    return Mxfp8Tensor(q, sf, (*x.shape[:-1], F))


def gemm_mxfp8(x: Mxfp8Tensor, w: Mxfp8Tensor, bias=None, out=None):
    """y = dq(x) @ dq(w).T (+ bias) on the block-scaled FP8 tensor cores; bf16 output."""
    K = x.shape[-1]
    M = x.q.shape[0]
    N = w.shape[0]
    if w.shape[1] != K or not w.packed or x.packed:
        raise B200Error("gemm_mxfp8", -1, f"x[..., {K}] (row-major) vs w{tuple(w.shape)} (tile-major, `quantize_mxfp8_weight`)")
    if out is None:
        out = torch.empty((*x.shape[:-1], N), dtype=BF16, device=x.q.device)
    lib = _lib.load()
    ws = _gemm_workspace(x.q.device, lib.b200_gemm_mxfp8_workspace_bytes(M, N, K), True)
    _launch("gemm", 1, x.q, x.sf, 0, w.q, w.sf, bias, out, ws, M, N, K)
    return out


def gemm_mxfp8_swiglu(x: Mxfp8Tensor, w: Mxfp8Tensor, quantize: bool = True):
    """swiglu(dq(x) @ dq(w).T) for a gated fc1 weight [2F, K] in [gate ; up] row order, one kernel: returns the fc2 input
    as `Mxfp8Tensor` [rows, F] (or bf16 with ``quantize=False``).  K is not split: see `gemm_mxfp8_swiglu_preferred`."""
    K = x.shape[-1]
    M, F = x.q.shape[0], w.shape[0] // 2
    if w.shape[1] != K or not w.packed:
        raise B200Error("gemm_mxfp8_swiglu", -1, f"x[..., {K}] vs w{tuple(w.shape)} (tile-major, `quantize_mxfp8_weight`)")
    if quantize:
        q, sf = _mx_buffers(M, F, x.q.device)
        _launch("gemm_mxfp8_swiglu", x.q, x.sf, w.q, w.sf, q, sf, None, M, F, K)
        return Mxfp8Tensor(q, sf, (*x.shape[:-1], F))
    out = torch.empty((*x.shape[:-1], F), dtype=BF16, device=x.q.device)
    _launch("gemm_mxfp8_swiglu", x.q, x.sf, w.q, w.sf, None, None, out, M, F, K)
    return out


def gemm_mxfp8_swiglu_preferred(M: int, F: int, K: int) -> bool:
    """Whether the one-kernel fc1 + SwiGLU (F / 128 CTAs, each streaming its rows over the whole of K) is the better
    choice: enough CTAs to keep most SMs streaming.  Below that the fc1 GEMM is split along K and the activation
    kernel reduces its partial sums."""
    return F % 128 == 0 and K % 128 == 0 and F // 128 >= 96


def activation_splitk(p: "GemmPartials", kind: str, bias=None, quantize=None):
    """`activation` / `activation_mxfp8` / `activation_fp8_rowblock` (by ``quantize``) with x = the reduced split-K
    partial sums of the fc1 GEMM."""
    if p.epoch != _gemm_epoch:
        raise B200Error("activation_splitk", -1, "another GEMM has reused the workspace that held these partial sums")
    k = _act_kind(kind)
    width = p.shape[-1]
    F = width if k == 1 else width // 2
    rows = 1
    for d in p.shape[:-1]:
        rows *= d
    dev = p.device
    shape = (*p.shape[:-1], F)
    if quantize == "mxfp8":
        q, sf = _mx_buffers(rows, F, dev)
        _launch("activation", None, p.buf, p.num_splits, bias, None, q, sf, 1, 0, rows, F, k)
        return Mxfp8Tensor(q, sf, shape)
    if quantize == "blockwise":
        q, scale, m_pad = _rowblock_buffers(rows, F, dev)
        _launch("activation", None, p.buf, p.num_splits, bias, None, q, scale, 2, m_pad, rows, F, k)
        return Fp8BlockTensor(q, scale, shape, m_pad)
    out = torch.empty(shape, dtype=BF16, device=dev)
    _launch("activation", None, p.buf, p.num_splits, bias, out, None, None, 0, 0, rows, F, k)
    return out


class Fp8BlockTensor:
    """FP8 matrix of the 128-block recipe.  Activations: q [rows, K] + scale [K/128, m_pad] (per token per 128
    of K); weights: q [N, K] + scale [ceil(N/128), K/128] (per 128 x 128 block)."""

    __slots__ = ("q", "scale", "shape", "m_pad")

    def __init__(self, q, scale, shape, m_pad=0):
        self.q, self.scale, self.shape, self.m_pad = q, scale, tuple(shape), m_pad


def _rowblock_buffers(rows: int, K: int, device):
    m_pad = (rows + 3) // 4 * 4
    q = torch.empty((rows, K), dtype=torch.uint8, device=device)
    scale = torch.empty((K // 128, m_pad), dtype=torch.float32, device=device)
    return q, scale, m_pad


def quantize_fp8_weight_block128(w) -> Fp8BlockTensor:
    _need(w, BF16, "w")
    N, K = w.shape
    q = torch.zeros((_lib.load().b200_fp8_weight_bytes(N, K),), dtype=torch.uint8, device=w.device)  # tile-major
    scale = torch.empty(((N + 127) // 128, K // 128), dtype=torch.float32, device=w.device)
    _launch("quantize", 4, w, q, scale, N, K, 0)
    return Fp8BlockTensor(q, scale, w.shape)


def quantize_fp8_rowblock(x) -> Fp8BlockTensor:
    _need(x, BF16, "x")
    K = x.shape[-1]
    rows = x.numel() // K
    q, scale, m_pad = _rowblock_buffers(rows, K, x.device)
    _launch("quantize", 2, x, q, scale, rows, K, m_pad)
    return Fp8BlockTensor(q, scale, x.shape, m_pad)


def add_norm_fp8_rowblock(x, gamma, *, bias=None, residual=None, beta=None, eps: float = 1e-5, want_hidden: bool = False):
    """`add_norm` whose normalised output is FP8 with per-token 1 x 128 scales."""
    _need(x, BF16, "x")
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    h = torch.empty_like(x) if want_hidden else None
    q, scale, m_pad = _rowblock_buffers(rows, hidden, x.device)
    _launch("add_norm", x, None, 0, bias, residual, gamma, beta, h, None, q, scale, 2, m_pad, rows, hidden, eps)
    return h, Fp8BlockTensor(q, scale, x.shape, m_pad)


def activation_fp8_rowblock(x, kind: str, bias=None) -> Fp8BlockTensor:
    _need(x, BF16, "x")
    rows = x.numel() // x.shape[-1]
    F = x.shape[-1] if _act_kind(kind) == 1 else x.shape[-1] // 2
    q, scale, m_pad = _rowblock_buffers(rows, F, x.device)
    _launch("activation", x, None, 0, bias, None, q, scale, 2, m_pad, rows, F, _act_kind(kind))
    return Fp8BlockTensor(q, scale, (*x.shape[:-1], F), m_pad)


def gemm_fp8_block(x: Fp8BlockTensor, w: Fp8BlockTensor, bias=None, out=None):
    """y = dq(x) @ dq(w).T (+ bias) for the 128-block recipe (fp32 scales promoted per K block)."""
    K = x.shape[-1]
    M, N = x.q.shape[0], w.shape[0]
    if w.shape[1] != K:
        raise B200Error("gemm_fp8_block", -1, f"shape mismatch x[..., {K}] vs w{tuple(w.shape)}")
    if out is None:
        out = torch.empty((*x.shape[:-1], N), dtype=BF16, device=x.q.device)
    lib = _lib.load()
    ws = _gemm_workspace(x.q.device, lib.b200_gemm_fp8_block_workspace_bytes(M, N, K), True)
    _launch("gemm", 2, x.q, x.scale, x.m_pad, w.q, w.scale, bias, out, ws, M, N, K)
    return out


def gemm_num_splits(fp8, M: int, N: int, K: int) -> int:
    """How many K splits the GEMM of this recipe (None / "mxfp8" / "blockwise") uses for the shape."""
    lib = _lib.load()
    fn = {None: lib.b200_gemm_bf16_splitk_bytes, "mxfp8": lib.b200_gemm_mxfp8_splitk_bytes,
          "blockwise": lib.b200_gemm_fp8_block_splitk_bytes}[fp8]
    return int(fn(M, N, K) // (4 * M * N))


class GemmPartials:
    """fp32 partial sums [num_splits, M, N] of a split-K GEMM, left in the shared GEMM workspace for a fused consumer
    (`add_norm_splitk`).  Valid until the next GEMM on the same device is enqueued."""

    __slots__ = ("buf", "num_splits", "shape", "epoch")

    def __init__(self, buf: torch.Tensor, num_splits: int, shape):
        self.buf, self.num_splits, self.shape, self.epoch = buf, num_splits, tuple(shape), _gemm_epoch

    @property
    def device(self):
        return self.buf.device


def gemm_splitk(x, w) -> GemmPartials:
    """x @ w.T as split-K partial sums (no reduction launch, no bias); x bf16, `Mxfp8Tensor` or `Fp8BlockTensor`
    with `w` of the same kind."""
    lib = _lib.load()
    if isinstance(x, Mxfp8Tensor):
        K, M, N, dev = x.shape[-1], x.q.shape[0], w.shape[0], x.q.device
        if not w.packed:
            raise B200Error("gemm_splitk", -1, "MXFP8 weights must be tile-major (`quantize_mxfp8_weight`)")
        ws = _gemm_workspace(dev, lib.b200_gemm_mxfp8_splitk_bytes(M, N, K))
        n = _launch("gemm_splitk", 1, x.q, x.sf, 0, w.q, w.sf, ws, M, N, K)
    elif isinstance(x, Fp8BlockTensor):
        K, M, N, dev = x.shape[-1], x.q.shape[0], w.shape[0], x.q.device
        ws = _gemm_workspace(dev, lib.b200_gemm_fp8_block_splitk_bytes(M, N, K))
        n = _launch("gemm_splitk", 2, x.q, x.scale, x.m_pad, w.q, w.scale, ws, M, N, K)
    else:
        _need(x, BF16, "x")
        _need(w, BF16, "w")
        K = x.shape[-1]
        M, N, dev = x.numel() // K, w.shape[0], x.device
        if w.shape[1] != K:
            raise B200Error("gemm_splitk", -1, f"shape mismatch x[..., {K}] vs w{tuple(w.shape)}")
        ws = _gemm_workspace(dev, lib.b200_gemm_bf16_splitk_bytes(M, N, K))
        n = _launch("gemm_splitk", 0, x, None, 0, w, None, ws, M, N, K)
    return GemmPartials(ws, int(n), (*x.shape[:-1], N))


def add_norm_splitk(p: GemmPartials, gamma, *, bias=None, residual=None, beta=None, eps: float = 1e-5,
                    want_hidden: bool = False, want_normed: bool = True, quantize=None):
    """`add_norm` / `add_norm_mxfp8` / `add_norm_fp8_rowblock` (by ``quantize``) with x = the reduced partial sums."""
    if p.epoch != _gemm_epoch:
        raise B200Error("add_norm_splitk", -1, "another GEMM has reused the workspace that held these partial sums")
    hidden = p.shape[-1]
    rows = 1
    for d in p.shape[:-1]:
        rows *= d
    dev = p.device
    h = torch.empty(p.shape, dtype=BF16, device=dev) if want_hidden else None
    if quantize == "mxfp8":
        q, sf = _mx_buffers(rows, hidden, dev)
        _launch("add_norm", None, p.buf, p.num_splits, bias, residual, gamma, beta, h, None, q, sf, 1, 0, rows, hidden, eps)
        return h, Mxfp8Tensor(q, sf, p.shape)
    if quantize == "blockwise":
        q, scale, m_pad = _rowblock_buffers(rows, hidden, dev)
        _launch("add_norm", None, p.buf, p.num_splits, bias, residual, gamma, beta, h, None, q, scale, 2, m_pad, rows, hidden,
                eps)
        return h, Fp8BlockTensor(q, scale, p.shape, m_pad)
    y = torch.empty(p.shape, dtype=BF16, device=dev) if want_normed else None
    _launch("add_norm", None, p.buf, p.num_splits, bias, residual, gamma, beta, h, y, None, None, 0, 0, rows, hidden, eps)
    return h, y


def allreduce_add_norm(pending, gamma, *, bias=None, residual=None, beta=None, eps: float = 1e-5,
                       want_hidden: bool = False, want_normed: bool = True, quantize=None):
    """`add_norm` (or its FP8-output forms, by ``quantize``) with x = the sum over the tensor-parallel ranks of the
    partial outputs in ``pending`` (`tensor_parallel.peer_allreduce.TpPending`): collective + add + norm in one kernel."""
    comm = pending.comm
    hidden = pending.shape[-1]
    rows = 1
    for d in pending.shape[:-1]:
        rows *= d
    dev = comm.device
    if getattr(comm, "two_shot", False):
        # every rank finishes its share of the rows and stores them into all ranks' buffers: the results are views of
        # this rank's buffers (valid until the next call through the same communicator)
        q_mode = {None: 0, "mxfp8": 1, "blockwise": 2}[quantize]
        global tp_splitk_exchanges
        parts = getattr(pending, "partials", None)
        if parts is not None:
            if parts.epoch != _gemm_epoch:
                raise B200Error("allreduce_add_norm", -1, "another GEMM has reused the workspace that held these partial sums")
            tp_splitk_exchanges += 1
        _launch("allreduce_add_norm", _blob(comm.comm), 1, 0, bias, residual, gamma, beta, None, None, None, None, q_mode, 0,
                rows, hidden, eps, None if parts is None else parts.buf, 0 if parts is None else parts.num_splits)
        return comm.hidden_view(pending.shape), comm.normed_view(rows, quantize, pending.shape)
    h = torch.empty(pending.shape, dtype=BF16, device=dev) if want_hidden else None
    c = _blob(comm.comm)
    if quantize == "mxfp8":
        q, sf = _mx_buffers(rows, hidden, dev)
        _launch("allreduce_add_norm", c, 0, pending.slot, bias, residual, gamma, beta, h, None, q, sf, 1, 0, rows, hidden, eps,
                None, 0)
        return h, Mxfp8Tensor(q, sf, pending.shape)
    if quantize == "blockwise":
        q, scale, m_pad = _rowblock_buffers(rows, hidden, dev)
        _launch("allreduce_add_norm", c, 0, pending.slot, bias, residual, gamma, beta, h, None, q, scale, 2, m_pad, rows,
                hidden, eps, None, 0)
        return h, Fp8BlockTensor(q, scale, pending.shape, m_pad)
    y = torch.empty(pending.shape, dtype=BF16, device=dev) if want_normed else None
    _launch("allreduce_add_norm", c, 0, pending.slot, bias, residual, gamma, beta, h, y, None, None, 0, 0, rows, hidden, eps,
            None, 0)
    return h, y


def attention_workspace(device, num_tokens: int, num_q_heads: int, head_dim: int, num_splits: int):
    nbytes = _lib.load().b200_paged_attention_workspace_bytes(num_tokens, num_q_heads, head_dim, num_splits)
    return _workspace.get(device, "attn", nbytes) if nbytes else None


def make_attention_args(*, qkv, k_cache, v_cache, block_table, kv_seq_lengths, out, num_q_heads: int,
                        num_kv_heads: int, head_dim: int, chunk_size: int, token_to_pos_ids=None,
                        token_to_pos_in_request=None, token_to_chunk_idx=None, token_to_local_pos=None,
                        row_of_token=None, rope_cos=None, rope_sin=None, num_splits: int = 1,
                        fuse_rope_append: bool = False, softmax_scale: float = 0.0, k_scale=None,
                        v_scale=None, row_order=None, fp8_single_term: bool = False, out_quantized=None) -> AttentionArgs:
    """Fill the C argument struct.  It holds raw pointers only: the caller keeps the tensors alive until the
    kernels have run.  ``k_scale`` / ``v_scale`` (fp32 [nkv]) select the FP8 (E4M3) KV pool; ``fp8_single_term`` its
    faster, less exact arithmetic (queries and probabilities as one E4M3 term instead of two)."""
    T = qkv.shape[0]
    a = AttentionArgs()
    if isinstance(qkv, GemmPartials):  # un-reduced output of the QKV GEMM (decode kernel only)
        if qkv.epoch != _gemm_epoch:
            raise B200Error("attention", -1, "another GEMM has reused the workspace that held the QKV partial sums")
        a.qkv, a.qkv_partials, a.qkv_num_splits = None, qkv.buf.data_ptr(), qkv.num_splits
        device = qkv.device
    else:
        a.qkv, a.qkv_partials, a.qkv_num_splits = qkv.data_ptr(), None, 0
        device = qkv.device
    a.k_cache = k_cache.data_ptr()
    a.v_cache = v_cache.data_ptr()
    a.block_table = block_table.data_ptr()
    a.kv_seq_lengths = kv_seq_lengths.data_ptr()
    a.row_of_token = _p(row_of_token)
    a.token_to_pos_ids = _p(token_to_pos_ids)
    a.token_to_pos_in_request = _p(token_to_pos_in_request)
    a.token_to_chunk_idx = _p(token_to_chunk_idx)
    a.token_to_local_pos = _p(token_to_local_pos)
    a.rope_cos = _p(rope_cos)
    a.rope_sin = _p(rope_sin)
    a.out = _p(out)
    a.num_tokens = T
    a.num_q_heads = num_q_heads
    a.num_kv_heads = num_kv_heads
    a.head_dim = head_dim
    a.chunk_size = chunk_size
    a.num_chunks = k_cache.shape[0]
    a.max_chunks_per_row = block_table.shape[1]
    a.num_splits = num_splits
    a.fuse_rope_append = int(fuse_rope_append)
    a.softmax_scale = softmax_scale
    a.kv_cache_fp8 = 0 if k_scale is None else (2 if fp8_single_term else 1)
    a.k_scale = _p(k_scale)
    a.v_scale = _p(v_scale)
    a.row_order = _p(row_order)
    if isinstance(out_quantized, Mxfp8Tensor):      # the decode kernel writes the out-projection's FP8 input itself
        a.out_q, a.out_scales, a.out_q_mode, a.out_m_pad = out_quantized.q.data_ptr(), out_quantized.sf.data_ptr(), 1, 0
    elif isinstance(out_quantized, Fp8BlockTensor):
        a.out_q, a.out_scales, a.out_q_mode, a.out_m_pad = (out_quantized.q.data_ptr(), out_quantized.scale.data_ptr(), 2,
                                                            out_quantized.m_pad)
    else:
        a.out_q, a.out_scales, a.out_q_mode, a.out_m_pad = None, None, 0, 0
    ws = attention_workspace(device, T, num_q_heads, head_dim, num_splits) if (out is not None or out_quantized is not None) else None
    a.workspace = _p(ws)
    a.workspace_bytes = 0 if ws is None else ws.numel()
    a._anchor = k_cache  # device + stream of the launches that take this struct
    return a


def quantized_like(kind: str, rows: int, K: int, device, lead_shape=None):
    """Empty `Mxfp8Tensor` (kind "mxfp8") or `Fp8BlockTensor` ("blockwise") for a [rows, K] activation that a producer
    kernel will fill."""
    shape = (*(lead_shape if lead_shape is not None else (rows,)), K)
    if kind == "mxfp8":
        q, sf = _mx_buffers(rows, K, device)
        return Mxfp8Tensor(q, sf, shape)
    q, scale, m_pad = _rowblock_buffers(rows, K, device)
    return Fp8BlockTensor(q, scale, shape, m_pad)


def rope_append(args: AttentionArgs) -> None:
    _launch("attention", _blob(args), args._anchor, 0, None, 0)


def paged_attention(args: AttentionArgs) -> None:
    global launch_count
    _launch("attention", _blob(args), args._anchor, 1, None, 0)
    if args.num_splits > 1:
        launch_count += 1  # the split-combine kernel


def fp8_value_positions(chunk_size: int) -> torch.Tensor:
    """positions[t] = where token t of a chunk sits in the FP8 value pool's innermost dimension."""
    lib = _lib.load()
    return torch.tensor([lib.b200_fp8_value_position(t) for t in range(chunk_size)], dtype=torch.int64)


def fp8_values_to_pool_layout(v: torch.Tensor) -> torch.Tensor:
    """E4M3 value bytes [chunks, chunk, heads, dim] (the reference's order) -> the byte order of the FP8 pool
    ([chunks, heads, dim, position], returned with the input's shape so that it drops into the pool tensor)."""
    pos = fp8_value_positions(v.shape[1]).to(v.device)
    out = torch.empty((v.shape[0], v.shape[2], v.shape[3], v.shape[1]), dtype=v.dtype, device=v.device)
    out[..., pos] = v.permute(0, 2, 3, 1)
    return out.view(v.shape)


def fp8_values_from_pool_layout(p: torch.Tensor) -> torch.Tensor:
    """Inverse of `fp8_values_to_pool_layout`."""
    chunks, chunk, heads, dim = p.shape
    pos = fp8_value_positions(chunk).to(p.device)
    return p.view(chunks, heads, dim, chunk)[..., pos].permute(0, 3, 1, 2).contiguous()


def paged_prefill_attention(args: AttentionArgs, units: torch.Tensor, num_units: int) -> None:
    """Prefill attention over ``units`` int32 [>= num_units, 4] = (block-table row, first token, token count, 0)."""
    _need(units, torch.int32, "units")
    _launch("attention", _blob(args), args._anchor, 2, units, int(num_units))


def prefill_q_block(num_q_heads: int, num_kv_heads: int) -> int:
    """Tokens per prefill unit for this head grouping (0: the prefill kernel does not support it)."""
    g = num_q_heads // max(num_kv_heads, 1)
    return 64 // g if g in (1, 2, 4, 8, 16) else 0


def argmax(logits):
    """Greedy token per row of bf16 logits [rows, vocab] -> int64 [rows]."""
    _need(logits, BF16, "logits")
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int64, device=logits.device)
    _launch("argmax", logits, out)
    return out


def argmax_shard(logits, index_offset: int, keys=None):
    """Per-row key of the largest logit of a vocabulary shard [rows, vocab_shard] (int64 bit patterns, see
    `argmax_merge`); ``index_offset`` = first vocabulary id of the shard."""
    _need(logits, BF16, "logits")
    rows, vocab = logits.shape
    if keys is None:
        keys = torch.empty((rows,), dtype=torch.int64, device=logits.device)
    _launch("argmax_shard", logits, keys, int(index_offset))
    return keys


def argmax_merge(keys):
    """Greedy token per row from the shards' keys [shards, rows] -> int64 [rows]."""
    _need(keys, torch.int64, "keys")
    shards, rows = keys.shape
    out = torch.empty((rows,), dtype=torch.int64, device=keys.device)
    _launch("argmax_merge", keys, shards, rows, out)
    return out


def topk_probs(logits, top_k: int, temperature: float = 1.0):
    """fp32 probabilities after temperature and top-k filtering, [rows, vocab]."""
    _need(logits, BF16, "logits")
    rows, vocab = logits.shape
    probs = torch.empty((rows, vocab), dtype=torch.float32, device=logits.device)
    if top_k <= 0:
        raise B200Error("topk_probs", -1, f"top_k must be positive, got {top_k}")
    _launch("filtered_probs", logits, probs, int(top_k), 0.0, float(temperature))
    return probs


def topp_probs(logits, top_p: float, temperature: float = 1.0):
    """fp32 probabilities after temperature and top-p (nucleus) filtering, [rows, vocab]."""
    _need(logits, BF16, "logits")
    rows, vocab = logits.shape
    probs = torch.empty((rows, vocab), dtype=torch.float32, device=logits.device)
    _launch("filtered_probs", logits, probs, 0, float(top_p), float(temperature))
    return probs
