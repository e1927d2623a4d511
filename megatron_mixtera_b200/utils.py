"""NVTX ranges with the reference's names (``megatron/core/utils.py:1845-1960``: ``configure_nvtx_profiling``,
``nvtx_range_push`` / ``nvtx_range_pop``), so that a timeline of this path lines up with one of the reference.

The reference names a range ``<module of the caller>.<calling function>.<suffix>``; the callers here pass the
reference's module path explicitly (``REF_ATTENTION`` ...), since the code lives in other modules.  Off by default;
switched on with `configure_nvtx_profiling(True)`.  Ranges inside a captured CUDA graph mark the capture, not the
replays - the engine's per-step "Prefill" / "Decode" ranges (``dynamic_engine.py:562, 658``) bracket those.
"""
from __future__ import annotations

from typing import List

import torch

REF_ATTENTION = "megatron.core.transformer.attention.forward"
REF_MLP = "megatron.core.transformer.mlp.forward"

_nvtx_enabled = False
_nvtx_range_messages: List[str] = []


def configure_nvtx_profiling(enabled: bool) -> None:
    global _nvtx_enabled
    _nvtx_enabled = bool(enabled) and torch.cuda.is_available()


def nvtx_enabled() -> bool:
    return _nvtx_enabled


def nvtx_range_push(msg: str = None, suffix: str = None) -> None:
    if not _nvtx_enabled:
        return
    msg = msg or "b200_decode"
    if suffix is not None:
        msg = f"{msg}.{suffix}"
    _nvtx_range_messages.append(msg)
    torch.cuda.nvtx.range_push(msg)


def nvtx_range_pop(msg: str = None, suffix: str = None) -> None:
    if not _nvtx_enabled:
        return
    if not _nvtx_range_messages:
        raise RuntimeError("Attempted to pop NVTX range from empty stack")
    last = _nvtx_range_messages.pop()
    if msg is not None:
        want = f"{msg}.{suffix}" if suffix is not None else msg
        if last != want:
            raise ValueError(f"Mismatching NVTX range messages in nvtx_range_pop: last pushed {last!r}, popping {want!r}")
    torch.cuda.nvtx.range_pop()
