"""ctypes binding of ``libb200_decode.so`` (declarations in ``include/b200_decode.h``).

There is no fallback: if the library is missing the import of any op fails with a clear
error.  The library is built in-tree by ``megatron_mixtera_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

from .build import LIB_PATH, TORCH_LIB_PATH

EXPORTED_SYMBOLS = (
    "b200_version",
    "b200_error_string",
    "b200_device_status",
    "b200_set_wait_limit_ns",
    "b200_copy_rows_h2d",
    "b200_gather_rows_bf16",
    "b200_add_norm_bf16",
    "b200_activation_bf16",
    "b200_set_gemm_split_policy",
    "b200_gemm_bf16_workspace_bytes",
    "b200_gemm_bf16",
    "b200_gemm_bf16_static_scratch_limit",
    "b200_gemm_bf16_static_scratch",
    "b200_mxfp8_scale_bytes",
    "b200_quantize_mxfp8",
    "b200_quantize_mxfp8_weight",
    "b200_fp8_weight_bytes",
    "b200_add_norm_mxfp8",
    "b200_activation_mxfp8",
    "b200_gemm_mxfp8_workspace_bytes",
    "b200_gemm_mxfp8",
    "b200_gemm_mxfp8_swiglu",
    "b200_quantize_fp8_weight_block128",
    "b200_quantize_fp8_rowblock",
    "b200_add_norm_fp8_rowblock",
    "b200_activation_fp8_rowblock",
    "b200_set_fp8_block_cta_pairs",
    "b200_gemm_fp8_block_workspace_bytes",
    "b200_gemm_fp8_block",
    "b200_gemm_bf16_swiglu_supported",
    "b200_gemm_bf16_swiglu",
    "b200_gemm_bf16_splitk_bytes",
    "b200_gemm_bf16_splitk",
    "b200_gemm_mxfp8_splitk_bytes",
    "b200_gemm_mxfp8_splitk",
    "b200_gemm_fp8_block_splitk_bytes",
    "b200_gemm_fp8_block_splitk",
    "b200_add_norm_splitk_bf16",
    "b200_add_norm_splitk_mxfp8",
    "b200_add_norm_splitk_fp8_rowblock",
    "b200_activation_splitk_bf16",
    "b200_activation_splitk_mxfp8",
    "b200_activation_splitk_fp8_rowblock",
    "b200_peer_buffer_create",
    "b200_peer_buffer_open",
    "b200_peer_buffer_close",
    "b200_peer_buffer_destroy",
    "b200_allreduce_add_norm_bf16",
    "b200_allreduce_add_norm_mxfp8",
    "b200_allreduce_add_norm_fp8_rowblock",
    "b200_allreduce2_add_norm",
    "b200_allreduce2_add_norm_splitk",
    "b200_paged_attention_workspace_bytes",
    "b200_rope_append",
    "b200_paged_attention",
    "b200_paged_prefill_attention",
    "b200_fp8_value_position",
    "b200_argmax_bf16",
    "b200_argmax_shard_bf16",
    "b200_argmax_merge",
    "b200_topk_probs_bf16",
    "b200_topp_probs_bf16",
)


class AttentionArgs(ctypes.Structure):
    """Mirror of ``b200_attention_args``."""

    _fields_ = [
        ("qkv", c_void_p),
        ("k_cache", c_void_p),
        ("v_cache", c_void_p),
        ("block_table", c_void_p),
        ("kv_seq_lengths", c_void_p),
        ("row_of_token", c_void_p),
        ("token_to_pos_ids", c_void_p),
        ("token_to_pos_in_request", c_void_p),
        ("token_to_chunk_idx", c_void_p),
        ("token_to_local_pos", c_void_p),
        ("rope_cos", c_void_p),
        ("rope_sin", c_void_p),
        ("out", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("num_tokens", c_int32),
        ("num_q_heads", c_int32),
        ("num_kv_heads", c_int32),
        ("head_dim", c_int32),
        ("chunk_size", c_int32),
        ("num_chunks", c_int32),
        ("max_chunks_per_row", c_int32),
        ("num_splits", c_int32),
        ("fuse_rope_append", c_int32),
        ("softmax_scale", c_float),
        ("kv_cache_fp8", c_int32),
        ("k_scale", c_void_p),
        ("v_scale", c_void_p),
        ("qkv_partials", c_void_p),
        ("qkv_num_splits", c_int32),
        ("row_order", c_void_p),
        ("out_q", c_void_p),
        ("out_scales", c_void_p),
        ("out_q_mode", c_int32),
        ("out_m_pad", c_int32),
    ]


class TpComm(ctypes.Structure):
    """Mirror of ``b200_tp_comm``."""

    _fields_ = [
        ("world_size", c_int32),
        ("rank", c_int32),
        ("max_rows", c_int32),
        ("hidden", c_int32),
        ("data", c_void_p * 8),
        ("flags", c_void_p * 8),
        ("counters", c_void_p),
    ]


class TpExchange(ctypes.Structure):
    """Mirror of ``b200_tp_exchange``."""

    _fields_ = [
        ("world_size", c_int32),
        ("rank", c_int32),
        ("max_rows", c_int32),
        ("hidden", c_int32),
        ("m_pad", c_int32),
        ("in_", c_void_p * 8),
        ("hidden_out", c_void_p * 8),
        ("normed_out", c_void_p * 8),
        ("scales_out", c_void_p * 8),
        ("flags", c_void_p * 8),
        ("counters", c_void_p),
    ]


class B200Error(RuntimeError):
    """A C-ABI entry point returned a negative code."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed: {text} ({code})")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    """Load (once) and type the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m megatron_mixtera_b200.build` "
            "(there is no CPU or PyTorch fallback for the decode kernels)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.b200_version.restype = c_int
    lib.b200_error_string.restype = c_char_p
    lib.b200_error_string.argtypes = [c_int]
    lib.b200_device_status.argtypes = [c_int, POINTER(c_int)]
    lib.b200_copy_rows_h2d.argtypes = [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p]
    lib.b200_gather_rows_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_void_p,
                                          c_void_p, c_void_p]
    lib.b200_add_norm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_float, c_void_p]
    lib.b200_activation_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_set_gemm_split_policy.argtypes = [c_int, c_int, c_int]
    lib.b200_set_fp8_block_cta_pairs.argtypes = [c_int]
    lib.b200_gemm_bf16_workspace_bytes.restype = c_size_t
    lib.b200_gemm_bf16_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.b200_gemm_bf16.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                   c_void_p, c_size_t, c_void_p]
    lib.b200_gemm_bf16_swiglu_supported.argtypes = [c_int, c_int, c_int]
    lib.b200_gemm_bf16_swiglu.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    lib.b200_gemm_bf16_static_scratch_limit.restype = c_size_t
    lib.b200_gemm_bf16_static_scratch_limit.argtypes = []
    lib.b200_gemm_bf16_static_scratch.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                                  c_int, c_void_p]
    lib.b200_mxfp8_scale_bytes.restype = c_size_t
    lib.b200_mxfp8_scale_bytes.argtypes = [c_int, c_int]
    lib.b200_quantize_mxfp8.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.b200_quantize_mxfp8_weight.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.b200_fp8_weight_bytes.restype = c_size_t
    lib.b200_fp8_weight_bytes.argtypes = [c_int, c_int]
    lib.b200_add_norm_mxfp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_float, c_void_p]
    lib.b200_activation_mxfp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_gemm_mxfp8_workspace_bytes.restype = c_size_t
    lib.b200_gemm_mxfp8_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.b200_gemm_mxfp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                    c_int, c_void_p, c_size_t, c_void_p]
    lib.b200_gemm_mxfp8_swiglu.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                           c_int, c_int, c_int, c_void_p]
    lib.b200_activation_splitk_bf16.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_activation_splitk_mxfp8.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_activation_splitk_fp8_rowblock.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                        c_int, c_void_p]
    lib.b200_quantize_fp8_weight_block128.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.b200_quantize_fp8_rowblock.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.b200_add_norm_fp8_rowblock.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200_activation_fp8_rowblock.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_void_p]
    lib.b200_gemm_fp8_block_workspace_bytes.restype = c_size_t
    lib.b200_gemm_fp8_block_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.b200_gemm_fp8_block.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                        c_int, c_int, c_void_p, c_size_t, c_void_p]
    for name in ("b200_gemm_bf16_splitk_bytes", "b200_gemm_mxfp8_splitk_bytes", "b200_gemm_fp8_block_splitk_bytes"):
        getattr(lib, name).restype = c_size_t
        getattr(lib, name).argtypes = [c_int, c_int, c_int]
    lib.b200_gemm_bf16_splitk.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t,
                                          POINTER(c_int), c_void_p]
    lib.b200_gemm_mxfp8_splitk.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t,
                                           POINTER(c_int), c_void_p]
    lib.b200_gemm_fp8_block_splitk.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                               c_size_t, POINTER(c_int), c_void_p]
    lib.b200_add_norm_splitk_bf16.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_int, c_int, c_float, c_void_p]
    lib.b200_add_norm_splitk_mxfp8.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_float, c_void_p]
    lib.b200_add_norm_splitk_fp8_rowblock.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200_peer_buffer_create.argtypes = [c_size_t, POINTER(c_void_p), ctypes.c_char_p]
    lib.b200_peer_buffer_open.argtypes = [ctypes.c_char_p, POINTER(c_void_p)]
    lib.b200_peer_buffer_close.argtypes = [c_void_p]
    lib.b200_peer_buffer_destroy.argtypes = [c_void_p]
    lib.b200_allreduce_add_norm_bf16.argtypes = [POINTER(TpComm), c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_int, c_int, c_float, c_void_p]
    lib.b200_allreduce_add_norm_mxfp8.argtypes = [POINTER(TpComm), c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]
    lib.b200_allreduce_add_norm_fp8_rowblock.argtypes = [POINTER(TpComm), c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200_allreduce2_add_norm.argtypes = [POINTER(TpExchange), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_float, c_void_p]
    lib.b200_allreduce2_add_norm_splitk.argtypes = [POINTER(TpExchange), c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                    c_int, c_int, c_int, c_float, c_void_p]
    lib.b200_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    lib.b200_paged_attention_workspace_bytes.restype = c_size_t
    lib.b200_paged_attention_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int]
    lib.b200_rope_append.argtypes = [POINTER(AttentionArgs), c_void_p]
    lib.b200_paged_attention.argtypes = [POINTER(AttentionArgs), c_void_p]
    lib.b200_fp8_value_position.argtypes = [c_int]
    lib.b200_paged_prefill_attention.argtypes = [POINTER(AttentionArgs), c_void_p, c_int, c_void_p]
    lib.b200_argmax_bf16.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]
    lib.b200_argmax_shard_bf16.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int64, c_void_p]
    lib.b200_argmax_merge.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.b200_topk_probs_bf16.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200_topp_probs_bf16.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_float, c_float, c_void_p]
    for name in EXPORTED_SYMBOLS:
        fn = getattr(lib, name)
        if fn.restype is c_int or name.startswith("b200_") and fn.restype not in (c_char_p, c_size_t):
            fn.restype = c_int
    _lib = lib
    return lib


_torch_ops = None


def load_torch_ops():
    """Register (once) the torch custom ops of ``libb200_decode_torch.so`` and return ``torch.ops.b200_decode``.

    The front links ``libb200_decode.so``; loading the C-ABI library first with its full path makes the dynamic
    linker reuse that copy.  Raises if either library has not been built: there is no fallback."""
    global _torch_ops
    if _torch_ops is not None:
        return _torch_ops
    load()
    if not os.path.exists(TORCH_LIB_PATH):
        raise ImportError(
            f"{TORCH_LIB_PATH} is missing: build it with `python -m megatron_mixtera_b200.build` "
            "(the decode operators have no CPU or PyTorch fallback)"
        )
    import torch

    torch.ops.load_library(TORCH_LIB_PATH)
    _torch_ops = torch.ops.b200_decode
    return _torch_ops


TORCH_OPS = (
    "gather_rows", "add_norm", "activation", "quantize", "gemm", "gemm_splitk", "gemm_bf16_swiglu", "gemm_mxfp8_swiglu",
    "attention", "argmax", "argmax_shard", "argmax_merge", "filtered_probs", "allreduce_add_norm",
)


def check(fn_name: str, code: int) -> None:
    if code != 0:
        raise B200Error(fn_name, code, load().b200_error_string(code).decode())
