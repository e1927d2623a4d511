"""Self-attention over the dynamic context's paged KV pool.

``SelfAttention`` keeps the reference's layout contract (``megatron/core/transformer/attention.py``):
``linear_qkv`` produces, per KV group, the group's query heads, then its key, then its value
(:985-1021), and ``linear_proj`` is row-parallel.  What the reference does in six calls - RoPE on q and
k through the context, KV append, K/V view, flash-attn (:394-414, 765-768, 588-600) - is one fused op here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union

import torch

from .. import ops, parallel_state
from ..utils import REF_ATTENTION, nvtx_range_pop, nvtx_range_push
from .spec_utils import ModuleSpec, build_module


@dataclass
class SelfAttentionSubmodules:
    linear_qkv: Union[ModuleSpec, type] = None
    core_attention: Union[ModuleSpec, type] = None
    linear_proj: Union[ModuleSpec, type] = None


_SM_COUNT = {}


def _sm_count() -> int:
    if not torch.cuda.is_available():
        return 148
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


def choose_attention_splits(num_rows: int, num_kv_heads: int, max_sequence_length: int, chunk_size: int) -> int:
    """Context splits per row (flash-decoding).  A function of capture-time constants only, so that a
    CUDA graph can replay it: enough (row, KV head, split) units for two CTAs per SM, and - contexts differ by
    large factors inside a batch, and a CTA runs for a time proportional to its share - no split longer than 8192
    tokens at the longest context; never shorter than 1024 tokens there."""
    sms = _sm_count()
    units = max(1, num_rows * num_kv_heads)
    want = max(-(-2 * sms // units), -(-max_sequence_length // 8192))
    cap = max(1, max_sequence_length // 1024)
    return int(max(1, min(want, cap, 64)))


class PagedFlashDecodeAttention(torch.nn.Module):
    """Core attention of the dynamic path: RoPE + KV append + paged attention in the sm_100a kernels."""

    def __init__(self, config, layer_number: int, **_):
        super().__init__()
        tp = parallel_state.get_tensor_model_parallel_world_size()
        self.config, self.layer_number = config, layer_number
        self.num_q_heads = config.num_attention_heads // tp
        self.num_kv_heads = config.num_query_groups // tp
        self.head_dim = config.kv_channels

    accepts_gemm_partials = True  # decode steps: the QKV GEMM's split-K partial sums instead of its bf16 output
    quantizes_output = True       # decode steps: FP8 output for an FP8 out-projection

    def forward(self, mixed_qkv, inference_context, rotary_pos_cos=None, rotary_pos_sin=None, quantize_output=None):
        """``mixed_qkv`` [T, (nq + 2 nkv) d / tp] (or, in decode steps, the `ops.GemmPartials` of the GEMM that
        computes it) -> [T, nq d / tp].  ``quantize_output`` ("mxfp8" | "blockwise"; honoured in decode steps): the
        kernel that finishes an output row writes it as the FP8 input of the out-projection (`ops.Mxfp8Tensor` /
        `ops.Fp8BlockTensor`) instead of bf16 - no stand-alone quantisation kernel between attention and out-proj."""
        ctx = inference_context
        T = mixed_qkv.shape[0]
        k_cache, v_cache, block_table = ctx.key_value_cache(self.layer_number)
        decode = ctx.is_decode_only()
        width = self.num_q_heads * self.head_dim
        out_q = None
        if (decode and quantize_output and width % 128 == 0 and (quantize_output == "mxfp8" or self.head_dim == 128)):
            out_q = ops.quantized_like(quantize_output, T, width, mixed_qkv.device)
        out = None if out_q is not None else torch.empty((T, width), dtype=torch.bfloat16, device=mixed_qkv.device)
        partials = isinstance(mixed_qkv, ops.GemmPartials)
        assert decode or not partials, "only the decode kernel reads un-reduced QKV partial sums"
        common = dict(out_quantized=out_q,
            qkv=mixed_qkv if partials else mixed_qkv.view(T, self.num_kv_heads, -1), k_cache=k_cache, v_cache=v_cache, out=out,
            num_q_heads=self.num_q_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
            chunk_size=ctx.chunk_size_tokens, token_to_pos_ids=ctx.token_to_pos_ids,
            token_to_pos_in_request=ctx.token_to_position_in_request, token_to_chunk_idx=ctx.token_to_chunk_idx,
            token_to_local_pos=ctx.token_to_local_position_within_kv_chunk, rope_cos=rotary_pos_cos,
            rope_sin=rotary_pos_sin,
        )
        if getattr(ctx, "kv_cache_fp8", False):  # E4M3 pool: per-head scales of this layer
            common.update(k_scale=ctx.kv_scales[self.layer_number - 1, 0], v_scale=ctx.kv_scales[self.layer_number - 1, 1],
                          fp8_single_term=getattr(ctx, "kv_fp8_single_term", False))
        if decode:
            # one new token per request: rows are requests, append fused into the attention kernel
            splits = choose_attention_splits(T, self.num_kv_heads, ctx.max_sequence_length, ctx.chunk_size_tokens)
            args = ops.make_attention_args(block_table=ctx.request_to_kv_chunk_ids_cudagraph_only,
                                           kv_seq_lengths=ctx.kv_seq_lengths_cudagraph_only, num_splits=splits,
                                           fuse_rope_append=True, row_order=ctx.attention_row_order, **common)
            ops.paged_attention(args)
            if out_q is not None:
                return out_q
        else:
            # prefill / mixed step: append every token first; then either blocks of a request's query tokens share
            # the K/V tiles (work list built by the context), or - FP8 pool, unusual head groupings - each token
            # is a row that sees its request's first (position + 1) keys
            args = ops.make_attention_args(block_table=ctx.request_to_kv_chunk_ids_cudagraph_only,
                                           kv_seq_lengths=ctx.token_kv_lengths, row_of_token=ctx.token_to_block_table_row,
                                           num_splits=1, fuse_rope_append=False, **common)
            ops.rope_append(args)
            if getattr(ctx, "prefill_q_block", 0) > 0 and ctx.prefill_q_block == ops.prefill_q_block(self.num_q_heads, self.num_kv_heads):
                out.zero_()  # padding tokens belong to no unit
                ops.paged_prefill_attention(args, ctx.prefill_units, ctx.prefill_unit_count)
            else:
                ops.paged_attention(args)
        return out


class SelfAttention(torch.nn.Module):
    def __init__(self, config, submodules: SelfAttentionSubmodules, layer_number: int, attn_mask_type=None, **_):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        d = config.kv_channels
        self.query_projection_size = d * config.num_attention_heads
        self.kv_projection_size = d * config.num_query_groups
        self.linear_qkv = build_module(
            submodules.linear_qkv, config.hidden_size, self.query_projection_size + 2 * self.kv_projection_size,
            config=config, bias=config.add_bias_linear, gather_output=False, skip_bias_add=False,
            tp_comm_buffer_name="qkv")
        self.core_attention = build_module(submodules.core_attention, config=config, layer_number=layer_number)
        self.linear_proj = build_module(
            submodules.linear_proj, self.query_projection_size, config.hidden_size, config=config,
            bias=config.add_bias_linear, input_is_parallel=True, skip_bias_add=True, tp_comm_buffer_name="proj")

    def forward(self, hidden_states, attention_mask=None, inference_context=None, rotary_pos_cos=None,
                rotary_pos_sin=None, defer_output_reduction: bool = False, **_):
        """``hidden_states`` [T, H] (already normalised) -> (output [T, H], bias or None).  With
        ``defer_output_reduction`` the output may be the out-projection's split-K partial sums."""
        if inference_context is None or inference_context.is_static_batching():
            raise NotImplementedError("only the dynamic-batching inference path is implemented")
        defer_qkv = (inference_context.is_decode_only() and getattr(self.config, "fuse_qkv_reduction_into_attention", False)
                     and getattr(self.linear_qkv, "supports_deferred_reduction", False)
                     and getattr(self.core_attention, "accepts_gemm_partials", False)
                     and not getattr(inference_context, "kv_cache_fp8", False))  # the E4M3-pool kernel reads bf16 qkv
        nvtx_range_push(REF_ATTENTION, "qkv")
        if defer_qkv:  # decode: the attention kernel sums the QKV GEMM's split-K partial sums itself
            mixed_qkv, _ = self.linear_qkv(hidden_states, defer_reduction=True)
        else:
            mixed_qkv, _ = self.linear_qkv(hidden_states)
        nvtx_range_pop(REF_ATTENTION, "qkv")
        # adjust_key_value (KV append), rotary_pos_emb and core_attention of the reference are one fused op here
        nvtx_range_push(REF_ATTENTION, "core_attention")
        fp8 = getattr(self.linear_proj, "fp8", None)
        if fp8 and getattr(self.config, "fuse_attention_output_quantization", True) \
                and getattr(self.core_attention, "quantizes_output", False):
            core = self.core_attention(mixed_qkv, inference_context, rotary_pos_cos, rotary_pos_sin, quantize_output=fp8)
        else:
            core = self.core_attention(mixed_qkv, inference_context, rotary_pos_cos, rotary_pos_sin)
        nvtx_range_pop(REF_ATTENTION, "core_attention")
        nvtx_range_push(REF_ATTENTION, "linear_proj")
        if defer_output_reduction and getattr(self.linear_proj, "supports_deferred_reduction", False):
            out = self.linear_proj(core, defer_reduction=True)
        else:
            out = self.linear_proj(core)
        nvtx_range_pop(REF_ATTENTION, "linear_proj")
        return out
