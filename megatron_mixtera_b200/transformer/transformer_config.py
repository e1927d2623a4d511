"""Configuration of the decoder stack: the fields of the reference's ``TransformerConfig``
(``megatron/core/transformer/transformer_config.py``) that the dynamic decode path reads."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class TransformerConfig:
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    num_query_groups: Optional[int] = None      # None: multi-head attention
    kv_channels: Optional[int] = None           # None: hidden_size // num_attention_heads
    ffn_hidden_size: Optional[int] = None       # None: 4 * hidden_size
    normalization: str = "LayerNorm"            # "LayerNorm" | "RMSNorm"
    layernorm_epsilon: float = 1e-5
    gated_linear_unit: bool = False             # True + activation "silu" = SwiGLU
    activation: str = "gelu"                    # "gelu" | "silu"
    add_bias_linear: bool = True
    params_dtype: torch.dtype = torch.bfloat16
    tensor_model_parallel_size: int = 1
    enable_cuda_graph: bool = False
    inference_sampling_seed: int = 42
    init_method_std: float = 0.02
    # not in the reference: hand the split-K partial sums of out-proj / fc2 to the residual-add + norm kernel
    # instead of reducing them in a kernel of their own (bit-identical results, two launches fewer per layer)
    fuse_splitk_reduction_into_norm: bool = True
    # not in the reference: in decode steps the attention kernel sums the QKV GEMM's split-K partial sums itself
    # (bit-identical, one launch fewer per layer; measured neutral on the step time, hence off by default)
    fuse_qkv_reduction_into_attention: bool = False
    # not in the reference: bf16 gated MLPs run fc1 + SwiGLU as one kernel; the fc1 weight is kept with its gate / up
    # rows interleaved per 64 (`ColumnParallelLinear.canonical_weight()` gives the reference's order back)
    fuse_swiglu_into_fc1: bool = True
    # not in the reference: at TP > 1 the all-reduce after out-proj / fc2 is done by the residual-add + norm kernel
    # itself with peer loads over NVLink (one node, <= 4 ranks, <= 512 token rows; NCCL otherwise)
    fuse_tp_allreduce_into_norm: bool = True
    # not in the reference: under an FP8 recipe the decode attention kernel writes its output already quantised for the
    # out-projection (same bits as the stand-alone quantiser, one launch fewer per layer)
    fuse_attention_output_quantization: bool = True
    # not in the reference: at TP > 1 the output layer hands the controller its vocabulary shard; greedy sampling then
    # exchanges one (value, index) key per row and rank instead of all-gathering the logits (False: the reference's way)
    defer_logits_gather: bool = True
    fp8: Optional[str] = None                   # None | "mxfp8" (E8M0 scale per 32) | "blockwise" (fp32, 128x128 / 1x128)

    def __post_init__(self):
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.params_dtype != torch.bfloat16:
            raise ValueError("the sm_100a decode kernels compute in bf16 (fp32 accumulation); params_dtype must be bfloat16")
        if self.fp8 not in (None, "mxfp8", "blockwise"):
            raise NotImplementedError(f"fp8 recipe {self.fp8!r} (supported: 'mxfp8', 'blockwise')")
        tp = self.tensor_model_parallel_size
        if self.num_attention_heads % tp or self.num_query_groups % tp:
            raise ValueError("attention heads and query groups must be divisible by the tensor parallel size")
        if self.num_attention_heads % self.num_query_groups:
            raise ValueError("num_attention_heads must be a multiple of num_query_groups")
        if self.gated_linear_unit and self.activation != "silu":
            raise NotImplementedError("gated MLPs are supported as SwiGLU only")
        if not self.gated_linear_unit and self.activation != "gelu":
            raise NotImplementedError("ungated MLPs are supported with GELU only")
