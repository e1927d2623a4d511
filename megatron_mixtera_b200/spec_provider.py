"""Layer spec that selects the sm_100a operator classes.

``B200SpecProvider`` answers the questions of the reference's ``BackendSpecProvider`` protocol
(``megatron/core/models/backends.py:26-70``) and ``get_gpt_layer_b200_spec`` assembles the layer spec
the way ``get_gpt_layer_local_spec`` does (``megatron/core/models/gpt/gpt_layer_specs.py:200-309``).
"""
from __future__ import annotations

from .tensor_parallel.layers import ColumnParallelLinear, RowParallelLinear
from .transformer.attention import PagedFlashDecodeAttention, SelfAttention, SelfAttentionSubmodules
from .transformer.mlp import MLP, MLPSubmodules
from .transformer.norm import B200Norm
from .transformer.spec_utils import ModuleSpec
from .transformer.transformer_layer import TransformerLayer, TransformerLayerSubmodules


class B200SpecProvider:
    def column_parallel_linear(self) -> type:
        return ColumnParallelLinear

    def row_parallel_linear(self) -> type:
        return RowParallelLinear

    def fuse_layernorm_and_linear(self) -> bool:
        # the norm is fused with the residual add that precedes it, not with the linear after it
        return False

    def column_parallel_layer_norm_linear(self):
        return None

    def layer_norm(self, rms_norm: bool = False, for_qk: bool = False) -> type:
        return B200Norm

    def core_attention(self) -> type:
        return PagedFlashDecodeAttention

    def activation_func(self):
        return None

    def grouped_mlp_modules(self, moe_use_grouped_gemm: bool, moe_use_legacy_grouped_gemm: bool):
        raise NotImplementedError("mixture-of-experts layers are outside the dense decode path")


def get_gpt_layer_b200_spec(normalization: str = "RMSNorm") -> ModuleSpec:
    b = B200SpecProvider()
    norm = b.layer_norm(rms_norm=normalization == "RMSNorm")
    return ModuleSpec(
        module=TransformerLayer,
        submodules=TransformerLayerSubmodules(
            input_layernorm=norm,
            self_attention=ModuleSpec(
                module=SelfAttention,
                submodules=SelfAttentionSubmodules(
                    linear_qkv=b.column_parallel_linear(),
                    core_attention=b.core_attention(),
                    linear_proj=b.row_parallel_linear(),
                ),
            ),
            pre_mlp_layernorm=norm,
            mlp=ModuleSpec(
                module=MLP,
                submodules=MLPSubmodules(linear_fc1=b.column_parallel_linear(), linear_fc2=b.row_parallel_linear()),
            ),
        ),
    )
