"""One decoder layer: norm -> attention -> residual -> norm -> MLP -> residual
(reference ``megatron/core/transformer/transformer_layer.py:433-660``).

The residual adds are fused with the norm that follows them, so a layer hands its *un-added* MLP
output to the next layer (``forward_fused``); ``forward`` completes the residual itself and is the
plain hidden-states-in / hidden-states-out interface of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch

from .. import ops
from .spec_utils import ModuleSpec, build_module


@dataclass
class TransformerLayerSubmodules:
    input_layernorm: Union[ModuleSpec, type] = None
    self_attention: Union[ModuleSpec, type] = None
    pre_mlp_layernorm: Union[ModuleSpec, type] = None
    mlp: Union[ModuleSpec, type] = None


class TransformerLayer(torch.nn.Module):
    def __init__(self, config, submodules: TransformerLayerSubmodules, layer_number: int = 1, **_):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        eps = config.layernorm_epsilon
        self.input_layernorm = build_module(submodules.input_layernorm, config=config, hidden_size=config.hidden_size, eps=eps)
        self.self_attention = build_module(submodules.self_attention, config=config, layer_number=layer_number)
        self.pre_mlp_layernorm = build_module(submodules.pre_mlp_layernorm, config=config, hidden_size=config.hidden_size, eps=eps)
        self.mlp = build_module(submodules.mlp, config=config)

    def forward_fused(self, hidden, branch, branch_bias, defer_mlp_reduction: bool = False, **attn_kwargs):
        """``hidden`` [T, H] residual stream; ``branch`` the previous layer's MLP output not yet added
        (None for the first layer).  Returns (hidden after the attention residual, MLP output, MLP bias).

        The out-projection hands its split-K partial sums straight to the residual-add + norm kernel when that
        norm can take them; the MLP output does the same when the caller says its consumer can
        (``defer_mlp_reduction``)."""
        fp8 = self.config.fp8  # with an FP8 recipe the norms emit the quantised input of the linear that follows
        small = self.config.hidden_size <= 8192  # one 16-byte vector per thread in the fused norm kernels
        defer_attn = small and getattr(self.pre_mlp_layernorm, "accepts_gemm_partials", False)
        if branch is None:
            normed = self.input_layernorm(hidden, quantize=fp8)
        else:
            hidden, normed = self.input_layernorm.add_and_norm(branch, hidden, branch_bias, quantize=fp8)
        attn_out, attn_bias = self.self_attention(normed, defer_output_reduction=defer_attn, **attn_kwargs)
        hidden, normed = self.pre_mlp_layernorm.add_and_norm(attn_out, hidden, attn_bias, quantize=fp8)
        mlp_out, mlp_bias = self.mlp(normed, defer_output_reduction=defer_mlp_reduction and small)
        return hidden, mlp_out, mlp_bias

    def forward(self, hidden_states, attention_mask=None, inference_context=None, rotary_pos_cos=None,
                rotary_pos_sin=None, **_):
        shape = hidden_states.shape
        h = hidden_states.reshape(-1, shape[-1])
        h, mlp_out, mlp_bias = self.forward_fused(h, None, None, inference_context=inference_context,
                                                  rotary_pos_cos=rotary_pos_cos, rotary_pos_sin=rotary_pos_sin)
        h, _ = ops.add_norm(mlp_out, None, bias=mlp_bias, residual=h, want_hidden=True, want_normed=False)
        return h.view(shape), None
