"""Stack of decoder layers + final norm (reference ``megatron/core/transformer/transformer_block.py:514-673``)."""
from __future__ import annotations

import torch

from .norm import B200Norm
from .spec_utils import build_module


class TransformerBlock(torch.nn.Module):
    def __init__(self, config, spec, post_layer_norm: bool = True, **_):
        super().__init__()
        self.config = config
        self.layers = torch.nn.ModuleList(
            [build_module(spec, config=config, layer_number=i + 1) for i in range(config.num_layers)])
        self.final_layernorm = (
            B200Norm(config=config, hidden_size=config.hidden_size, eps=config.layernorm_epsilon) if post_layer_norm else None)

    def forward(self, hidden_states, attention_mask=None, inference_context=None, rotary_pos_cos=None,
                rotary_pos_sin=None, **_):
        """``hidden_states`` [T, 1, H] or [T, H] -> final-normed hidden states of the same shape."""
        shape = hidden_states.shape
        hidden = hidden_states.reshape(-1, shape[-1])
        branch = bias = None
        kw = dict(inference_context=inference_context, rotary_pos_cos=rotary_pos_cos, rotary_pos_sin=rotary_pos_sin)
        consumers = list(self.layers[1:]) + [None]
        for layer, nxt in zip(self.layers, consumers):
            # the MLP output of a layer is consumed by the next layer's input norm, or by the final norm
            norm = nxt.input_layernorm if nxt is not None else self.final_layernorm
            defer = getattr(norm, "accepts_gemm_partials", False)
            hidden, branch, bias = layer.forward_fused(hidden, branch, bias, defer_mlp_reduction=defer, **kw)
        if self.final_layernorm is not None:
            _, out = self.final_layernorm.add_and_norm(branch, hidden, bias)
        else:
            from .. import ops

            out, _ = ops.add_norm(branch, None, bias=bias, residual=hidden, want_hidden=True, want_normed=False)
        return out.view(shape)
