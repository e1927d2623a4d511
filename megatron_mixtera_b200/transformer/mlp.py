"""Feed-forward block: fc1 -> SwiGLU or bias+GELU -> fc2 (reference ``megatron/core/transformer/mlp.py:140-234``).
fc1's weight holds ``[gate ; up]`` halves per rank for the gated case (``fused_bias_swiglu.py:25``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch

from .. import ops
from ..utils import REF_MLP, nvtx_range_pop, nvtx_range_push
from .spec_utils import ModuleSpec, build_module


@dataclass
class MLPSubmodules:
    linear_fc1: Union[ModuleSpec, type] = None
    linear_fc2: Union[ModuleSpec, type] = None


class MLP(torch.nn.Module):
    def __init__(self, config, submodules: MLPSubmodules, **_):
        super().__init__()
        self.config = config
        ffn = config.ffn_hidden_size * (2 if config.gated_linear_unit else 1)
        self.linear_fc1 = build_module(submodules.linear_fc1, config.hidden_size, ffn, config=config,
                                       bias=config.add_bias_linear, gather_output=False, skip_bias_add=True,
                                       tp_comm_buffer_name="fc1")
        self.linear_fc2 = build_module(submodules.linear_fc2, config.ffn_hidden_size, config.hidden_size, config=config,
                                       bias=config.add_bias_linear, input_is_parallel=True, skip_bias_add=True,
                                       tp_comm_buffer_name="fc2")

        # bf16 SwiGLU: fc1 and the activation run as one kernel on a weight whose gate / up rows are interleaved
        # per 64 (arranged in place when the weights are loaded)
        if (config.gated_linear_unit and config.fp8 is None and getattr(config, "fuse_swiglu_into_fc1", True)
                and hasattr(self.linear_fc1, "forward_swiglu") and self.linear_fc1.bias is None
                and (self.linear_fc1.weight.shape[0] // 2) % 64 == 0):
            self.linear_fc1.gate_up_interleaved = True

    def forward(self, hidden_states, defer_output_reduction: bool = False):
        # ranges as in the reference (mlp.py:143-226); where fc1 and the activation are one kernel, "linear_fc1" covers both
        nvtx_range_push(REF_MLP, "linear_fc1")
        inter = self._fc1_and_activation(hidden_states)
        nvtx_range_pop(REF_MLP, "linear_fc1")
        nvtx_range_push(REF_MLP, "linear_fc2")
        if defer_output_reduction and getattr(self.linear_fc2, "supports_deferred_reduction", False):
            out = self.linear_fc2(inter, defer_reduction=True)
        else:
            out = self.linear_fc2(inter)
        nvtx_range_pop(REF_MLP, "linear_fc2")
        return out

    def _fc1_and_activation(self, hidden_states):
        if getattr(self.linear_fc1, "_layout_interleaved", False):
            return self.linear_fc1.forward_swiglu(hidden_states)
        if self.config.gated_linear_unit and self.linear_fc1.bias is None and hasattr(self.linear_fc1, "forward_gated"):
            return self.linear_fc1.forward_gated(hidden_states)
        inter, bias = self.linear_fc1(hidden_states)
        act = {None: ops.activation, "mxfp8": ops.activation_mxfp8, "blockwise": ops.activation_fp8_rowblock}[self.config.fp8]
        if self.config.gated_linear_unit:
            if bias is not None:
                raise NotImplementedError("SwiGLU with an fc1 bias")
            return act(inter, "swiglu")
        return act(inter, "gelu", bias)
