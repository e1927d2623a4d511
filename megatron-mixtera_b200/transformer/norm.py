"""RMSNorm / LayerNorm module over the fused add+norm kernel.

Stands where the reference uses ``WrappedTorchNorm`` (``megatron/core/transformer/torch_norm.py:38-51``)
or ``TENorm`` (``megatron/core/extensions/transformer_engine.py:204-238``): same constructor
(``config, hidden_size, eps``), same parameter names (``weight``, and ``bias`` for LayerNorm).
"""
from __future__ import annotations

import torch

from .. import ops


class B200Norm(torch.nn.Module):
    def __init__(self, config, hidden_size: int, eps: float = 1e-5, **_):
        super().__init__()
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=config.params_dtype, device=dev), requires_grad=False)
        if config.normalization == "LayerNorm":
            self.bias = torch.nn.Parameter(torch.zeros(hidden_size, dtype=config.params_dtype, device=dev), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def forward(self, x, quantize: bool = False):
        """Normalised rows; with ``quantize`` the output is an `ops.Mxfp8Tensor` for an FP8 linear."""
        if quantize:
            return ops.add_norm_mxfp8(x, self.weight, beta=self.bias, eps=self.eps)[1]
        return ops.add_norm(x, self.weight, beta=self.bias, eps=self.eps)[1]

    def add_and_norm(self, x, residual, bias=None, quantize: bool = False):
        """(hidden, normed) with hidden = x (+bias) + residual: the bias-dropout-add of the
        reference (``fused_bias_dropout.py:11-57``, eval mode) fused with the norm that follows it
        and, with ``quantize``, with the MXFP8 quantisation of the next linear's input."""
        fn = ops.add_norm_mxfp8 if quantize else ops.add_norm
        return fn(x, self.weight, bias=bias, residual=residual, beta=self.bias, eps=self.eps, want_hidden=True)
