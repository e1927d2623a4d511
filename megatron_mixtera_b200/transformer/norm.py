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

    accepts_gemm_partials = True  # add_and_norm takes the split-K partial sums of the linear before it

    @staticmethod
    def _op(quantize):
        return {None: ops.add_norm, False: ops.add_norm, "mxfp8": ops.add_norm_mxfp8,
                "blockwise": ops.add_norm_fp8_rowblock}[quantize]

    def forward(self, x, quantize=None):
        """Normalised rows; ``quantize`` ("mxfp8" | "blockwise") makes the output the FP8 input of a linear."""
        return self._op(quantize)(x, self.weight, beta=self.bias, eps=self.eps)[1]

    def add_and_norm(self, x, residual, bias=None, quantize=None):
        """(hidden, normed) with hidden = x (+bias) + residual: the bias-dropout-add of the
        reference (``fused_bias_dropout.py:11-57``, eval mode) fused with the norm that follows it
        and, with ``quantize``, with the FP8 quantisation of the next linear's input.  ``x`` may be the
        un-reduced split-K partial sums of the linear that produced it (`ops.GemmPartials`)."""
        if type(x).__name__ == "TpPending":  # partial outputs of the tensor-parallel ranks, summed by the kernel
            return ops.allreduce_add_norm(x, self.weight, bias=bias, residual=residual, beta=self.bias, eps=self.eps,
                                          want_hidden=True, quantize=quantize or None)
        if isinstance(x, ops.GemmPartials):
            return ops.add_norm_splitk(x, self.weight, bias=bias, residual=residual, beta=self.bias, eps=self.eps,
                                       want_hidden=True, quantize=quantize or None)
        return self._op(quantize)(x, self.weight, bias=bias, residual=residual, beta=self.bias, eps=self.eps, want_hidden=True)
