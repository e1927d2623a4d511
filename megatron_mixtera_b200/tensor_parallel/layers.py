"""Tensor-parallel linear layers and embedding backed by the sm_100a kernels.

Constructor arguments, parameter names / shapes (``weight [out/tp, in]`` or ``[out, in/tp]``, ``bias``)
and the ``forward(x) -> (output, bias_or_None)`` contract follow the reference's
``ColumnParallelLinear`` / ``RowParallelLinear`` / ``VocabParallelEmbedding``
(``megatron/core/tensor_parallel/layers.py:158-295, 743-1057, 1060-1303``), so a state dict of one loads
into the other.  Only the inference forward exists: there is no autograd path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops, parallel_state
from .mappings import gather_from_tensor_model_parallel_region, reduce_from_tensor_model_parallel_region


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class VocabParallelLogits:
    """This rank's shard ``[rows, V / tp]`` of the output layer's logits, standing in for the gathered ``[rows, V]``
    tensor that the reference materialises on every step (``layers.py:1037-1039``).  Greedy sampling needs 8 bytes per
    row and rank (`TextGenerationController.sample_from_logits`); everything else calls `gather()` (or `float()`),
    which is the reference's all-gather.  Implements the few tensor methods the wrapper / controller path uses."""

    def __init__(self, local: torch.Tensor, vocab_start: int, vocab_size: int, group=None):
        self.local, self.vocab_start, self.vocab_size, self.group = local, int(vocab_start), int(vocab_size), group

    @property
    def shape(self):
        return (self.local.shape[0], self.vocab_size)

    @property
    def device(self):
        return self.local.device

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    def __getitem__(self, rows):
        if not isinstance(rows, slice):
            raise TypeError("vocabulary-parallel logits can be sliced along the rows only")
        return VocabParallelLogits(self.local[rows], self.vocab_start, self.vocab_size, self.group)

    def unsqueeze(self, dim):
        return self

    squeeze = unsqueeze

    def contiguous(self):
        return self

    def gather(self) -> torch.Tensor:
        """The full ``[rows, V]`` logits (all-gather over the tensor-parallel group)."""
        return gather_from_tensor_model_parallel_region(self.local, self.group)

    def float(self) -> torch.Tensor:
        return self.gather().float()

    def greedy_tokens(self) -> torch.Tensor:
        """argmax over the whole vocabulary (ties: smallest id) without gathering the logits: per-shard
        (value, index) keys, an all-gather of 8 bytes per row and rank, then the maximum key."""
        tp = parallel_state.get_tensor_model_parallel_world_size()
        local = self.local if self.local.is_contiguous() else self.local.contiguous()
        keys = ops.argmax_shard(local, self.vocab_start)
        allk = torch.empty((tp, keys.shape[0]), dtype=torch.int64, device=keys.device)
        torch.distributed.all_gather_into_tensor(allk, keys, group=self.group or parallel_state.get_tensor_model_parallel_group())
        return ops.argmax_merge(allk)


class _ParallelLinearBase(torch.nn.Module):
    """Shared by the column- and row-parallel linears: optional MXFP8 execution.

    With ``config.fp8`` set ("mxfp8": E8M0 scale per 32 elements; "blockwise": fp32 scale per 128 x 128 weight
    block and per token per 128 of K) and ``fp8_enabled``, the bf16 ``weight`` parameter stays the checkpoint
    format and a quantised copy is made by `quantize_weights` - called by the model after weights are loaded,
    or lazily on the first forward - and streamed by the FP8 GEMM.  The input may arrive already quantised
    (`ops.Mxfp8Tensor` / `ops.Fp8BlockTensor`, from a producer kernel that fused the quantisation) or as
    bf16, in which case it is quantised here.
    """

    fp8 = None
    _wq = None

    def get_extra_state(self):
        return None

    def set_extra_state(self, state):
        pass

    # Gated fc1 only: `gate_up_interleaved` asks for the row order of the fused fc1 + SwiGLU kernel; the weight is
    # rearranged in place by `quantize_weights` (i.e. after every load of canonical [gate ; up] weights) and
    # `_layout_interleaved` says that this has happened.  `canonical_weight()` undoes it for export.
    gate_up_interleaved = False
    _layout_interleaved = False

    def quantize_weights(self) -> None:
        if self.gate_up_interleaved and not self._layout_interleaved and self.weight is not None:
            self.weight.data.copy_(ops.interleave_gate_up(self.weight.data))
            self._layout_interleaved = True
        if self.fp8 and self.weight is not None and self._weight_shape is None:
            fn = ops.quantize_mxfp8_weight if self.fp8 == "mxfp8" else ops.quantize_fp8_weight_block128
            self._wq = fn(self.weight.data)

    @property
    def weight_shape(self):
        """(out, in) of this rank's shard, also after `release_checkpoint_weight`."""
        return self._weight_shape if self._weight_shape is not None else tuple(self.weight.shape)

    _weight_shape = None

    def release_checkpoint_weight(self) -> bool:
        """Free the bf16 ``weight`` once its FP8 copy exists (serving from the quantised weights only: the bf16
        tensor is the checkpoint format and is not read by any FP8 GEMM).  The parameter object stays, empty;
        `state_dict` can then no longer export this layer.  Returns True if memory was released."""
        if not self.fp8 or self.weight is None:
            return False
        if self._wq is None:
            self.quantize_weights()
        self._weight_shape = tuple(self.weight.shape)
        self.weight.data = torch.empty(0, dtype=self.weight.dtype, device=self.weight.device)
        return True

    def canonical_weight(self) -> torch.Tensor:
        """The weight in the reference's row order (a copy when the rows are interleaved for the fused kernel)."""
        return ops.deinterleave_gate_up(self.weight.data) if self._layout_interleaved else self.weight.data

    def _matmul(self, input_, weight, bias, defer_reduction: bool = False, out=None):
        """``defer_reduction``: return the split-K partial sums (`ops.GemmPartials`) for a consumer that reduces
        them itself, instead of the bf16 product; no bias then."""
        assert not (defer_reduction and bias is not None)
        quantised_input = isinstance(input_, (ops.Mxfp8Tensor, ops.Fp8BlockTensor))
        if self.fp8 and weight is self.weight:
            if self._wq is None:
                self.quantize_weights()
            if self.fp8 == "mxfp8":
                x = input_ if quantised_input else ops.quantize_mxfp8(input_)
                return ops.gemm_splitk(x, self._wq) if defer_reduction else ops.gemm_mxfp8(x, self._wq, bias, out=out)
            x = input_ if quantised_input else ops.quantize_fp8_rowblock(input_)
            return ops.gemm_splitk(x, self._wq) if defer_reduction else ops.gemm_fp8_block(x, self._wq, bias, out=out)
        if quantised_input:
            raise ops.B200Error("linear", -1, "got an FP8 input but this layer runs in bf16")
        return ops.gemm_splitk(input_, weight) if defer_reduction else ops.gemm(input_, weight, bias, out=out)


class ColumnParallelLinear(_ParallelLinearBase):
    """Y = X A^T + b with A split along its output rows: rank r holds rows [r*out/tp, (r+1)*out/tp)."""

    def __init__(self, input_size, output_size, *, config, init_method=None, bias=True, gather_output=False,
                 skip_bias_add=False, is_expert=False, tp_comm_buffer_name=None, tp_group=None,
                 skip_weight_param_allocation=False, stride=1, fp8_enabled=True, **_):
        super().__init__()
        self.fp8 = getattr(config, "fp8", None) if fp8_enabled else None
        tp = parallel_state.get_tensor_model_parallel_world_size()
        assert output_size % tp == 0, f"output_size {output_size} not divisible by tp {tp}"
        self.input_size, self.output_size = input_size, output_size
        self.output_size_per_partition = output_size // tp
        self.gather_output, self.skip_bias_add, self.tp_group = gather_output, skip_bias_add, tp_group
        self.config = config
        dt, dev = config.params_dtype, _device()
        self.weight = None
        if not skip_weight_param_allocation:
            self.weight = torch.nn.Parameter(torch.empty(self.output_size_per_partition, input_size, dtype=dt, device=dev),
                                             requires_grad=False)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=dt, device=dev), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    supports_deferred_reduction = True

    def forward(self, input_, weight: Optional[torch.Tensor] = None, runtime_gather_output: Optional[bool] = None,
                defer_reduction: bool = False):
        """``input_`` [..., in] -> ([..., out/tp] or gathered [..., out], bias if ``skip_bias_add``).  With
        ``defer_reduction`` (and no bias to add, no gather) the output is the GEMM's split-K partial sums
        (`ops.GemmPartials`) for a consumer that reduces them itself."""
        w = self.weight if weight is None else weight
        fuse_bias = self.bias if (self.bias is not None and not self.skip_bias_add) else None
        gather_now = self.gather_output if runtime_gather_output is None else runtime_gather_output
        if defer_reduction and fuse_bias is None and not gather_now and weight is None:
            return self._matmul(input_, w, None, defer_reduction=True), (self.bias if self.skip_bias_add else None)
        out = self._matmul(input_, w, fuse_bias)
        gather = self.gather_output if runtime_gather_output is None else runtime_gather_output
        if gather == "deferred":  # hand out the shard; the consumer gathers only if it needs the full rows
            if parallel_state.get_tensor_model_parallel_world_size() > 1:
                per = self.output_size_per_partition
                out = VocabParallelLogits(out.view(-1, per), parallel_state.get_tensor_model_parallel_rank() * per,
                                          self.output_size, self.tp_group)
        elif gather:
            out = gather_from_tensor_model_parallel_region(out, self.tp_group)
        return out, (self.bias if self.skip_bias_add else None)


    def forward_gated(self, input_):
        """Gated fc1 in the reference's [gate ; up] row order followed by SwiGLU: the fc2 input, quantised under an
        FP8 recipe.  One of three forms, all with the same bits: the one-kernel gate / up pair GEMM with the
        activation and quantisation in its epilogue (MXFP8, enough output features to fill the GPU without
        splitting K); the split-K GEMM whose partial sums the activation kernel reduces itself (no reduction
        launch); or GEMM followed by the activation kernel."""
        assert self.bias is None and not self.gather_output
        fp8, cfg = self.fp8, self.config
        quantised_input = isinstance(input_, (ops.Mxfp8Tensor, ops.Fp8BlockTensor))
        M = input_.q.shape[0] if quantised_input else input_.numel() // input_.shape[-1]
        N, K = self.weight_shape
        if fp8 == "mxfp8" and getattr(cfg, "fuse_swiglu_into_fc1", True) and ops.gemm_mxfp8_swiglu_preferred(M, N // 2, K):
            if self._wq is None:
                self.quantize_weights()
            x = input_ if quantised_input else ops.quantize_mxfp8(input_)
            return ops.gemm_mxfp8_swiglu(x, self._wq)
        if getattr(cfg, "fuse_splitk_reduction_into_norm", True) and ops.gemm_num_splits(fp8, M, N, K) > 1:
            return ops.activation_splitk(self._matmul(input_, self.weight, None, defer_reduction=True), "swiglu", quantize=fp8)
        act = {None: ops.activation, "mxfp8": ops.activation_mxfp8, "blockwise": ops.activation_fp8_rowblock}[fp8]
        return act(self._matmul(input_, self.weight, None), "swiglu")

    def forward_swiglu(self, input_):
        """fc1 followed by SwiGLU for a weight in the interleaved row order: one kernel when the GEMM is not split
        along K, else GEMM + the activation kernel on the interleaved columns.  Same bits either way."""
        assert self._layout_interleaved and self.bias is None and not self.gather_output
        K = input_.shape[-1]
        M, N = input_.numel() // K, self.weight.shape[0]
        if ops.gemm_swiglu_supported(M, N, K):
            return ops.gemm_swiglu(input_, self.weight)
        return ops.activation(ops.gemm(input_, self.weight), "swiglu_interleaved")


class RowParallelLinear(_ParallelLinearBase):
    """Y = X A^T + b with A split along its input columns; partial products are all-reduced."""

    def __init__(self, input_size, output_size, *, config, init_method=None, bias=True, input_is_parallel=True,
                 skip_bias_add=False, is_expert=False, tp_comm_buffer_name=None, tp_group=None, fp8_enabled=True, **_):
        super().__init__()
        self.fp8 = getattr(config, "fp8", None) if fp8_enabled else None
        tp = parallel_state.get_tensor_model_parallel_world_size()
        assert input_size % tp == 0, f"input_size {input_size} not divisible by tp {tp}"
        assert input_is_parallel, "the decode path always feeds the row-parallel layer its own shard"
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = input_size // tp
        self.skip_bias_add, self.tp_group, self.config = skip_bias_add, tp_group, config
        dt, dev = config.params_dtype, _device()
        self.weight = torch.nn.Parameter(torch.empty(output_size, self.input_size_per_partition, dtype=dt, device=dev),
                                         requires_grad=False)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(output_size, dtype=dt, device=dev), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    supports_deferred_reduction = True

    def forward(self, input_, defer_reduction: bool = False):
        """``defer_reduction`` (honoured at TP=1 when no bias has to be added here): the output is the GEMM's
        split-K partial sums (`ops.GemmPartials`), to be reduced by the residual-add + norm kernel that follows."""
        tp = parallel_state.get_tensor_model_parallel_world_size()
        # The bias must be added once, after the reduction: fuse it into the GEMM only at TP=1.
        fuse_bias = self.bias if (self.bias is not None and not self.skip_bias_add and tp == 1) else None
        if defer_reduction and tp == 1 and fuse_bias is None and getattr(self.config, "fuse_splitk_reduction_into_norm", True):
            return self._matmul(input_, self.weight, None, defer_reduction=True), (self.bias if self.skip_bias_add else None)
        if defer_reduction and tp > 1 and (self.bias is None or self.skip_bias_add) \
                and getattr(self.config, "fuse_tp_allreduce_into_norm", True):
            # The partial product goes into this rank's peer-visible slot; the norm kernel that follows sums the
            # ranks' slots itself (collective + residual add + norm in one launch).
            from .peer_allreduce import TpPending, get_peer_allreduce

            rows = (input_.q.shape[0] if hasattr(input_, "q") else input_.numel() // input_.shape[-1])
            comm = get_peer_allreduce(self.output_size, rows)
            if comm is not None:
                lead = input_.shape[:-1]
                fp8 = self.fp8
                if getattr(comm, "two_shot", False) and comm.accepts_partials(rows) \
                        and getattr(self.config, "fuse_splitk_reduction_into_norm", True) \
                        and ops.gemm_num_splits(fp8, rows, self.output_size, self.weight_shape[1]) > 1:
                    # split-K GEMM: its partial sums go to the exchange kernel, which sums them into the peer-visible
                    # buffer itself (no reduction launch)
                    parts = self._matmul(input_, self.weight, None, defer_reduction=True)
                    return (TpPending(comm, 0, (*lead, self.output_size), partials=parts),
                            (self.bias if self.skip_bias_add else None))
                slot, view = comm.output_slot(rows)
                self._matmul(input_, self.weight, None, out=view)
                return TpPending(comm, slot, (*lead, self.output_size)), (self.bias if self.skip_bias_add else None)
        out = self._matmul(input_, self.weight, fuse_bias)
        if tp > 1:
            out = reduce_from_tensor_model_parallel_region(out, self.tp_group)
            if self.bias is not None and not self.skip_bias_add:
                out, _ = ops.add_norm(out, None, bias=self.bias, want_hidden=True, want_normed=False)
        return out, (self.bias if self.skip_bias_add else None)


class VocabParallelEmbedding(torch.nn.Module):
    """Embedding split along the vocabulary: masked local lookup, then all-reduce
    (reference ``layers.py:158-295``)."""

    def __init__(self, num_embeddings, embedding_dim, *, config, init_method=None, tp_group=None, **_):
        super().__init__()
        tp, rank = parallel_state.get_tensor_model_parallel_world_size(), parallel_state.get_tensor_model_parallel_rank()
        assert num_embeddings % tp == 0
        per = num_embeddings // tp
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.vocab_start_index, self.vocab_end_index = rank * per, (rank + 1) * per
        self.tp_group = tp_group
        self.weight = torch.nn.Parameter(torch.empty(per, embedding_dim, dtype=config.params_dtype, device=_device()),
                                         requires_grad=False)

    def forward(self, input_ids, add_table=None, add_ids=None):
        """``input_ids`` int64 [..]; returns [n, H].  ``add_table[add_ids]`` (position embedding) is
        added in the same kernel at TP=1 and after the reduction otherwise."""
        ids = input_ids.reshape(-1)
        tp = parallel_state.get_tensor_model_parallel_world_size()
        if tp == 1:
            return ops.gather_rows(self.weight, ids, add_table=add_table, add_ids=add_ids)
        out = ops.gather_rows(self.weight, ids, vocab_start=self.vocab_start_index, vocab_end=self.vocab_end_index)
        out = reduce_from_tensor_model_parallel_region(out, self.tp_group)
        if add_table is not None:
            pos = ops.gather_rows(add_table, add_ids.reshape(-1))
            out, _ = ops.add_norm(out, None, residual=pos, want_hidden=True, want_normed=False)
        return out
