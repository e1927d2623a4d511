"""GPT decoder model for the dynamic inference path.

Module tree and ``state_dict`` keys follow the reference's ``GPTModel``
(``megatron/core/models/gpt/gpt_model.py``): ``embedding.word_embeddings``,
``embedding.position_embeddings`` (learned absolute positions only), ``decoder.layers.N.*``,
``decoder.final_layernorm``, ``output_layer``.  ``forward`` has the reference's signature and returns
``[1, rows, vocab]`` logits (``gpt_model.py:344, 509-560``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import ops, parallel_state
from ..spec_provider import get_gpt_layer_b200_spec
from ..tensor_parallel.layers import ColumnParallelLinear, VocabParallelEmbedding
from ..transformer.transformer_block import TransformerBlock
from ..transformer.transformer_config import TransformerConfig


def rope_tables(max_seq_len: int, dim: int, base: float, dtype: torch.dtype, device) -> tuple:
    """cos / sin of ``pos * base^(-2i/dim)`` as ``[max_seq_len, dim/2]`` tables in ``dtype``.

    The angles are formed in fp32 exactly as ``RotaryEmbedding.forward`` does
    (``megatron/core/models/common/embeddings/rotary_pos_embedding.py:79-81, 150-181``) and the cast to
    the activation dtype happens before use, as ``_apply_rotary_pos_emb_bshd`` does
    (``rope_utils.py:122-123``).  Computed on the host so that the values do not depend on the device's
    trigonometric routines.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv_freq)
    return torch.cos(freqs).to(dtype).to(device).contiguous(), torch.sin(freqs).to(dtype).to(device).contiguous()


class _PositionEmbedding(torch.nn.Module):
    def __init__(self, n, h, dtype, device):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty(n, h, dtype=dtype, device=device), requires_grad=False)


class LanguageModelEmbedding(torch.nn.Module):
    """Word (+ learned position) embeddings (reference ``language_model_embedding.py:99-149``)."""

    def __init__(self, config, vocab_size, max_sequence_length, position_embedding_type):
        super().__init__()
        self.word_embeddings = VocabParallelEmbedding(vocab_size, config.hidden_size, config=config)
        self.add_position_embedding = position_embedding_type == "learned_absolute"
        if self.add_position_embedding:
            self.position_embeddings = _PositionEmbedding(max_sequence_length, config.hidden_size, config.params_dtype,
                                                          self.word_embeddings.weight.device)

    def forward(self, input_ids, position_ids):
        if self.add_position_embedding:
            return self.word_embeddings(input_ids, self.position_embeddings.weight, position_ids.reshape(-1))
        return self.word_embeddings(input_ids)


class GPTModel(torch.nn.Module):
    def __init__(self, config: TransformerConfig, transformer_layer_spec=None, vocab_size: int = None,
                 max_sequence_length: int = None, pre_process: bool = True, post_process: bool = True,
                 parallel_output: bool = True, share_embeddings_and_output_weights: bool = False,
                 position_embedding_type: str = "learned_absolute", rotary_base: float = 10000.0, **_):
        super().__init__()
        assert pre_process and post_process, "pipeline stages are outside the decode path built here"
        self.config, self.vocab_size, self.max_sequence_length = config, vocab_size, max_sequence_length
        self.position_embedding_type = position_embedding_type
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        if transformer_layer_spec is None:
            transformer_layer_spec = get_gpt_layer_b200_spec(config.normalization)
        self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type)
        self.decoder = TransformerBlock(config, transformer_layer_spec)
        self.output_layer = ColumnParallelLinear(
            config.hidden_size, vocab_size, config=config, bias=False, gather_output=not parallel_output,
            skip_bias_add=False, skip_weight_param_allocation=share_embeddings_and_output_weights,
            fp8_enabled=False)  # the reference's output layer is a plain bf16 ColumnParallelLinear too
        self.rotary_pos_cos = self.rotary_pos_sin = None
        if position_embedding_type == "rope":
            self.rotary_pos_cos, self.rotary_pos_sin = rope_tables(
                max_sequence_length, config.kv_channels, rotary_base, config.params_dtype,
                self.embedding.word_embeddings.weight.device)

    # ------------------------------------------------------------------------------------------
    def forward_rows(self, input_ids, position_ids, inference_context, row_indices=None,
                     runtime_gather_output: Optional[bool] = None):
        """Logits ``[rows, vocab]``: every token row when ``row_indices`` is None, else the given rows
        (int64 device tensor) of the final hidden states."""
        from ..tensor_parallel import peer_allreduce

        comms_at_entry = peer_allreduce.begin_forward()
        hidden = self.embedding(input_ids.reshape(-1), position_ids)
        hidden = self.decoder(hidden, inference_context=inference_context, rotary_pos_cos=self.rotary_pos_cos,
                              rotary_pos_sin=self.rotary_pos_sin)
        peer_allreduce.end_forward(comms_at_entry)
        if row_indices is not None:
            hidden = ops.gather_rows(hidden, row_indices)
        weight = self.embedding.word_embeddings.weight if self.share_embeddings_and_output_weights else None
        logits, _ = self.output_layer(hidden, weight=weight, runtime_gather_output=runtime_gather_output)
        return logits

    def forward(self, input_ids, position_ids, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None, runtime_gather_output: Optional[bool] = None, **_):
        """``input_ids`` / ``position_ids`` ``[1, T]`` of the context's padded step.  Returns
        ``[1, active requests, vocab]`` when the context materialises last-token logits only, else
        ``[1, T, vocab]``."""
        ctx = inference_context
        if ctx is None or labels is not None:
            raise NotImplementedError("only inference with a dynamic context is implemented")
        if ctx.materialize_only_last_token_logits:
            n_req = ctx.total_request_count - ctx.paused_request_count
            if ctx.is_decode_only():
                logits = self.forward_rows(input_ids, position_ids, ctx, None, runtime_gather_output)[:n_req]
            else:
                idx = torch.from_numpy(ctx.last_token_indices()).to(input_ids.device)
                logits = self.forward_rows(input_ids, position_ids, ctx, idx, runtime_gather_output)
        else:
            logits = self.forward_rows(input_ids, position_ids, ctx, None, runtime_gather_output)
        return logits.unsqueeze(0)

    # ------------------------------------------------------------------------------------------
    def full_parameter_shapes(self) -> Dict[str, tuple]:
        """``state_dict`` key -> UNSHARDED shape (what a TP=1 model of the reference holds)."""
        tp = parallel_state.get_tensor_model_parallel_world_size()
        out = {}
        for k, v in self.state_dict().items():
            if v is None or k.endswith("_extra_state"):
                continue
            shape = list(v.shape)
            dim = _partition_dim(k)
            if dim is not None:
                shape[dim] *= tp
            out[k] = tuple(shape)
        return out

    def load_full_state_dict(self, full: Dict[str, torch.Tensor]) -> None:
        """Load UNSHARDED tensors, keeping this rank's shard of each (see `shard_for_rank`)."""
        tp, rank = parallel_state.get_tensor_model_parallel_world_size(), parallel_state.get_tensor_model_parallel_rank()
        own = self.state_dict()
        for k, dst in own.items():
            if dst is None or k.endswith("_extra_state"):
                continue
            dst.copy_(shard_for_rank(k, full[k], rank, tp, gated=self.config.gated_linear_unit))
        self._weights_are_canonical()
        self.quantize_weights()

    def load_tensor_parallel_checkpoint(self, shards: List[Dict[str, torch.Tensor]]) -> None:
        """Load a checkpoint that was written at ANY tensor-parallel size (``shards[r]`` = rank r's ``state_dict``, the
        layout of the reference's ``mp_rank_XX`` files): the shards are merged with the reference's partition rules
        and re-sharded for this model's tensor-parallel size."""
        self.load_full_state_dict(merge_tensor_parallel_shards(shards, gated=self.config.gated_linear_unit))

    def sharded_state_dict(self, prefix: str = "") -> Dict[str, List[ShardedTensorInfo]]:
        """``state_dict`` key -> the piece(s) of the unsharded tensor this rank holds (see `ShardedTensorInfo`).
        Weights come out in the reference's row order (`ColumnParallelLinear.canonical_weight`)."""
        tp, rank = parallel_state.get_tensor_model_parallel_world_size(), parallel_state.get_tensor_model_parallel_rank()
        canonical = {n + ".weight": m.canonical_weight() for n, m in self.named_modules() if hasattr(m, "canonical_weight") and m.weight is not None}
        out = {}
        full = self.full_parameter_shapes()
        for k, v in self.state_dict().items():
            if v is None or k.endswith("_extra_state"):
                continue
            v = canonical.get(k, v)
            dim, gshape = _partition_dim(k), full[k]
            if dim is None or tp == 1:
                out[prefix + k] = [ShardedTensorInfo(prefix + k, v, gshape, (0,) * v.dim(), replica_id=rank if dim is None else 0)]
            elif self.config.gated_linear_unit and k.endswith(("linear_fc1.weight", "linear_fc1.bias")):
                gate, up = torch.chunk(v, 2, dim=0)
                per, F = gate.shape[0], gshape[0] // 2
                rest = (0,) * (v.dim() - 1)
                out[prefix + k] = [ShardedTensorInfo(prefix + k, gate, gshape, (rank * per, *rest)),
                                   ShardedTensorInfo(prefix + k, up, gshape, (F + rank * per, *rest))]
            else:
                off = [0] * v.dim()
                off[dim] = rank * v.shape[dim]
                out[prefix + k] = [ShardedTensorInfo(prefix + k, v, gshape, tuple(off))]
        return out

    # ---- offline quantisation: serve from FP8 weights without ever holding the bf16 ones ----
    def quantized_state_dict(self) -> Dict[str, torch.Tensor]:
        """The FP8 copies of this rank's linear weights (what `quantize_weights` built), as plain tensors:
        ``<module>.weight_fp8`` (tile-major E4M3 bytes) and ``<module>.weight_scales`` (E8M0 tile bytes for "mxfp8",
        fp32 ``[N/128, K/128]`` for "blockwise"), plus every tensor that is not an FP8 linear weight.  Written once by
        an offline job; `load_quantized_state_dict` is the matching loader."""
        out = {}
        fp8_weights = set()
        for n, m in self.named_modules():
            if getattr(m, "fp8", None) and getattr(m, "weight", None) is not None:
                if m._wq is None:
                    m.quantize_weights()
                out[n + ".weight_fp8"] = m._wq.q
                out[n + ".weight_scales"] = m._wq.sf if m.fp8 == "mxfp8" else m._wq.scale
                fp8_weights.add(n + ".weight")
        for k, v in self.state_dict().items():
            if v is not None and not k.endswith("_extra_state") and k not in fp8_weights:
                out[k] = v
        return out

    def load_quantized_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Counterpart of `quantized_state_dict` (same tensor-parallel size and recipe): FP8 linears take their
        quantised weights as they are and release the bf16 parameter; everything else is copied."""
        from .. import ops

        own = self.state_dict()
        for n, m in self.named_modules():
            if getattr(m, "fp8", None) and getattr(m, "weight", None) is not None:
                q, sc = sd[n + ".weight_fp8"].to(m.weight.device), sd[n + ".weight_scales"].to(m.weight.device)
                shape = m.weight_shape
                m._wq = ops.Mxfp8Tensor(q, sc, shape, packed=True) if m.fp8 == "mxfp8" else ops.Fp8BlockTensor(q, sc, shape)
                m._weight_shape = tuple(shape)
                m.weight.data = torch.empty(0, dtype=m.weight.dtype, device=m.weight.device)
                own.pop(n + ".weight", None)
        for k, dst in own.items():
            if dst is not None and not k.endswith("_extra_state"):
                dst.copy_(sd[k])

    def _weights_are_canonical(self) -> None:
        """Called after the parameters were overwritten with weights in the reference's layout."""
        for m in self.modules():
            if getattr(m, "_layout_interleaved", False):
                m._layout_interleaved = False

    def quantize_weights(self) -> None:
        """After weights were loaded: build the FP8 copies of the linear weights and arrange gated fc1 weights for
        the fused fc1 + SwiGLU kernel."""
        for m in self.modules():
            if hasattr(m, "quantize_weights") and m is not self:
                m.quantize_weights()

    def release_checkpoint_weights(self) -> int:
        """Serve from the FP8 weight copies only: free the bf16 tensors of every FP8 linear (2 bytes per weight).
        Returns the number of layers released; loading or exporting a state dict is not possible afterwards."""
        return sum(1 for m in self.modules() if hasattr(m, "release_checkpoint_weight") and m.release_checkpoint_weight())

    def init_synthetic_weights(self, seed: int = 0, std: float = 0.02, device=None) -> None:
        """Seeded N(0, std) weights (norm scales 1 + N(0, std)), identical across TP sizes."""
        from ..synthetic import canonical_tensor

        tp, rank = parallel_state.get_tensor_model_parallel_world_size(), parallel_state.get_tensor_model_parallel_rank()
        own = self.state_dict()
        for k, shape in self.full_parameter_shapes().items():
            dev = own[k].device if device is None else device
            full = canonical_tensor(k, shape, seed=seed, std=std, dtype=self.config.params_dtype, device=dev)
            own[k].copy_(shard_for_rank(k, full, rank, tp, gated=self.config.gated_linear_unit))
            del full
        self._weights_are_canonical()
        self.quantize_weights()


@dataclass(frozen=True)
class ShardedTensorInfo:
    """What the reference's ``ShardedTensor`` records about one local tensor (``dist_checkpointing/mapping.py``; built by
    ``make_sharded_tensors_for_checkpoint`` from ``ColumnParallelLinear.sharded_state_dict`` / ``RowParallelLinear.
    sharded_state_dict``, ``megatron/core/tensor_parallel/layers.py:1045-1050, 1283-1288``): the checkpoint key, the
    local data, the shape of the whole tensor and where the local piece sits in it.  A gated fc1 is two pieces per rank
    - the rank's gate rows and its up rows - exactly as ``apply_swiglu_sharded_factory`` (``mlp.py:260-297``) writes it."""

    key: str
    data: torch.Tensor
    global_shape: tuple
    global_offset: tuple
    replica_id: int = 0


def merge_tensor_parallel_shards(shards, *, gated: bool) -> Dict[str, torch.Tensor]:
    """Inverse of `shard_for_rank`: the per-rank state dicts of a checkpoint written at tensor-parallel size
    ``len(shards)`` (rank order) -> unsharded tensors.  Replicated tensors are taken from rank 0."""
    tp = len(shards)
    out = {}
    for k, first in shards[0].items():
        if first is None or k.endswith("_extra_state"):
            continue
        dim = _partition_dim(k)
        if dim is None or tp == 1:
            out[k] = first
        elif gated and k.endswith(("linear_fc1.weight", "linear_fc1.bias")):
            halves = [torch.chunk(sd[k], 2, dim=0) for sd in shards]
            out[k] = torch.cat([h[0] for h in halves] + [h[1] for h in halves], dim=0)
        else:
            out[k] = torch.cat([sd[k] for sd in shards], dim=dim)
    return out


def _partition_dim(key: str) -> Optional[int]:
    """Dimension along which tensor parallelism splits the tensor behind ``key`` (None: replicated)."""
    if key.endswith(("linear_qkv.weight", "linear_qkv.bias", "linear_fc1.weight", "linear_fc1.bias",
                     "output_layer.weight", "word_embeddings.weight")):
        return 0
    if key.endswith(("linear_proj.weight", "linear_fc2.weight")):
        return 1
    return None


def shard_for_rank(key: str, full: torch.Tensor, rank: int, tp: int, *, gated: bool) -> torch.Tensor:
    """This rank's shard of an unsharded tensor.

    QKV rows are grouped per KV group ``[q_0..q_{g-1}, k, v]`` (``attention.py:992-1021``), so the
    contiguous row split is a split by KV group.  For a gated MLP, fc1 holds ``[gate ; up]`` and rank r
    takes ``[gate_r ; up_r]``, the layout checkpoints use (``mlp.py:260-297``); a plain contiguous split
    would change the function with the TP size.  fc2 / out-proj split along the input dimension;
    embedding and LM head split contiguously along the vocabulary (``layers.py:223-228``).
    """
    dim = _partition_dim(key)
    if dim is None or tp == 1:
        return full
    if gated and key.endswith(("linear_fc1.weight", "linear_fc1.bias")):
        gate, up = torch.chunk(full, 2, dim=0)
        return torch.cat([torch.chunk(gate, tp, dim=0)[rank], torch.chunk(up, tp, dim=0)[rank]], dim=0)
    return torch.chunk(full, tp, dim=dim)[rank]
