"""Dynamic inference context: in-flight batching bookkeeping + the chunked (paged) KV pool.

Public surface and integer semantics follow the reference's ``DynamicInferenceContext``
(``megatron/core/inference/contexts/dynamic_context.py``): the same constructor arguments, the same
per-request / per-token state tensors under the same names, the same chunk ids in the same order
(bit-exact block tables and KV slots), the same overflow errors.

What is different is where the state lives.  The reference keeps every bookkeeping tensor on the GPU
and drives it with ~60 tiny kernels and several ``.item()`` syncs per step.  Here the request-level
state (``request_*``, the chunk stack) is authoritative on the HOST as CPU int32 tensors, updated
with a few vectorised numpy operations, and only what the kernels consume is mirrored to the device
with asynchronous copies from pinned staging buffers: the ``token_to_*`` arrays, ``kv_seq_lengths``,
the block table and, for prefill steps, per-token block-table rows and KV lengths.  One step costs
one device->host read (the sampled tokens) and a handful of host->device copies.
"""
from __future__ import annotations

import math
import warnings
from enum import Enum
from typing import List, Optional, Tuple

import numpy as np
import torch
from torch import Tensor

from ... import parallel_state
from .dynamic_chunk_allocator import ChunkAllocator


class ContextOverflowError(Exception):
    """A new request does not fit.  ``is_transient``: retrying later may work (reference :30-45)."""

    def __init__(self, request_id: Optional[int], message: Optional[str] = None, *, is_transient: bool = True):
        request_str = "--" if request_id is None else str(request_id)
        message = "" if message is None else f" | {message}"
        super().__init__(f"request {request_str}{message}")
        self.request_id = request_id
        self.is_transient = is_transient


class RequestOverflowError(ContextOverflowError):
    """Adding the request would exceed ``max_requests``."""


class TokenOverflowError(ContextOverflowError):
    """Adding the request would exceed ``max_tokens``."""


class MaxSequenceLengthOverflowError(ContextOverflowError):
    """Prompt + output would exceed ``max_sequence_length``; never transient."""

    def __init__(self, request_id, message: Optional[str] = None):
        super().__init__(request_id, message=message, is_transient=False)


class ChunkOverflowError(ContextOverflowError):
    """Not enough free KV chunks (outside the guaranteed reserve)."""


class ActiveRequestCountOverflowError(ContextOverflowError):
    """``initialize_attention_state`` asked to warm up more tokens than ``max_requests``."""

    def __init__(self, max_request_count, active_request_count):
        assert active_request_count > max_request_count
        super().__init__(
            None, "active_request_count (%d) > max_request_count (%d)." % (active_request_count, max_request_count)
        )


class WarmupEngineMode(Enum):
    DECODE = "decode"
    NON_DECODE = "non_decode"


class BaseInferenceContext:
    """Minimal base (reference ``base_context.py:6-43``)."""

    def __init__(self, materialize_only_last_token_logits: bool):
        self.materialize_only_last_token_logits = materialize_only_last_token_logits

    def is_static_batching(self) -> bool:
        raise NotImplementedError

    def is_dynamic_batching(self) -> bool:
        return not self.is_static_batching()

    def increment_sequence_len_offset(self, increment: int) -> None:
        pass

    def increment_batch_size_offset(self, increment: int) -> None:
        pass

    def reset_batch_size_offset(self) -> None:
        pass


class AttentionStateError(RuntimeError):
    """`DynamicInferenceContext.validate_attention_state` found an index the kernels must not be given."""


# rows of the token-level arena
_TOK_INPUT, _TOK_POS, _TOK_REQ, _TOK_CHUNK, _TOK_POS_IN_REQ, _TOK_LOCAL = range(6)
_LEN_Q, _LEN_KV, _LEN_ORDER, _LEN_CUQ, _LEN_CUKV = range(5)  # rows of the per-request length matrix


class DynamicInferenceContext(BaseInferenceContext):
    TOKEN_ROUNDER = 64
    REQUEST_ROUNDER = 4

    def __init__(
        self,
        *,
        params_dtype: torch.dtype,
        num_layers: int,
        kv_channels: int,
        num_attention_heads: int,
        max_sequence_length: int,
        buffer_size_gb: float,
        buffer_guaranteed_fraction: float,
        chunk_size_tokens: int = 256,
        buffer_overflow_factor: Optional[float] = None,
        max_requests_override: Optional[int] = None,
        max_tokens_override: Optional[int] = None,
        tensor_model_parallel_size: Optional[int] = None,
        cache_mla_latent: bool = False,
        kv_lora_rank: Optional[int] = None,
        qk_pos_emb_head_dim: Optional[int] = None,
        num_cuda_graphs: Optional[int] = None,
        materialize_only_last_token_logits: bool = True,
        use_cuda_graphs_for_non_decode_steps: bool = True,
        device: Optional[torch.device] = None,
        allocate_memory_buffer: bool = True,
        kv_cache_dtype: Optional[torch.dtype] = None,
        kv_fp8_single_term: bool = False,
        debug_validate: bool = False,
    ):
        """``num_attention_heads`` is the number of KV heads (query groups), as in the reference.

        ``device``: where the KV pool and the kernel-facing index arrays live (default: the current
        CUDA device; pass ``'cpu'`` to exercise the bookkeeping alone).  ``allocate_memory_buffer=False``
        skips the KV pool for such bookkeeping-only uses.  ``kv_cache_dtype=torch.float8_e4m3fn`` (an
        extension; the reference's pool is always ``params_dtype``) stores keys and values as E4M3 bytes with
        one fp32 scale per layer and KV head (``kv_scales [L, 2, heads]``, 1.0 until the caller sets them),
        halving the bytes the attention kernel streams.
        """
        super().__init__(materialize_only_last_token_logits=materialize_only_last_token_logits)
        # Debug mode: every `initialize_attention_state` checks on the host what the kernels are about to index with
        # (`validate_attention_state`): the stand-in for a memory checker on machines where none can be run.
        self.debug_validate = bool(debug_validate)
        if cache_mla_latent:
            raise NotImplementedError("multi-latent attention caches are outside this decode path")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.cache_mla_latent = False

        tp_size = (
            parallel_state.get_tensor_model_parallel_world_size()
            if tensor_model_parallel_size is None
            else tensor_model_parallel_size
        )
        self.tp_size = tp_size
        if num_attention_heads % tp_size != 0:
            raise ValueError(f"{num_attention_heads} KV heads are not divisible by tensor parallel size {tp_size}")
        heads_per_partition = num_attention_heads // tp_size
        self.num_kv_heads_per_partition = heads_per_partition
        self.kv_channels = kv_channels

        # Chunk geometry (reference :194-217, 285).
        self.chunk_size_tokens = chunk_size_tokens
        self.kv_cache_dtype = params_dtype if kv_cache_dtype is None else kv_cache_dtype
        self.kv_cache_fp8 = self.kv_cache_dtype == torch.float8_e4m3fn
        # E4M3 pool only: one E4M3 term for queries / probabilities in the attention kernel (1.6x faster, ~30 % more error)
        self.kv_fp8_single_term = bool(kv_fp8_single_term)
        if self.kv_cache_dtype not in (params_dtype, torch.float8_e4m3fn):
            raise ValueError("kv_cache_dtype must be params_dtype or torch.float8_e4m3fn")
        self.chunk_size_bytes = (
            self.kv_cache_dtype.itemsize * 2 * num_layers * chunk_size_tokens * heads_per_partition * kv_channels
        )
        buffer_size_bytes = int(buffer_size_gb * 1024**3)
        buffer_size_bytes -= buffer_size_bytes % self.chunk_size_bytes
        chunk_count_total = buffer_size_bytes // self.chunk_size_bytes

        # max_requests / max_tokens (reference :219-242).
        n_tokens = buffer_size_bytes / self.chunk_size_bytes * chunk_size_tokens
        n_requests = n_tokens / max_sequence_length
        self.max_requests = self.round_up_requests(int(n_requests), tp_size=tp_size)
        self.max_tokens = self.round_up_tokens(int(n_tokens), tp_size=tp_size)
        if buffer_overflow_factor is not None:
            self.max_requests = self.round_up_requests(int(self.max_requests * buffer_overflow_factor), tp_size=tp_size)
            self.max_tokens = self.round_up_tokens(int(self.max_tokens * buffer_overflow_factor / 50.0), tp_size=tp_size)
        if max_requests_override is not None:
            self.max_requests = self.round_up_requests(max_requests_override, tp_size=tp_size)
        if max_tokens_override is not None:
            self.max_tokens = self.round_up_tokens(max_tokens_override, tp_size=tp_size)
        self.max_requests = min(self.max_requests, self.max_tokens)

        self.params_dtype = params_dtype
        self.num_layers = num_layers
        self.max_sequence_length = max_sequence_length

        self.total_request_count = 0
        self.active_token_count = 0
        self.paused_request_count = 0
        self.padded_active_token_count = None
        self.padded_active_request_count = None
        self.paused_tokens = None

        # ---- request-level state: host, int32 (authoritative) ----
        R = self.max_requests
        self.request_ids = torch.full((R,), -1, dtype=torch.int32)
        self.request_query_lengths = torch.zeros((R,), dtype=torch.int32)
        self.request_output_lengths = torch.zeros((R,), dtype=torch.int32)
        self.request_kv_length_offsets = torch.zeros((R,), dtype=torch.int32)
        self.request_kv_chunk_counts = torch.zeros((R,), dtype=torch.int32)
        self.request_last_kv_chunk_id = torch.zeros((R,), dtype=torch.int32)
        self.request_last_kv_chunk_offset = torch.zeros((R,), dtype=torch.int32)
        self.max_kv_chunk_count = math.ceil(max_sequence_length / chunk_size_tokens)
        self.request_to_kv_chunk_ids = torch.full((R, self.max_kv_chunk_count), -1, dtype=torch.int32)

        # ---- token-level state: host staging (pinned) + device arrays the kernels read ----
        pin = self.device.type == "cuda"
        Tm = self.max_tokens
        self._h_tok = torch.zeros((6, Tm), dtype=torch.int64, pin_memory=pin)
        self._h_tok_np = self._h_tok.numpy()
        self._d_tok = torch.zeros((6, Tm), dtype=torch.int64, device=self.device)
        self.token_to_input_ids = self._d_tok[_TOK_INPUT]
        self.token_to_pos_ids = self._d_tok[_TOK_POS]
        self.token_to_request_idx = self._d_tok[_TOK_REQ]
        self.token_to_chunk_idx = self._d_tok[_TOK_CHUNK]
        self.token_to_position_in_request = self._d_tok[_TOK_POS_IN_REQ]
        self.token_to_local_position_within_kv_chunk = self._d_tok[_TOK_LOCAL]
        # Prefill steps run the decode kernel once per prompt token: row of the block table and
        # number of visible keys for every token.
        self._h_tok32 = torch.zeros((2, Tm), dtype=torch.int32, pin_memory=pin)
        self._h_tok32_np = self._h_tok32.numpy()
        self._d_tok32 = torch.zeros((2, Tm), dtype=torch.int32, device=self.device)
        self.token_to_block_table_row = self._d_tok32[0]
        self.token_kv_lengths = self._d_tok32[1]

        # ---- KV pool ----
        self.memory_buffer = None
        self.kv_scales = None
        if allocate_memory_buffer:
            shape = (2, num_layers, chunk_count_total, chunk_size_tokens, heads_per_partition, kv_channels)
            if self.kv_cache_fp8:
                if chunk_size_tokens % 128 != 0 or kv_channels != 128:
                    raise ValueError("the E4M3 KV pool needs chunk_size_tokens % 128 == 0 and kv_channels == 128")
                # raw E4M3 bytes; 0xB8 is -1.0, the fill value of the 16-bit pool.  The value half of the buffer is
                # read by the kernels as [chunk][head][dim][position] (see b200_fp8_value_position).
                self.memory_buffer = torch.full(shape, 0xB8, dtype=torch.uint8, device=self.device)
                self.kv_scales = torch.ones((num_layers, 2, heads_per_partition), dtype=torch.float32, device=self.device)
            else:
                self.memory_buffer = torch.full(shape, -1, dtype=params_dtype, device=self.device)

        # ---- CUDA-graph token counts (reference :319-356) ----
        self.cuda_graph_token_counts = None
        if num_cuda_graphs is not None:
            num_cuda_graphs = min(max(num_cuda_graphs, 1), self.max_requests)
            rounder = 8
            step = self.max_requests / num_cuda_graphs
            step = math.ceil(step / rounder) * rounder
            step = math.ceil(step / tp_size) * tp_size
            self.cuda_graph_step_size = step
            if num_cuda_graphs == 1:
                self.cuda_graph_token_counts = [self.max_requests]
            else:
                counts = list(range(step, self.max_requests, step))
                if not counts or counts[-1] != self.max_requests:
                    counts.append(self.max_requests)
                counts.reverse()
                self.cuda_graph_token_counts = counts
            self.cuda_graph_token_counts_set = set(self.cuda_graph_token_counts)
            self.max_cuda_graph_token_count = max(self.cuda_graph_token_counts)
        self.cuda_graph_request_counts = self.cuda_graph_token_counts
        self.non_decode_cuda_graphs = use_cuda_graphs_for_non_decode_steps and (num_cuda_graphs is not None)

        # ---- attention state with stable device addresses (reference :358-382) ----
        dev = self.device
        # [query lens | kv lens | attention row order | cu query | cu kv]: rows of ONE device matrix mirrored from one
        # pinned staging matrix, so that a step publishes them with a single 2-D copy
        self._d_len = torch.zeros((5, R + 1), dtype=torch.int32, device=dev)
        self._d_len[_LEN_ORDER, :R] = torch.arange(R, dtype=torch.int32, device=dev)
        self.query_seq_lengths_cudagraph_only = self._d_len[_LEN_Q, :R]
        self.kv_seq_lengths_cudagraph_only = self._d_len[_LEN_KV, :R]
        # rows processed by the attention kernel in this order (longest context first); decode steps only
        self.attention_row_order = self._d_len[_LEN_ORDER, :R]
        self.cu_query_seq_lengths_cudagraph_only = self._d_len[_LEN_CUQ]
        self.cu_kv_seq_lengths_cudagraph_only = self._d_len[_LEN_CUKV]
        self.request_to_kv_chunk_ids_cudagraph_only = torch.zeros((R, self.max_kv_chunk_count), dtype=torch.int32, device=dev)
        self._h_len = torch.zeros((5, R + 1), dtype=torch.int32, pin_memory=pin)
        self._h_len_np = self._h_len.numpy()
        self._h_bt = torch.zeros((R, self.max_kv_chunk_count), dtype=torch.int32, pin_memory=pin)
        self._h_bt_np = self._h_bt.numpy()
        # Work list of the prefill attention kernel: (block-table row, first token, token count, 0) per block of
        # `prefill_q_block` consecutive query tokens of one request; built every non-decode step once
        # `set_prefill_q_block` has been called (by the model wrapper, which knows the head grouping).
        self.prefill_q_block = 0
        self.prefill_units = None
        self.prefill_unit_count = 0
        self._copy_event = torch.cuda.Event() if pin else None
        self._copies_pending = False
        self.h2d_bytes = 0  # bytes mirrored host -> device so far (benchmark accounting)
        # The device copy of the block table is refreshed only when rows or the set of active requests changed.
        self._bt_version = 0
        self._bt_pushed = None

        # ---- guaranteed-request reserve (reference :384-401) ----
        gtd_chunk_count = min(int(buffer_guaranteed_fraction * chunk_count_total), chunk_count_total)
        self.gtd_request_count = max(1, gtd_chunk_count // self.max_kv_chunk_count)
        self.gtd_chunk_count = self.gtd_request_count * self.max_kv_chunk_count
        self.chunk_allocator = ChunkAllocator(chunk_count_total=chunk_count_total, gtd_chunk_count=self.gtd_chunk_count)
        self.dummy_chunk_idx = self.chunk_allocator.dummy_chunk_idx

        self.reset_attention_state()

    def set_prefill_q_block(self, q_block: int) -> None:
        """Tokens per prefill work unit (64 / query heads per KV head); 0 disables the work list."""
        self.prefill_q_block = int(q_block)
        if self.prefill_q_block > 0:
            n = -(-self.max_tokens // self.prefill_q_block) + self.max_requests + 1
            pin = self.device.type == "cuda"
            self._h_units = torch.zeros((n, 4), dtype=torch.int32, pin_memory=pin)
            self._h_units_np = self._h_units.numpy()
            self.prefill_units = torch.zeros((n, 4), dtype=torch.int32, device=self.device)
            self.prefill_unit_count = 0

    def _build_prefill_units(self, ql: np.ndarray, n_rows: int, padded: int, graphs: bool) -> None:
        """Split every request's query tokens into blocks of `prefill_q_block` (host side, vectorised)."""
        qb = self.prefill_q_block
        ql = ql.astype(np.int64)
        nb = -(-ql // qb)
        total = int(nb.sum())
        u = self._h_units_np
        # under a CUDA graph the launch size is fixed by the padded sizes; unused entries have 0 tokens
        bound = (-(-padded // qb) + n_rows) if graphs else max(total, 1)
        bound = min(max(bound, total), u.shape[0])
        if total:
            first = np.cumsum(nb) - nb
            within = np.arange(total, dtype=np.int64) - np.repeat(first, nb)
            tok0 = np.repeat(np.cumsum(ql) - ql, nb) + within * qb
            u[:total, 0] = np.repeat(np.arange(ql.shape[0], dtype=np.int64), nb)
            u[:total, 1] = tok0
            u[:total, 2] = np.minimum(qb, np.repeat(ql, nb) - within * qb)
            u[:total, 3] = 0
        u[total:bound] = 0
        self.prefill_units[:bound].copy_(self._h_units[:bound], non_blocking=True)
        self.prefill_unit_count = bound
        self.h2d_bytes += 16 * bound

    # ------------------------------------------------------------------ rounding helpers
    @classmethod
    def round_up_tokens(cls, value, tp_size=None):
        """Next multiple of ``TOKEN_ROUNDER`` that is divisible by the tensor-parallel size."""
        if tp_size is None:
            tp_size = parallel_state.get_tensor_model_parallel_world_size()
        rounder = math.ceil(cls.TOKEN_ROUNDER / tp_size) * tp_size
        return rounder * int(math.ceil(int(value) / rounder))

    @classmethod
    def round_up(cls, value):
        """Deprecated predecessor of `round_up_tokens` / `round_up_requests` (reference :458-466): multiples of
        ``ROUNDER`` (64 unless a subclass sets it), no tensor-parallel divisibility."""
        warnings.warn("`round_up` is deprecated in favor of `round_up_tokens` or `round_up_requests`")
        rounder = getattr(cls, "ROUNDER", 64)
        return rounder * int(math.ceil(int(value) / rounder))

    @classmethod
    def round_up_requests(cls, value, tp_size=None):
        """Next multiple of ``REQUEST_ROUNDER`` that is divisible by the tensor-parallel size."""
        if tp_size is None:
            tp_size = parallel_state.get_tensor_model_parallel_world_size()
        rounder = math.ceil(cls.REQUEST_ROUNDER / tp_size) * tp_size
        return rounder * int(math.ceil(int(value) / rounder))

    # ------------------------------------------------------------------ simple queries
    def is_static_batching(self) -> bool:
        return False

    def is_decode_only(self) -> bool:
        """Every active request contributes exactly one token (reference :472-479)."""
        return (self.total_request_count - self.paused_request_count) == self.active_token_count

    def has_unfinished_requests(self) -> bool:
        return self.total_request_count > 0

    def cu_query_lengths(self) -> Tuple[Optional[Tensor], int]:
        return self.cu_query_seq_lengths, self.max_seqlen_q

    def cu_kv_lengths(self) -> Tuple[Optional[Tensor], Tensor, int]:
        return (self.cu_kv_seq_lengths, self.kv_seq_lengths, self.max_seqlen_k)

    def get_active_sequence_lengths(self) -> Tensor:
        """Query + cached length of the active requests (host int32)."""
        p, t = self.paused_request_count, self.total_request_count
        return (self.request_kv_length_offsets + self.request_query_lengths)[p:t]

    def get_max_sequence_lengths(self) -> Tensor:
        return self.request_output_lengths[self.paused_request_count : self.total_request_count]

    def get_active_request_count(self) -> int:
        return int(torch.less(self.get_active_sequence_lengths(), self.get_max_sequence_lengths()).sum())

    # ------------------------------------------------------------------ KV pool access
    def key_value_cache(self, layer_number: int) -> Tuple[Tensor, Tensor, Tensor]:
        """(K pool, V pool, block table) of 1-based ``layer_number`` (reference :547-564)."""
        return (self.memory_buffer[0, layer_number - 1], self.memory_buffer[1, layer_number - 1], self.block_table)

    def append_key_value_cache(self, layer_number: int, key: Tensor, value: Tensor) -> None:
        raise NotImplementedError(
            "KV append is fused into the attention op (b200_paged_attention with fuse_rope_append, or "
            "b200_rope_append for prefill steps); see SelfAttention.forward"
        )

    def apply_rotary_emb_query(self, query, query_emb, config, cu_seqlens_q, cp_group, mscale=1.0):
        """Not a separate step here: the attention kernel rotates the query as it loads it (reference :566-600)."""
        raise NotImplementedError("RoPE is applied inside the fused attention op; see SelfAttention.forward")

    def apply_rotary_emb_key(self, key, key_emb, config, cp_group, mscale=1.0):
        """Not a separate step here: the append kernel rotates the key before it stores it (reference :602-631)."""
        raise NotImplementedError("RoPE is applied inside the fused attention op; see SelfAttention.forward")

    # ------------------------------------------------------------------ host -> device mirroring
    def _wait_copies(self) -> None:
        """The pinned staging buffers may be rewritten only after earlier copies have run."""
        if self._copies_pending and self._copy_event is not None:
            self._copy_event.synchronize()
        self._copies_pending = False

    def _mark_copies(self) -> None:
        if self._copy_event is not None:
            self._copy_event.record()
            self._copies_pending = True

    def _push_rows(self, dst: Tensor, src: Tensor, rows: int, lo: int, hi: int, first_row: int = 0) -> None:
        """dst[first_row : first_row + rows, lo:hi] = src[same] (pinned host -> device), one 2-D copy on a GPU."""
        if hi <= lo or rows <= 0:
            return
        d, s_ = dst[first_row : first_row + rows], src[first_row : first_row + rows]
        if dst.is_cuda:
            from ... import ops

            ops.copy_rows_h2d(d, s_, rows, lo, hi)
        else:
            d[:, lo:hi].copy_(s_[:, lo:hi])
        self.h2d_bytes += rows * (hi - lo) * src.element_size()
        self._mark_copies()

    def _push_token_rows(self, rows, lo: int, hi: int) -> None:
        rows = sorted(rows)
        start = 0
        while start < len(rows):  # runs of consecutive rows go out together
            end = start
            while end + 1 < len(rows) and rows[end + 1] == rows[end] + 1:
                end += 1
            self._push_rows(self._d_tok, self._h_tok, end - start + 1, lo, hi, first_row=rows[start])
            start = end + 1

    # ------------------------------------------------------------------ attention state
    def reset_attention_state(self) -> None:
        """Forget the per-step views (reference :633-645).  The device buffers are rewritten by
        the next `initialize_attention_state`, padding rows included, so they are not cleared here."""
        self.max_seqlen_q = None
        self.max_seqlen_k = None
        self.cu_query_seq_lengths = None
        self.cu_kv_seq_lengths = None
        self.kv_seq_lengths = None
        self.block_table = None

    def using_cuda_graph_this_step(self) -> bool:
        has = self.cuda_graph_token_counts is not None
        can = self.is_decode_only() or self.non_decode_cuda_graphs
        fits = has and (self.active_token_count <= self.max_cuda_graph_token_count)
        return has and can and fits

    def initialize_attention_state(
        self,
        *,
        num_warmup_tokens: Optional[int] = None,
        warmup_engine_mode: WarmupEngineMode = WarmupEngineMode.DECODE,
        num_warmup_requests: Optional[int] = None,
    ) -> None:
        """Pad the step and publish lengths / block table to the device (reference :656-825)."""
        if num_warmup_requests is not None:
            warnings.warn("'num_warmup_requests' is deprecated, use 'num_warmup_tokens'", DeprecationWarning)
            if num_warmup_tokens is None:
                num_warmup_tokens = num_warmup_requests
        if num_warmup_tokens is not None:
            if num_warmup_tokens > self.max_requests:
                raise ActiveRequestCountOverflowError(self.max_requests, num_warmup_tokens)
            if warmup_engine_mode == WarmupEngineMode.NON_DECODE:
                assert self.non_decode_cuda_graphs, "Set non-decode cuda graphs to True"
                self.total_request_count = 1  # makes is_decode_only() False for the warm-up
        active_token_count = self.active_token_count if num_warmup_tokens is None else num_warmup_tokens

        graphs = self.using_cuda_graph_this_step()
        decode = self.is_decode_only()
        if graphs:
            padded = math.ceil(active_token_count / self.cuda_graph_step_size) * self.cuda_graph_step_size
            padded = min(padded, self.max_requests)
            assert padded in self.cuda_graph_token_counts_set and padded >= active_token_count
        else:
            padded = self.round_up_tokens(self.active_token_count, tp_size=self.tp_size)
            if decode:
                padded = min(padded, self.max_requests)
        self.padded_active_token_count = padded
        p, t = self.paused_request_count, self.total_request_count
        n_req = t - p
        self.padded_active_request_count = padded if (graphs or decode) else n_req

        self._wait_copies()
        a = self.active_token_count
        tok = self._h_tok_np
        if padded > a:  # padding tokens write to the dummy chunk, slot 0
            tok[_TOK_CHUNK, a:padded] = self.dummy_chunk_idx
            tok[_TOK_LOCAL, a:padded] = 0
            tok[_TOK_POS_IN_REQ, a:padded] = 0
            self._push_token_rows((_TOK_CHUNK, _TOK_LOCAL, _TOK_POS_IN_REQ), a, padded)

        ql = self.request_query_lengths.numpy()[p:t]
        kv = (self.request_kv_length_offsets.numpy() + self.request_query_lengths.numpy())[p:t]
        n_rows = self.padded_active_request_count
        lens = self._h_len_np
        lens[:, : n_rows + 1] = 0
        lens[_LEN_Q, :n_req] = ql
        lens[_LEN_KV, :n_req] = kv
        dev_rows = max(n_rows, 1)
        if decode:
            self.cu_query_seq_lengths = None
            self.cu_kv_seq_lengths = None
            self.max_seqlen_q = 1
            self.max_seqlen_k = self.max_sequence_length
        else:
            lens[_LEN_CUQ, 1 : n_req + 1] = np.cumsum(ql)
            lens[_LEN_CUKV, 1 : n_req + 1] = np.cumsum(kv)
            if n_rows > n_req:
                lens[_LEN_CUQ, n_req + 1 : n_rows + 1] = lens[_LEN_CUQ, n_req]
                lens[_LEN_CUKV, n_req + 1 : n_rows + 1] = lens[_LEN_CUKV, n_req]
            self.cu_query_seq_lengths = self.cu_query_seq_lengths_cudagraph_only[: n_rows + 1]
            self.cu_kv_seq_lengths = self.cu_kv_seq_lengths_cudagraph_only[: n_rows + 1]
            if graphs:
                self.max_seqlen_q = padded
                self.max_seqlen_k = self.max_sequence_length
            else:
                self.max_seqlen_q = int(ql.max()) if n_req else 0
                self.max_seqlen_k = int(kv.max()) if n_req else 0
            # per-token rows / visible key counts for the token-as-row prefill attention
            t32 = self._h_tok32_np
            t32[0, :a] = tok[_TOK_REQ, :a] - p
            t32[1, :a] = tok[_TOK_POS_IN_REQ, :a] + 1
            if padded > a:
                t32[0, a:padded] = 0
                t32[1, a:padded] = 0
            self._push_rows(self._d_tok32, self._h_tok32, 2, 0, padded)
            if self.prefill_q_block > 0:
                self._build_prefill_units(ql, n_rows, padded, graphs)
        if decode:
            # One CTA per (row, KV head) runs for a time proportional to the row's context: starting the long rows
            # first keeps the SMs evenly loaded to the end of the kernel.  Padding rows (length 0) come last.
            lens[_LEN_ORDER, :dev_rows] = np.argsort(-lens[_LEN_KV, :dev_rows], kind="stable")
            self._push_rows(self._d_len, self._h_len, 3, 0, dev_rows)           # query lens, kv lens, row order
        else:
            lens[_LEN_ORDER, : n_rows + 1] = np.arange(n_rows + 1)
            self._push_rows(self._d_len, self._h_len, 5, 0, n_rows + 1)         # ... and the cumulative lengths
        self.kv_seq_lengths = self.kv_seq_lengths_cudagraph_only[:n_rows]

        state = (self._bt_version, p, t, n_rows)
        if state != self._bt_pushed or num_warmup_tokens is not None:  # unchanged since the last step: already there
            bt = self._h_bt_np
            bt[:n_req] = self.request_to_kv_chunk_ids.numpy()[p:t]
            if n_rows > n_req:
                bt[n_req:n_rows] = 0
            self.request_to_kv_chunk_ids_cudagraph_only[:dev_rows].copy_(self._h_bt[:dev_rows], non_blocking=True)
            self.h2d_bytes += dev_rows * 4 * self.max_kv_chunk_count
            self._bt_pushed = None if num_warmup_tokens is not None else state
            self._mark_copies()
        self.block_table = self.request_to_kv_chunk_ids_cudagraph_only[:n_rows]
        if self.debug_validate:
            self.validate_attention_state()

    def validate_attention_state(self) -> None:
        """Host-side check of every index array the attention kernels consume for the step just published (the
        staging copies are what the device receives).  Raises `AttentionStateError` naming the first violation:
        block-table ids outside ``[0, chunk_count_total)`` in a column a row's length reaches, a length that exceeds
        the row's chunks, a row order that is not a permutation, a token slot outside its chunk or the pool."""
        n_rows = self.padded_active_request_count
        padded = self.padded_active_token_count
        p, t = self.paused_request_count, self.total_request_count
        n_req = t - p
        total = self.chunk_allocator.chunk_count_total
        chunk = self.chunk_size_tokens
        lens = self._h_len_np
        bt = self._h_bt_np
        kv = lens[_LEN_KV, :n_rows].astype(np.int64)
        if (kv < 0).any() or (kv > self.max_sequence_length).any():
            raise AttentionStateError(f"kv_seq_lengths outside [0, {self.max_sequence_length}]: {kv[(kv < 0) | (kv > self.max_sequence_length)][:4]}")
        if (kv[n_req:] != 0).any():
            raise AttentionStateError("a padding row has a non-zero length")
        need = -(-kv // chunk)
        if (need > self.max_kv_chunk_count).any():
            raise AttentionStateError("a length needs more chunks than a block-table row holds")
        cols = np.arange(self.max_kv_chunk_count)[None, :]
        used = cols < need[:, None]
        ids = bt[:n_rows]
        bad = used & ((ids < 0) | (ids >= total))
        if bad.any():
            r, c = np.argwhere(bad)[0]
            raise AttentionStateError(f"block table row {r} column {c} holds chunk id {ids[r, c]} (pool has {total}) inside its length {kv[r]}")
        if self.is_decode_only():
            rows = max(n_rows, 1)
            order = np.sort(lens[_LEN_ORDER, :rows])
            if not np.array_equal(order, np.arange(rows)):
                raise AttentionStateError("attention_row_order is not a permutation of the rows")
        tok = self._h_tok_np
        ci, lp = tok[_TOK_CHUNK, :padded], tok[_TOK_LOCAL, :padded]
        if ((ci < 0) | (ci >= total)).any() or ((lp < 0) | (lp >= chunk)).any():
            raise AttentionStateError("a token's KV slot (chunk id, position in chunk) lies outside the pool")
        a = self.active_token_count
        if (ci[a:] != self.dummy_chunk_idx).any():
            raise AttentionStateError("a padding token does not point at the dummy chunk")
        if (ci[:a] == self.dummy_chunk_idx).any():
            raise AttentionStateError("an active token points at the dummy chunk")

    def reset(self) -> None:
        """Drop every request and return all chunks (reference :827-869)."""
        self._wait_copies()
        self.total_request_count = 0
        self.active_token_count = 0
        self.paused_request_count = 0
        self.padded_active_token_count = 0
        self.padded_active_request_count = 0
        self.paused_tokens = None
        self.request_ids.fill_(-1)
        self.request_query_lengths.fill_(0)
        self.request_output_lengths.fill_(0)
        self.request_kv_length_offsets.fill_(0)
        self.request_kv_chunk_counts.fill_(0)
        self.request_last_kv_chunk_id.fill_(-1)
        self.request_last_kv_chunk_offset.fill_(0)
        self.request_to_kv_chunk_ids.fill_(-1)
        self._h_tok.fill_(0)
        self._h_tok[_TOK_REQ].fill_(-1)
        self._h_tok[_TOK_CHUNK].fill_(-1)
        self._d_tok.copy_(self._h_tok, non_blocking=True)
        self._mark_copies()
        self.reset_attention_state()
        self.chunk_allocator.reset()
        self._bt_version += 1

    def current_input_and_position_ids(self, *, num_warmup_tokens: Optional[int] = None) -> Tuple[Tensor, Tensor]:
        """Flattened ``[1, T]`` input and position ids of the padded step (device views)."""
        n = num_warmup_tokens or self.padded_active_token_count
        return (self.token_to_input_ids[:n].unsqueeze(0), self.token_to_pos_ids[:n].unsqueeze(0))

    def last_token_indices(self) -> np.ndarray:
        """Index of the last token of every active request in the flattened step (host)."""
        p, t = self.paused_request_count, self.total_request_count
        return np.cumsum(self.request_query_lengths.numpy()[p:t], dtype=np.int64) - 1

    def last_token_logits(self, logits: Tensor) -> Tensor:
        """Rows of ``logits [1, T, V]`` that belong to each request's last token (reference :890-918)."""
        assert logits.size(0) == 1
        assert logits.size(1) == self.padded_active_token_count, (
            f"logits.size(1) ({tuple(logits.shape)}) != padded_active_token_count ({self.padded_active_token_count})."
        )
        idx = torch.from_numpy(self.last_token_indices()).to(logits.device)
        return logits.squeeze(0)[idx, :]

    # ------------------------------------------------------------------ admission
    def add_request(self, request_id: int, tokens, num_tokens_to_generate: Optional[int] = None) -> None:
        """Admit a request: pop ``ceil(len / chunk)`` chunks, fill its row and its token entries
        (reference :920-1015).  Unlike the reference, the sequence-length check runs before chunks
        are popped, so a rejected request does not leak chunks."""
        if isinstance(tokens, Tensor):
            context_length = tokens.numel()
        else:
            tokens = np.asarray(tokens, dtype=np.int64)
            context_length = int(tokens.size)
        if context_length > self.max_tokens:
            raise TokenOverflowError(request_id, is_transient=True)
        if self.active_token_count + context_length > self.max_tokens:
            raise TokenOverflowError(request_id)
        if self.total_request_count >= self.max_requests:
            raise RequestOverflowError(request_id)
        if num_tokens_to_generate is not None and context_length + num_tokens_to_generate > self.max_sequence_length:
            raise MaxSequenceLengthOverflowError(request_id)
        num_chunks_needed = math.ceil(context_length / self.chunk_size_tokens)
        new_chunk_ids = self.chunk_allocator.allocate_memory_chunks(num_chunks_needed, safe=True)
        if new_chunk_ids is None:
            raise ChunkOverflowError(request_id)
        if num_tokens_to_generate is None:
            num_tokens_to_generate = self.max_sequence_length - context_length
        # Admission succeeded: only now does the state change.  (A request that is rejected - e.g. one that waits in
        # the engine's queue and is retried after every step - must leave the version alone, or every step would
        # invalidate the block table on the device and the forward the controller enqueued early.)
        self._bt_version += 1

        r = self.total_request_count
        self.request_ids[r] = request_id
        self.request_query_lengths[r] = context_length
        self.request_output_lengths[r] = context_length + num_tokens_to_generate
        self.request_kv_length_offsets[r] = 0
        self.request_to_kv_chunk_ids[r, :num_chunks_needed] = new_chunk_ids
        self.request_kv_chunk_counts[r] = num_chunks_needed
        self.request_last_kv_chunk_id[r] = new_chunk_ids[-1]
        self.request_last_kv_chunk_offset[r] = (context_length - 1) % self.chunk_size_tokens

        self._wait_copies()
        a, b = self.active_token_count, self.active_token_count + context_length
        ar = np.arange(context_length, dtype=np.int64)
        tok = self._h_tok_np
        tok[_TOK_POS, a:b] = ar
        tok[_TOK_REQ, a:b] = r
        tok[_TOK_POS_IN_REQ, a:b] = ar
        tok[_TOK_CHUNK, a:b] = new_chunk_ids.numpy()[ar // self.chunk_size_tokens]
        tok[_TOK_LOCAL, a:b] = ar % self.chunk_size_tokens
        if isinstance(tokens, Tensor) and tokens.device.type != "cpu":
            # prompt already on the device: copy it there directly, keep the host mirror in sync lazily
            self._d_tok[_TOK_INPUT, a:b].copy_(tokens.reshape(-1), non_blocking=True)
            tok[_TOK_INPUT, a:b] = tokens.reshape(-1).cpu().numpy()
            self._push_token_rows((_TOK_POS, _TOK_REQ, _TOK_CHUNK, _TOK_POS_IN_REQ, _TOK_LOCAL), a, b)
        else:
            tok[_TOK_INPUT, a:b] = tokens.reshape(-1).numpy() if isinstance(tokens, Tensor) else tokens.reshape(-1)
            self._push_token_rows(range(6), a, b)
        self.total_request_count += 1
        self.active_token_count += context_length

    # ------------------------------------------------------------------ per-step update
    def _move_book_keeping_tensors(self, src_idxs, dst_idxs, next_tokens) -> None:
        """rows[dst] = rows[src] for every request-level array and the pending tokens (reference :1017-1030)."""
        for arr in (
            self.request_kv_length_offsets,
            self.request_query_lengths,
            self.request_output_lengths,
            self.request_ids,
            self.request_to_kv_chunk_ids,
            self.request_kv_chunk_counts,
            self.request_last_kv_chunk_id,
            self.request_last_kv_chunk_offset,
        ):
            a = arr.numpy()
            a[dst_idxs] = a[src_idxs]
        next_tokens[dst_idxs] = next_tokens[src_idxs]

    @property
    def state_version(self) -> int:
        """Changes whenever requests are admitted, finish, are paused / resumed, get a new chunk, or on reset."""
        return self._bt_version

    FAST_DECODE_UPDATE = True  # shortcut for the steady state of decoding (tests switch it off to compare)

    def update_requests(self, active_requests_mask, new_tokens) -> Optional[Tensor]:
        """Advance the context after a step (reference :1033-1298).

        ``active_requests_mask`` (1 = continues, 0 = finished) and ``new_tokens`` hold one entry per
        active request; tensors on any device, arrays or lists are accepted (device tensors cost one
        synchronising read).  Finished requests release their chunks (LIFO stack), rows are compacted
        to [paused | active], requests whose last chunk is full are paused and - chunks permitting -
        resumed at once with a freshly popped chunk, and the token arrays of the next step are
        written.  Returns the ids of requests newly paused in this call (host int32) or None.
        """
        mask = _to_host(active_requests_mask).astype(np.int64)
        new_tokens = _to_host(new_tokens).astype(np.int64)
        active_request_count = int(np.count_nonzero(mask == 1))
        finished_request_count = mask.size - active_request_count
        assert finished_request_count == int(np.count_nonzero(mask == 0)), "the mask holds 0 / 1 only"
        assert active_request_count + finished_request_count + self.paused_request_count == self.total_request_count
        self.reset_attention_state()
        P = self.paused_request_count
        if self.FAST_DECODE_UPDATE and finished_request_count == 0 and P == 0 and active_request_count > 0:
            n = active_request_count
            last_off = self.request_last_kv_chunk_offset.numpy()
            if not (last_off[:n] == self.chunk_size_tokens - 1).any():
                # Steady state of decoding - every request continues inside its current chunk: nothing moves, no
                # chunk is popped or pushed, the block table stays as it is.  (The general path below computes
                # exactly this in that case.)
                self.active_token_count = n
                offs = self.request_kv_length_offsets.numpy()
                qlen = self.request_query_lengths.numpy()
                offs[:n] += qlen[:n]
                qlen[:n] = 1
                last_off[:n] += 1
                self._wait_copies()
                tok = self._h_tok_np
                tok[_TOK_INPUT, :n] = new_tokens
                tok[_TOK_POS, :n] = offs[:n]
                tok[_TOK_REQ, :n] = np.arange(n)
                tok[_TOK_POS_IN_REQ, :n] = offs[:n]
                tok[_TOK_CHUNK, :n] = self.request_last_kv_chunk_id.numpy()[:n]
                tok[_TOK_LOCAL, :n] = last_off[:n]
                self._push_token_rows(range(6), 0, n)
                return None
        self._bt_version += 1
        chunk_ids = self.request_to_kv_chunk_ids.numpy()

        if active_request_count + P == 0:
            if finished_request_count > 0:
                rows = chunk_ids[np.nonzero(mask == 0)[0] + P]
                self.chunk_allocator.release_memory_chunks(rows[rows != -1])
            chunk_ids.fill(-1)
            self.total_request_count = 0
            self.active_token_count = 0
            return None

        next_tokens = new_tokens.copy() if P == 0 else np.concatenate([_to_host(self.paused_tokens).astype(np.int64), new_tokens])

        if finished_request_count > 0:
            finished_idxs = np.nonzero(mask == 0)[0] + P
            rows = chunk_ids[finished_idxs]
            self.chunk_allocator.release_memory_chunks(rows[rows != -1])
            chunk_ids[finished_idxs] = -1
            if active_request_count > 0:
                finished_on_left = np.nonzero(mask[:active_request_count] == 0)[0] + P
                active_on_right = np.nonzero(mask[active_request_count:])[0] + active_request_count + P
                self._move_book_keeping_tensors(active_on_right, finished_on_left, next_tokens)
                chunk_ids[active_on_right] = -1

        newly_paused_request_ids = None
        if active_request_count > 0:
            last = self.request_last_kv_chunk_offset.numpy()[P : P + active_request_count]
            needs_chunk = last == self.chunk_size_tokens - 1
            n_need = int(needs_chunk.sum())
            if 0 < n_need != active_request_count:
                active_on_left = np.nonzero(~needs_chunk[:n_need])[0] + P
                paused_on_right = np.nonzero(needs_chunk[n_need:])[0] + n_need + P
                dst = np.concatenate([active_on_left, paused_on_right])
                src = np.concatenate([paused_on_right, active_on_left])
                self._move_book_keeping_tensors(src, dst, next_tokens)
                newly_paused_request_ids = self.request_ids[torch.from_numpy(dst)].clone()
            self.paused_request_count += n_need
            active_request_count -= n_need

        non_gtd = max(0, self.chunk_allocator.chunk_count_avail - self.gtd_chunk_count)
        if non_gtd:
            resume = min(non_gtd, self.paused_request_count)
        else:
            resume = min(max(self.gtd_request_count - active_request_count, 0), self.paused_request_count)
        self.paused_request_count -= resume
        active_request_count += resume
        assert active_request_count > 0, "active_request_count == %d." % active_request_count
        if newly_paused_request_ids is not None and resume > 0:
            newly_paused_request_ids = newly_paused_request_ids[:-resume]

        self.total_request_count = active_request_count + self.paused_request_count
        self.active_token_count = active_request_count
        P, T = self.paused_request_count, self.total_request_count
        n = active_request_count
        if P > 0:
            self.paused_tokens = torch.from_numpy(next_tokens[:P].copy())
        offs = self.request_kv_length_offsets.numpy()
        qlen = self.request_query_lengths.numpy()
        offs[P:T] += qlen[P:T]
        qlen[P:T] = 1
        last_off = self.request_last_kv_chunk_offset.numpy()
        last_off[P:T] = (last_off[P:T] + 1) % self.chunk_size_tokens

        if resume > 0:
            assert np.all(last_off[P : P + resume] == 0), "resumed requests must start a fresh chunk"
            ids = self.chunk_allocator.allocate_memory_chunks(resume).numpy()
            counts = self.request_kv_chunk_counts.numpy()
            chunk_ids[np.arange(P, P + resume), counts[P : P + resume]] = ids
            counts[P : P + resume] += 1
            self.request_last_kv_chunk_id.numpy()[P : P + resume] = ids

        self._wait_copies()
        tok = self._h_tok_np
        tok[_TOK_INPUT, :n] = next_tokens[P:T]
        tok[_TOK_POS, :n] = offs[P:T]
        tok[_TOK_REQ, :n] = np.arange(P, T)
        tok[_TOK_POS_IN_REQ, :n] = offs[P:T]
        tok[_TOK_CHUNK, :n] = self.request_last_kv_chunk_id.numpy()[P:T]
        tok[_TOK_LOCAL, :n] = last_off[P:T]
        self._push_token_rows(range(6), 0, n)
        return newly_paused_request_ids

    # ------------------------------------------------------------------ log-probs (optional path)
    def calculate_log_probs(self, logits: Tensor, new_tokens: Tensor, only_last_token_logits: Optional[bool] = False) -> List[List[float]]:
        """Log-probability of the chosen token(s) per active request (reference :1300-1365)."""
        log_probs = torch.log_softmax(logits.squeeze(0).float(), dim=-1)
        new_tokens = torch.as_tensor(new_tokens, device=log_probs.device)
        if only_last_token_logits or self.is_decode_only():
            idx = torch.arange(len(new_tokens), device=log_probs.device)
            return [[lp] for lp in log_probs[idx, new_tokens].flatten().tolist()]
        p, t = self.paused_request_count, self.total_request_count
        active_token_ids = self.token_to_input_ids[: self.active_token_count].roll(-1, 0).to(log_probs.device)
        qlens = self.request_query_lengths[p:t]
        new_token_idx = (qlens.cumsum(0) - 1).long().to(log_probs.device)
        active_token_ids[new_token_idx] = new_tokens
        idx = torch.arange(self.active_token_count, device=log_probs.device)
        selected = log_probs[idx, active_token_ids].cpu().split(qlens.tolist(), dim=0)
        return [lp.tolist() for lp in selected]


def _to_host(x) -> np.ndarray:
    if isinstance(x, Tensor):
        return x.detach().cpu().numpy().reshape(-1)
    return np.asarray(x).reshape(-1)
